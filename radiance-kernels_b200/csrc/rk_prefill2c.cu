// MX flash-attention prefill, two 128-row query tiles per CTA (head dim <= 128), one thread per query row and
// separate correction warps.
//
// Stages as in fa_entry, kernels/flash_attention_mx_gqa/kernel.cpp:91-184 (QK_j -> fused softmax + requant ->
// scale pack -> PV_j -> rescale/accumulate -> finalize); what this file decides is who does what:
//
//   warps 0-3    softmax of query tile A: thread = row (the one-lane-per-row form of fused_softmax_requant_tpr,
//   warps 4-7    softmax of query tile B   kernels/flash_attention_mx_gqa/flash_mx_impl.hpp:314-394): a row's 128
//                scores of a key tile sit in the thread's registers, so row max and row sum need no exchange
//   warps 8-11   correction: rescale_accumulate (flash_mx_impl.hpp:508-532) on the O accumulators in TMEM, off the
//                softmax warps' critical path; warp 8+q serves TMEM lane quadrant q of both tiles
//   warp  12     TMA producer (one elected lane)
//   warp  13     issuer of the S = Q K^T MMAs (one elected lane) + TMEM allocation
//   warp  14     issuer of the O += P V MMAs (one elected lane): two issuers, so that a P V waiting for its P tile
//                never holds back the next Q K^T
//   warp  15     fills the fourth warpgroup (register reallocation works on whole warpgroups)
//
// Registers are moved between the warpgroups with setmaxnreg: the softmax threads hold a whole 128-score row
// (kRegSoftmax), correction, TMA and MMA threads need few.  The S accumulator (128 TMEM columns) is shared by the
// two tiles: a softmax group copies its rows to registers at once and hands the columns back, the Q K^T issuer
// alternates QK_A, QK_B.  Every K/V tile brought in by TMA serves both query tiles.
#include <type_traits>

#include "rk_prefill.cuh"

namespace rk {

namespace c2 {
constexpr int kStages = 3;
constexpr int kThreads = 512;
#ifndef RK_SLEEP_NS
#define RK_SLEEP_NS 100
#endif
constexpr uint32_t kSleepNs = RK_SLEEP_NS;     // back-off of the warps that wait off the critical path
constexpr int kWarpCorr = 8, kWarpTma = 12, kWarpQk = 13, kWarpPv = 14;
// 128 * (2*176 + 96 + 64) = 65536 registers.  Measured: the softmax warps are 2 % faster with 176 registers than with 184
// or 168 (no spills in any of them; what changes is the order ptxas gives the tile body).
constexpr uint32_t kRegSoftmax = 176, kRegCorr = 96, kRegIssue = 64;
// TMEM columns
constexpr uint32_t cS = 0, cO = 128 /* + g*128 */, cSfQ = 384 /* + g*4 */, cSfK = 392 /* + st*4 */,
                   cSfP = 404 /* + (g*2+pb)*4 */, cSfV = 420 /* + st*4 */;
// shared memory
constexpr int q_off = 0;                                   // [2][16 KB]
constexpr int k_off = q_off + 2 * kTileBytes;              // [3]
constexpr int v_off = k_off + kStages * kTileBytes;        // [3]
constexpr int p_off = v_off + kStages * kTileBytes;        // [2 groups][2]
constexpr int sfq_off = p_off + 4 * kTileBytes;            // [2]
constexpr int sfk_off = sfq_off + 2 * kSfAtomBytes;        // [3]
constexpr int sfv_off = sfk_off + kStages * kSfAtomBytes;  // [3]
constexpr int sfp_off = sfv_off + kStages * kSfAtomBytes;  // [2][2]
constexpr int bar_off = sfp_off + 4 * kSfAtomBytes;
// barrier indices
constexpr int bQ = 0, bKF = 1, bKE = 4, bVF = 7, bVE = 10, bSF = 13 /* +g */, bSE = 15 /* +g */,
              bPF = 17 /* + g*2+pb */, bPV = 21 /* + g*2+pb */, bCF = 25 /* + (g*4+slot)*4+quad */, bOR = 57 /* + g*2+pb */,
              bDRAIN = 61, bDRAIN2 = 62, nBars = 63;
constexpr int misc_off = bar_off + nBars * 8;
constexpr int corr_off = misc_off + 16;                    // [2 groups][4 slots][128] floats: the O rescale factors of a tile
constexpr int total = corr_off + 2 * 4 * 128 * 4;
// test hook: which role sleeps a little at every key tile (schedule perturbation)
constexpr int kPerturbSoftmaxA = 1 /* 2 = softmax of tile B */, kPerturbCorr = 3, kPerturbTma = 4, kPerturbQk = 5, kPerturbPv = 6;
}  // namespace c2

template <uint32_t N> RK_DEVINL void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N> RK_DEVINL void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

RK_DEVINL void perturb(const PrefillParams& p, int role, int j) {
  if (__builtin_expect(p.perturb == role, 0)) __nanosleep(400 + 97 * (j & 7));
}

// ---- softmax warps: thread = query row -----------------------------------------------------------------------
// The body of a key tile exists twice: PLAIN for tiles no row of which needs a mask (every tile below the causal
// diagonal), and the general one with the mask code; the stage dump (tests) only in the DUMP instantiation of the
// kernel.  The loop over plain tiles is what runs nearly all the time, and it is kept small and contiguous: this
// kernel's softmax warps stall on instruction fetch, and code that sits inside the loop costs time even when it
// is jumped over.
// The blocking form of the two waits a key tile starts with (its S, and the P buffer it will write): out of line, so
// that the tile body carries only the test of two flags.  Returns 0, or the code of the wait that gave up.
__device__ __forceinline__ int wait_tile_inputs(uint64_t* s_full, uint32_t s_parity, uint64_t* pv_done, uint32_t pv_parity,
                                             int need_pv, volatile int* abort_flag) {
  if (!mbar_wait_lean(s_full, s_parity, abort_flag)) return 101;
  if (need_pv && !mbar_wait_lean(pv_done, pv_parity, abort_flag)) return 102;
  return 0;
}

template <bool SOFTCAP, bool DUMP>
__device__ __forceinline__ void softmax_row_group(const PrefillParams& p, uint8_t* smem, uint64_t* bars, uint32_t tmem_base,
                                                  volatile int* abort_flag, int grp, int qt, int bh, int n_tiles, int j0) {
  using namespace c2;
  uint64_t* s_full = bars + bSF + grp;
  uint64_t* s_empty = bars + bSE + grp;
  uint64_t* p_full = bars + bPF + grp * 2;
  uint64_t* pv_done = bars + bPV + grp * 2;
  uint64_t* corr_full = bars + bCF + grp * 16;
  float* corr_sm = reinterpret_cast<float*>(smem + corr_off) + grp * 512;

  const int lane = threadIdx.x & 31;
  const int quad = (threadIdx.x >> 5) & 3;
  const int row = quad * 32 + lane;
  const uint32_t lane_addr = ((uint32_t)(quad * 32)) << 16;
  const int q_row = qt * kBlockM + row;
  const int q_pos = p.q_pos0 + q_row;
  const float NEG_INF = __int_as_float(0xff800000);
  const bool dump = DUMP && p.dbg && qt == p.n_q_tiles - 1 && bh == 0;
  const float sc_mul = SOFTCAP ? 1.0f : p.scale_log2;

  float m_run = NEG_INF, l_run = 0.0f;
  bool ok = true;
  bool s_ready = false;       // results of early, non-blocking tests of the next tile's S barrier and P buffer
  int fail = 0;               // which wait gave up (reported after the loops: the tile body carries no reporting code)

  auto tile = [&](const int j, auto plain_tag) -> bool {
    constexpr bool PLAIN = decltype(plain_tag)::value;
    const int pb = j & 1;
    perturb(p, kPerturbSoftmaxA + grp, j);
    const bool stamp = (quad == 0 && lane == 0);
    if (stamp) RK_STAMP(grp, j, 0);
    if (__builtin_expect(!__all_sync(0xffffffffu, s_ready), 0)) {   // a test issued during the previous tile said "not yet"
      const int w = wait_tile_inputs(s_full, j & 1, &pv_done[pb], ((j - 2) >> 1) & 1, j >= 2, abort_flag);
      if (__any_sync(0xffffffffu, w != 0)) { fail = w ? w : 101; return false; }
    }
    tc_fence_after();
    if (stamp) RK_STAMP(grp, j, 1);

    float s[128];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld32(tmem_base + lane_addr + cS + c * 32, reinterpret_cast<uint32_t*>(s) + c * 32);
    tc_wait_ld();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(s_empty);       // hand the S columns back: the other query tile's QK^T may use them
    if (stamp) RK_STAMP(grp, j, 2);

    if (DUMP && dump && j == 0) {
#pragma unroll
      for (int c = 0; c < 128; ++c) p.dbg[row * 128 + c] = s[c];
    }

    // ---- (soft-cap,) mask, block maxima ----------------------------------------------------------------
    const int key0 = (j + j0) * kBlockN;                      // first key of this tile (j counts from the first tile inside the window)
    const bool tail = (key0 + kBlockN > p.S_kv);
    const bool diag = p.causal && (key0 + kBlockN - 1 > p.q_pos0 + qt * kBlockM);
    const bool need_mask = !PLAIN && (tail || diag || (p.window > 0));
    if (SOFTCAP) softcap_scores(s, p.scale_log2, p.cap_log2, p.inv_cap_scale);   // cap * tanh(s * scale / cap), pre-multiplied by log2 e
    if (__builtin_expect(need_mask, 0)) {
      int hi = p.S_kv - 1 - key0;                             // masked iff c > hi || c <= lo
      if (p.causal) hi = min(hi, q_pos - key0);
      const int lo = (p.window > 0) ? (q_pos - p.window - key0) : -1;
#pragma unroll
      for (int c = 0; c < 128; ++c) s[c] = (c > hi || c <= lo) ? NEG_INF : s[c];
    }
    // block maxima: eight independent chains (two per 32-key block), advanced in turn so that no instruction waits
    // for the one before it
    float bmax[4];
    {
      float a0[4], a1[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        a0[g] = fmax3(s[g * 32 + 0], s[g * 32 + 1], s[g * 32 + 2]);
        a1[g] = fmax3(s[g * 32 + 3], s[g * 32 + 4], s[g * 32 + 5]);
      }
#pragma unroll
      for (int c = 6; c < 30; c += 4) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          a0[g] = fmax3(a0[g], s[g * 32 + c], s[g * 32 + c + 1]);
          a1[g] = fmax3(a1[g], s[g * 32 + c + 2], s[g * 32 + c + 3]);
        }
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) bmax[g] = fmax3(a0[g], a1[g], fmaxf(s[g * 32 + 30], s[g * 32 + 31]));
    }
    const float mx = fmaxf(fmax3(bmax[0], bmax[1], bmax[2]), bmax[3]);
    // The running maximum follows every tile (rescale_accumulate, flash_mx_impl.hpp:508-532).  Letting it lag
    // while the maximum grows little would save most O rescales, but p would then differ from the reference's by a
    // factor that is no power of two, its truncated E4M3 codes with it, and O by the size of the truncation noise.
    const float m_new = fmaxf(m_run, mx * sc_mul);
    // exponent = fma(s, scale, -m): lowering m by 2^-21 |m| keeps the row-max p in [1, 1 + 1e-5) in spite of
    // the rounding residue of s*scale; the common factor cancels in O = sum(p v) / sum(p).
    const float m_use = (m_new == NEG_INF) ? 0.0f : (SOFTCAP ? m_new : fmaf(-fabsf(m_new), 4.76837158203125e-7f, m_new));
    const float corr = (m_run == NEG_INF) ? 1.0f : ex2_approx(m_run - m_new);
    m_run = m_new;
    // The correction warp of this lane quadrant can start on O while the exponentials run here.  Slot j & 3: this
    // group is never more than two tiles ahead of the correction warp (the wait for the P buffer at the top of the
    // tile sees to that), so a slot is free again long before it comes round.
    corr_sm[(j & 3) * 128 + row] = corr;
    __syncwarp();
    if (lane == 0) mbar_arrive(&corr_full[(j & 3) * 4 + quad]);
    if (stamp) RK_STAMP(grp, j, 3);

    // ---- p = 2^(x - m), row sum from the unquantised p, requant per 32-key block ---------------------
    // ex2.approx.ftz never returns a subnormal, so every non-zero p has an exponent field >= 1 and one multiply by
    // 2^(7-sc) puts the E4M3 code into bits [20,27) whatever the block scale code sc is (sc < 7 needs no other
    // path: all its non-zero elements lie within 2^6 of the block maximum).
    uint8_t* p_tile = smem + p_off + (grp * 2 + pb) * kTileBytes + row * 128;
    uint64_t lsA = 0ull, lsB = 0ull;                                  // two packed pairs of partial row sums
    uint32_t scale_word = 0;
    uint64_t fmul2[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const float pmax = ex2_approx(fmaf(bmax[g], sc_mul, -m_use));   // p of the block's arg-max element
      int sc = (int)(__float_as_uint(pmax) >> 23);                    // E8M0 code: se = floor(log2 pmax) <= 0
      sc = min(sc, 127);
      scale_word |= (uint32_t)sc << (8 * g);
      const float f = __uint_as_float((uint32_t)(134 - sc) << 23);   // 2^(7-sc)
      fmul2[g] = pack2(f, f);
    }
    const uint64_t sc2 = pack2(sc_mul, sc_mul), nm2 = pack2(-m_use, -m_use);
    // Four elements at a time: exponentials of block g+1 (special-function unit) next to the requantization of block
    // g (integer and FMA pipes), in one instruction stream, so that the units work side by side.
    auto exp4 = [&](int g, int c) {
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        float x0, x1;
        unpack2(fma2p(pack2(s[g * 32 + c + e], s[g * 32 + c + e + 1]), sc2, nm2), x0, x1);
        s[g * 32 + c + e] = ex2_approx(x0);
        s[g * 32 + c + e + 1] = ex2_approx(x1);
      }
    };
    // y = p * 2^(7-sc): exponent field = E4M3 exponent field, mantissa kept, so the truncated code is
    // y's bits [20,27); .ftz zeroes everything below 2^-6 of the block scale.
    auto requant4 = [&](int g, int c) -> uint32_t {
      const uint64_t p01 = pack2(s[g * 32 + c + 0], s[g * 32 + c + 1]);
      const uint64_t p23 = pack2(s[g * 32 + c + 2], s[g * 32 + c + 3]);
      lsA = add2p(lsA, p01);
      lsB = add2p(lsB, p23);
      uint32_t y0, y1, y2, y3;
      unpack2u(mul2p_ftz(p01, fmul2[g]), y0, y1);
      unpack2u(mul2p_ftz(p23, fmul2[g]), y2, y3);
      return pack_u8x2(y1 >> 20, y0 >> 20, pack_u8x2(y3 >> 20, y2 >> 20, 0u));
    };
#pragma unroll
    for (int c = 0; c < 32; c += 4) exp4(0, c);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (g < 3) exp4(g + 1, q * 4);
        w[q] = requant4(g, q * 4);
      }
      const int c0 = (2 * g) ^ (row & 7), c1 = (2 * g + 1) ^ (row & 7);     // 128-byte swizzle
      *reinterpret_cast<uint4*>(p_tile + c0 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(p_tile + c1 * 16) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    float ls0, ls1, ls2, ls3;
    unpack2(lsA, ls0, ls1);
    unpack2(lsB, ls2, ls3);
    l_run = l_run * corr + ((ls0 + ls1) + (ls2 + ls3));
    // the row's four block scales: bytes (row%32)*16 + (row/32)*4 + 0..3 of the 512-byte scale atom
    *reinterpret_cast<uint32_t*>(smem + sfp_off + (grp * 2 + pb) * kSfAtomBytes + (row & 31) * 16 + (row >> 5) * 4) = scale_word;

    if (DUMP && dump && j == 0) {
      uint32_t* d32 = reinterpret_cast<uint32_t*>(p.dbg + 128 * 128);
#pragma unroll
      for (int lc = 0; lc < 8; ++lc) {
        const uint4 v4 = *reinterpret_cast<const uint4*>(p_tile + ((lc ^ (row & 7)) * 16));
        d32[row * 32 + lc * 4 + 0] = v4.x; d32[row * 32 + lc * 4 + 1] = v4.y;
        d32[row * 32 + lc * 4 + 2] = v4.z; d32[row * 32 + lc * 4 + 3] = v4.w;
      }
      d32[128 * 32 + row] = scale_word;
    }
    // a look ahead at the next tile's S barrier and at its P buffer (free once the P.V that read it two tiles
    // before has finished): asked here, used at the top of the next tile
    s_ready = (j + 1 < n_tiles) && mbar_test_wait(s_full, (j + 1) & 1) &&
              (j < 1 || mbar_test_wait(&pv_done[(j + 1) & 1], ((j - 1) >> 1) & 1));
    if (stamp) RK_STAMP(grp, j, 4);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&p_full[pb]);
    if (stamp) RK_STAMP(grp, j, 5);
    return true;
  };

  // Tiles 0 .. n_plain-1 need no mask for any row of this query tile: no sliding window, all 128 keys inside S_kv,
  // and the tile's last key not beyond the first row's position.  Both bounds grow with j, so the plain tiles come
  // first; the general body decides again for every tile it gets.
  int n_plain = 0;
  if (p.window == 0) {
    n_plain = min(n_tiles, p.S_kv / kBlockN - j0);
    if (p.causal) {
      const int t = p.q_pos0 + qt * kBlockM - (kBlockN - 1);            // plain iff (j + j0) * kBlockN <= t
      n_plain = min(n_plain, t < 0 ? 0 : t / kBlockN + 1 - j0);
    }
    n_plain = max(n_plain, 0);
  }
  int j = 0;
  for (; j < n_plain && ok; ++j) ok = tile(j, std::true_type{});
  for (; j < n_tiles && ok; ++j) ok = tile(j, std::false_type{});
  if (!ok) report_wait_failure(abort_flag, p.status, fail);

  // ---- epilogue: O / l -> bf16 (finalize_O, flash_mx_impl.hpp:535-553) ----------------------------------------
  if (ok) {
    const int last = n_tiles - 1;
    ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[last & 1], (last >> 1) & 1, abort_flag, p.status, 103));
  }
  if (ok) {
    tc_fence_after();
    if (quad == 0 && lane == 0) RK_STAMP(grp, 0, 6);
    const float inv_l = (l_run > 0.0f) ? 1.0f / l_run : 1.0f;
    const bool live = q_row < p.S_q;
    __nv_bfloat16* orow = p.o + ((size_t)bh * p.S_q + q_row) * p.d;
    if (DUMP && dump) {
      p.dbg[128 * 128 + 128 * 32 + 128 + row * 2 + 0] = m_run;
      p.dbg[128 * 128 + 128 * 32 + 128 + row * 2 + 1] = l_run;
    }
    // the row's registers are free now: all of O is fetched with one wait (two halves when d > 64)
    const int n_c32 = p.d / 32;
#pragma unroll 1
    for (int h = 0; h < n_c32; h += 2) {
      uint32_t r[64];
      tmem_ld32(tmem_base + lane_addr + cO + grp * 128 + h * 32, r);
      if (h + 1 < n_c32) tmem_ld32(tmem_base + lane_addr + cO + grp * 128 + (h + 1) * 32, r + 32);
      tc_wait_ld();
      if (live) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (h + c < n_c32) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(r[c * 32 + 2 * i]) * inv_l, __uint_as_float(r[c * 32 + 2 * i + 1]) * inv_l);
              packed[i] = *reinterpret_cast<const uint32_t*>(&b2);
            }
            uint4* dst = reinterpret_cast<uint4*>(orow + (h + c) * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          }
        }
      }
    }
    if (p.lse && live)
      p.lse[(size_t)bh * p.S_q + q_row] = (l_run > 0.0f) ? m_run * 0.6931471805599453f + logf(l_run) : NEG_INF;
    if (quad == 0 && lane == 0) RK_STAMP(grp, 0, 7);
  }
  tc_fence_before();
}

// ---- correction warps: O <- O * corr before the tile's P.V is added ---------------------------------------------
__device__ __forceinline__ void correction_quadrant(const PrefillParams& p, uint8_t* smem, uint64_t* bars, uint32_t tmem_base,
                                                    volatile int* abort_flag, const int nt[2], int n_all) {
  using namespace c2;
  const int lane = threadIdx.x & 31;
  const int quad = (threadIdx.x >> 5) & 3;
  const int row = quad * 32 + lane;
  const uint32_t lane_addr = ((uint32_t)(quad * 32)) << 16;
  const float* corr_sm = reinterpret_cast<const float*>(smem + corr_off);
  const int o_chunks = p.d / 32;
  bool ok = true;
  for (int j = 0; j < n_all && ok; ++j) {
    const int pb = j & 1;
    perturb(p, kPerturbCorr, j);
#pragma unroll 1
    for (int g = 0; g < 2 && ok; ++g) {
      if (j >= nt[g]) continue;
      if (quad == 0 && lane == 0) RK_STAMP(3, j, g * 4 + 0);
      ok = __all_sync(0xffffffffu, mbar_wait_relaxed<kSleepNs>(&bars[bCF + (g * 4 + (j & 3)) * 4 + quad], (j >> 2) & 1, abort_flag, p.status, 401));
      if (!ok) break;
      const float corr = corr_sm[(g * 4 + (j & 3)) * 128 + row];
      if (quad == 0 && lane == 0) RK_STAMP(3, j, g * 4 + 1);
      if (j > 0) {
        // Always wait for the previous P.V of this tile, rescale or not: an arrival on the O-ready barrier then
        // implies that its previous phase has been consumed, which is what keeps the two-deep barrier from wrapping.
        ok = __all_sync(0xffffffffu, mbar_wait_relaxed<kSleepNs>(&bars[bPV + g * 2 + ((j - 1) & 1)], ((j - 1) >> 1) & 1, abort_flag, p.status, 402));
        if (!ok) break;
      }
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
        tc_fence_after();
        if (quad == 0 && lane == 0) RK_STAMP(3, j, g * 4 + 2);
#pragma unroll 1
        for (int ch = 0; ch < o_chunks; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_addr + cO + g * 128 + ch * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) mul2_ftz_inplace(r[i], r[i + 1], corr);
          tmem_st32(tmem_base + lane_addr + cO + g * 128 + ch * 32, r);
        }
        tc_wait_st();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[bOR + g * 2 + pb]);   // the tile's P.V may accumulate into O now
      if (quad == 0 && lane == 0) RK_STAMP(3, j, g * 4 + 3);
    }
  }
}

template <bool SOFTCAP, bool DUMP>
__global__ void __launch_bounds__(c2::kThreads, 1)
prefill2c_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p, const uint32_t idesc_qk,
                 const uint32_t idesc_pv) {
  using namespace c2;
  extern __shared__ __align__(1024) uint8_t smem_raw2c[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw2c) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + bar_off);
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc_off + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;   // an earlier launch gave up on a wait
  if (threadIdx.x == 0) RK_STAMP(2, 0, 6);
  const int n_pairs = (p.n_q_tiles + 1) / 2;
  // Work order over the 1-D grid: (batch, head) pairs are taken in groups of p.head_group; inside a group the
  // heaviest (latest) query-tile pairs of all its heads come first and the lightest last, so the grid ends on
  // short CTAs, while a group's K/V still fits in L2.
  const int n_bh = p.B * p.H;
  const int per_group = n_pairs * p.head_group;
  const int grp_i = (int)blockIdx.x / per_group, r = (int)blockIdx.x % per_group;
  const int heads_here = min(p.head_group, n_bh - grp_i * p.head_group);
  const int qp = n_pairs - 1 - r / heads_here;
  const int bh_lin = grp_i * p.head_group + r % heads_here;
  const int h = bh_lin % p.H, b = bh_lin / p.H;
  const int bh = b * p.H + h;
  const int bhkv = b * p.H_kv + h / (p.H / p.H_kv);

  // key tiles each query tile needs (causal tiles wholly above the diagonal are never touched,
  // kernels/flash_attention_mx_gqa/flash_attention_model.py:182-186); a tile past S_q needs none
  int nt[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int qt = 2 * qp + g;
    int n = (qt < p.n_q_tiles) ? p.n_kv_tiles : 0;
    if (n > 0 && p.causal) {
      const int max_qpos = p.q_pos0 + min(qt * kBlockM + kBlockM, p.S_q) - 1;
      n = max_qpos < 0 ? 0 : min(n, max_qpos / kBlockN + 1);
    }
    nt[g] = n;
  }
  // sliding window: key tiles wholly below the window of the pair's first row are masked for every row of both tiles
  int j0 = 0;
  if (p.window > 0) {
    const int first_key = p.q_pos0 + 2 * qp * kBlockM - p.window + 1;  // lowest key the first row may see
    j0 = min(max(first_key, 0) / kBlockN, max(min(nt[0], nt[1] > 0 ? nt[1] : nt[0]) - 1, 0));
    nt[0] = max(nt[0] - j0, 0);                                         // tiles j0 .. j0 + nt - 1 are visited
    nt[1] = max(nt[1] - j0, 0);
  }
  const int n_all = max(nt[0], nt[1]);

  // The TMA producer's lane sets up the barriers its first loads complete on and starts them at once (Q, and
  // K/V of the first key tile), so that their latency runs under the rest of the set-up; the other barriers
  // are set up one per thread.  Arrival counts: S-empty, P-full and O-ready take one arrival per warp of four.
  auto issue_kv = [&](int j) {
    const int st = j % kStages;
    mbar_arrive_expect_tx(&bars[bKF + st], p.kv_tile_tx + kSfAtomBytes);
    tma_load_3d(smem + k_off + st * kTileBytes, &tmap_k, &bars[bKF + st], 0, (j + j0) * kBlockN, bhkv);
    bulk_load_1d(smem + sfk_off + st * kSfAtomBytes, p.k_sf + ((size_t)bhkv * p.n_kv_tiles + j + j0) * kSfAtomBytes,
                 kSfAtomBytes, &bars[bKF + st]);
  };
  auto issue_v = [&](int j) {
    const int st = j % kStages;
    mbar_arrive_expect_tx(&bars[bVF + st], p.kv_tile_tx + kSfAtomBytes);
    if (p.v_transposed) tma_load_3d(smem + v_off + st * kTileBytes, &tmap_v, &bars[bVF + st], (j + j0) * kBlockN, 0, bhkv);
    else tma_load_3d(smem + v_off + st * kTileBytes, &tmap_v, &bars[bVF + st], 0, (j + j0) * kBlockN, bhkv);
    bulk_load_1d(smem + sfv_off + st * kSfAtomBytes, p.v_sf + ((size_t)bhkv * p.n_kv_tiles + j + j0) * kSfAtomBytes,
                 kSfAtomBytes, &bars[bVF + st]);
  };
  if (warp == kWarpTma) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(&bars[bQ], 1);
      for (int i = 0; i < kStages; ++i) { mbar_init(&bars[bKF + i], 1); mbar_init(&bars[bVF + i], 1); }
      fence_barrier_init();
      if (n_all > 0) {
        prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
        const int nq = (2 * qp + 1 < p.n_q_tiles) ? 2 : 1;
        mbar_arrive_expect_tx(&bars[bQ], nq * (p.q_tile_tx + kSfAtomBytes));
        for (int g = 0; g < nq; ++g) {
          tma_load_3d(smem + q_off + g * kTileBytes, &tmap_q, &bars[bQ], 0, (2 * qp + g) * kBlockM, bh);
          bulk_load_1d(smem + sfq_off + g * kSfAtomBytes, p.q_sf + ((size_t)bh * p.n_q_tiles + 2 * qp + g) * kSfAtomBytes,
                       kSfAtomBytes, &bars[bQ]);
        }
        issue_kv(0);
        issue_v(0);
      }
    }
  } else {
    const int i = (int)threadIdx.x;                  // barrier index this thread sets up (warps 0 and 1 suffice)
    if (i > bQ && i < nBars && !(i >= bKF && i < bKF + kStages) && !(i >= bVF && i < bVF + kStages)) {
      const bool per_warp = (i >= bSE && i < bSE + 2) || (i >= bPF && i < bPF + 4) || (i >= bOR && i < bOR + 4);
      mbar_init(&bars[i], per_warp ? 4 : 1);
      fence_barrier_init();
    }
  }
  if (threadIdx.x == 0) RK_STAMP_RAW(0);
  if (warp == kWarpQk) { if (lane == 0) RK_STAMP_RAW(1); tmem_alloc(tmem_ptr, kTmemCols); tmem_relinquish(); if (lane == 0) RK_STAMP_RAW(2); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  if (threadIdx.x == 0) RK_STAMP_RAW(3);
  if (threadIdx.x == kWarpTma * 32) RK_STAMP_RAW(4);

  // (The softmax branch comes last in the code: measured 1-1.5 % faster than first.)
  if (warp >= kWarpTma) {
    reg_dec<kRegIssue>();
    if (threadIdx.x == kWarpQk * 32) RK_STAMP_RAW(6);
    if (warp == kWarpTma) {
      // ================= TMA producer =================
      // Q and the first key tile are already on their way (issued before the block-wide barrier above)
      if (lane == 0 && n_all > 0) {
        bool ok = true;
        for (int j = 1; j < n_all && ok; ++j) {
          const int st = j % kStages, use = j / kStages;
          perturb(p, kPerturbTma, j);
          if (use > 0) ok = mbar_wait_relaxed<kSleepNs>(&bars[bKE + st], (use - 1) & 1, abort_flag, p.status, 201);
          if (!ok) break;
          issue_kv(j);
          if (use > 0) ok = mbar_wait_relaxed<kSleepNs>(&bars[bVE + st], (use - 1) & 1, abort_flag, p.status, 202);
          if (!ok) break;
          issue_v(j);
        }
      }
    } else if (warp == kWarpQk) {
      // ================= issuer of S = Q K^T =================
      // One thread issues; what it runs per key tile is kept short (a lone thread executes one instruction every
      // few cycles): descriptors are built once, a tile's descriptor is the base plus an offset in its low word.
      if (lane == 0 && n_all > 0) {
        const uint64_t dq = make_smem_desc(smem_u32(smem + q_off), 16, 1024, kLayoutSw128);
        const uint64_t dk = make_smem_desc(smem_u32(smem + k_off), 16, 1024, kLayoutSw128);
        const uint64_t dsfq = make_smem_desc(smem_u32(smem + sfq_off), 0, 128, kLayoutNone);
        const uint64_t dsfk = make_smem_desc(smem_u32(smem + sfk_off), 0, 128, kLayoutNone);
        RK_STAMP_RAW(7);
        bool ok = mbar_wait(&bars[bQ], 0, abort_flag, p.status, 301);
        RK_STAMP_RAW(8);
        if (ok) {
          tc_cp_32x128b_warpx4(tmem_base + cSfQ, dsfq);
          tc_cp_32x128b_warpx4(tmem_base + cSfQ + 4, dsfq + (kSfAtomBytes >> 4));
        }
        int st = 0, use_par = 0;                 // K stage of tile j and the parity of its use
        int last_g = -1, last_par = 0;           // which group read the shared S columns last, and at which tile parity
        for (int j = 0; j < n_all && ok; ++j) {
          perturb(p, kPerturbQk, j);
          RK_STAMP(2, j, 0);
          ok = mbar_wait_relaxed<kSleepNs>(&bars[bKF + st], use_par, abort_flag, p.status, 302);
          if (!ok) break;
          tc_cp_32x128b_warpx4(tmem_base + cSfK + st * 4, dsfk + (uint32_t)(st * (kSfAtomBytes >> 4)));
          const uint64_t dkt = dk + (uint32_t)(st * (kTileBytes >> 4));
          RK_STAMP(2, j, 1);
          // rolled on purpose (as in the P V issuer below): this warp shares its scheduler's instruction cache with
          // two softmax warps, and a lone thread loses nothing by a few loop instructions
#pragma unroll 1
          for (int g = 0; g < 2; ++g) {
            if (j >= (g == 0 ? nt[0] : nt[1])) continue;
            if (last_g >= 0) { ok = mbar_wait(&bars[bSE + last_g], last_par, abort_flag, p.status, 305); if (!ok) break; }
            tc_fence_after();
            const uint64_t dqt = dq + (uint32_t)(g * (kTileBytes >> 4));
#pragma unroll 1
            for (int kk = 0; kk < 4; ++kk)
              mma_mxf8f6f4_ss(tmem_base + cS, dqt + kk * 2, dkt + kk * 2, idesc_with_sf(idesc_qk, kk, kk), tmem_base + cSfQ + g * 4,
                              tmem_base + cSfK + st * 4, kk > 0 ? 1u : 0u);
            tc_commit(&bars[bSF + g]);
            last_g = g; last_par = j & 1;
            RK_STAMP(2, j, 2 + g);
          }
          if (ok) tc_commit(&bars[bKE + st]);
          if (++st == kStages) { st = 0; use_par ^= 1; }
        }
        tc_commit(&bars[bDRAIN]);
        mbar_wait(&bars[bDRAIN], 0, abort_flag, p.status, 306);
      }
      __syncwarp();
    } else if (warp == kWarpPv) {
      // ================= issuer of O += P V =================
      if (lane == 0 && n_all > 0) {
        const uint64_t dp = make_smem_desc(smem_u32(smem + p_off), 16, 1024, kLayoutSw128);
        // V tile [keys][d] is the MN-major B operand (32 keys = 32 rows of 128 bytes); a 6-bit V is stored
        // transposed and is K-major like K
        const uint64_t dv = p.v_transposed ? make_smem_desc(smem_u32(smem + v_off), 16, 1024, kLayoutSw128)
                                           : make_smem_desc(smem_u32(smem + v_off), kTileBytes, 1024, kLayoutSw128);
        const uint32_t v_kk = p.v_transposed ? 2u : (uint32_t)(4096 >> 4);
        const uint64_t dsfv = make_smem_desc(smem_u32(smem + sfv_off), 0, 128, kLayoutNone);
        const uint64_t dsfp = make_smem_desc(smem_u32(smem + sfp_off), 0, 128, kLayoutNone);
        bool ok = true;
        int st = 0, use_par = 0;
        for (int i = 0; i < n_all && ok; ++i) {
          const int pb = i & 1, par2 = (i >> 1) & 1;
          perturb(p, kPerturbPv, i);
          ok = mbar_wait_relaxed<kSleepNs>(&bars[bVF + st], use_par, abort_flag, p.status, 303);
          if (!ok) break;
          tc_cp_32x128b_warpx4(tmem_base + cSfV + st * 4, dsfv + (uint32_t)(st * (kSfAtomBytes >> 4)));
          const uint64_t dvt = dv + (uint32_t)(st * (kTileBytes >> 4));
#pragma unroll 1
          for (int g = 0; g < 2; ++g) {
            if (i >= (g == 0 ? nt[0] : nt[1])) continue;
            const int gb = g * 2 + pb;
            ok = mbar_wait_relaxed<kSleepNs>(&bars[bPF + gb], par2, abort_flag, p.status, 304) &&
                 mbar_wait_relaxed<kSleepNs>(&bars[bOR + gb], par2, abort_flag, p.status, 307);      // P written, O rescaled for this tile
            if (!ok) break;
            tc_fence_after();
            tc_cp_32x128b_warpx4(tmem_base + cSfP + gb * 4, dsfp + (uint32_t)(gb * (kSfAtomBytes >> 4)));
            const uint64_t dpt = dp + (uint32_t)(gb * (kTileBytes >> 4));
#pragma unroll 1
            for (int kk = 0; kk < 4; ++kk)
              mma_mxf8f6f4_ss(tmem_base + cO + g * 128, dpt + kk * 2, dvt + kk * v_kk, idesc_with_sf(idesc_pv, kk, kk),
                              tmem_base + cSfP + gb * 4, tmem_base + cSfV + st * 4, (i > 0 || kk > 0) ? 1u : 0u);
            tc_commit(&bars[bPV + gb]);
            RK_STAMP(2, i, 4 + g);
          }
          if (ok) tc_commit(&bars[bVE + st]);
          if (++st == kStages) { st = 0; use_par ^= 1; }
        }
        tc_commit(&bars[bDRAIN2]);
        mbar_wait(&bars[bDRAIN2], 0, abort_flag, p.status, 308);
      }
      __syncwarp();
    }
  } else if (warp >= kWarpCorr) {
    reg_dec<kRegCorr>();
    correction_quadrant(p, smem, bars, tmem_base, abort_flag, nt, n_all);
  } else {
    reg_inc<kRegSoftmax>();
    if (threadIdx.x == 0) RK_STAMP_RAW(5);
    const int grp = warp >> 2;
    const int qt = 2 * qp + grp;
    if (nt[grp] > 0) {
      softmax_row_group<SOFTCAP, DUMP>(p, smem, bars, tmem_base, abort_flag, grp, qt, bh, nt[grp], j0);
    } else if (qt < p.n_q_tiles) {
      // no visible key: O = 0 (the l <= 0 guard of finalize_O, kernels/flash_attention_mx_gemma/flash_mx_impl.hpp:554-560)
      const int q_row = qt * kBlockM + (int)(threadIdx.x & 127);
      if (q_row < p.S_q) {
        __nv_bfloat16* orow = p.o + ((size_t)bh * p.S_q + q_row) * p.d;
        for (int c = 0; c < p.d; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        if (p.lse) p.lse[(size_t)bh * p.S_q + q_row] = __int_as_float(0xff800000);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) RK_STAMP(2, 0, 7);
  if (warp == kWarpQk) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

template <bool SOFTCAP, bool DUMP>
static int launch2c_cfg(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                        uint32_t idesc_qk, uint32_t idesc_pv, dim3 grid, cudaStream_t st) {
  const int smem_bytes = c2::total + 1024;
  auto kern = prefill2c_kernel<SOFTCAP, DUMP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_before, st);
  kern<<<grid, c2::kThreads, smem_bytes, st>>>(tq, tk, tv, p, idesc_qk, idesc_pv);
  if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_after, st);
  return (int)cudaGetLastError();
}

int launch_prefill2c(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                     uint32_t idesc_qk, uint32_t idesc_pv, bool softcap, int B, cudaStream_t st) {
  dim3 grid(((p.n_q_tiles + 1) / 2) * p.H * B, 1, 1);
  if (p.dbg)      // the stage dump lives in an instantiation of its own, so that the kernel that ships carries none of its code
    return softcap ? launch2c_cfg<true, true>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st)
                   : launch2c_cfg<false, true>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st);
  return softcap ? launch2c_cfg<true, false>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st)
                 : launch2c_cfg<false, false>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st);
}

}  // namespace rk
