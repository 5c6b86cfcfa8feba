// MX flash-attention prefill for sm_100a: TMA -> shared memory -> tcgen05
// block-scaled MMA (kind::mxf8f6f4, E8M0 scales in TMEM) -> fp32 online softmax
// in registers -> P re-quantized to E4M3 + E8M0 per 32 keys -> second
// block-scaled MMA accumulating O in TMEM.
//
// Follows the streaming tile loop of fa_entry,
// kernels/flash_attention_mx_gqa/kernel.cpp:91-184 (QK_j -> fused softmax+requant
// -> scale pack -> PV_j -> rescale/accumulate -> finalize), with the stages
// mapped onto Blackwell units:
//   mxgemm_prefetch_tile / mxgemm_compute_tile (mesh)  -> TMA + tcgen05.mma
//   fused_softmax_requant_tpr (one lane per row,
//     flash_mx_impl.hpp:314-394)                       -> four threads per row, one 32-key block each in registers
//   pack_scales_to_sfmem (flash_mx_impl.hpp:625-639)   -> one st.shared per row + tcgen05.cp
//   rescale_accumulate / finalize_O (:508-553)         -> O kept in TMEM, rescaled in place
//
// One CTA = one 128-row query tile of one (batch, head).  608 threads:
//   warps 0-15  softmax: four threads per query row (TMEM lane = row), one 32-key block of the tile each
//   warp  16    TMA producer (one elected lane)
//   warp  17    issuer of the S = Q K^T MMAs (one elected lane), TMEM allocation
//   warp  18    issuer of the O += P V MMAs (one elected lane): a P V that waits for its P tile never holds back
//               the next Q K^T, and each issuing thread runs a short instruction stream per key tile
// Keys are walked in tiles of 128 (the online-softmax step, "block_n").
//
// Roofline: tensor-core bound by FLOP count (4*S_q*S_kv*d per head, half of it
// when causal); in practice the softmax/requant ALU work per S element bounds it.
#include <cuda.h>
#include <algorithm>
#include <type_traits>
#include <cuda_bf16.h>

#include "rk_common.cuh"
#include "rk_internal.h"
#include "rk_prefill.cuh"

namespace rk {

template <int DCH, int KV_STAGES>
struct SmemLayout {
  static constexpr int q_off = 0;
  static constexpr int k_off = q_off + DCH * kTileBytes;
  static constexpr int v_off = k_off + KV_STAGES * DCH * kTileBytes;
  static constexpr int p_off = v_off + KV_STAGES * DCH * kTileBytes;
  static constexpr int sfq_off = p_off + 2 * kTileBytes;
  static constexpr int sfk_off = sfq_off + DCH * kSfAtomBytes;
  static constexpr int sfv_off = sfk_off + KV_STAGES * DCH * kSfAtomBytes;
  static constexpr int sfp_off = sfv_off + KV_STAGES * DCH * kSfAtomBytes;
  static constexpr int bar_off = sfp_off + 2 * kSfAtomBytes;
  // barriers: q_full, k_full[S], k_empty[S], v_full[S], v_empty[S], s_full, s_empty, p_full[2], pv_done[2], drain, pair[4], drain2
  static constexpr int n_bars = 1 + 4 * KV_STAGES + 2 + 4 + 1 + 4 + 1;
  static constexpr int misc_off = bar_off + n_bars * 8;
  static constexpr int xchg_off = misc_off + 16;          // row-max / row-sum exchange: 3 x kParts x 128 floats
  static constexpr int total = xchg_off + 3 * kParts * 128 * 4;
};

// ---- softmax warps -----------------------------------------------------------------------------
// 4 * kParts warps: warp w serves TMEM lane quadrant q = w & 3 (rows 32q..32q+31) and the 32-key block
// w >> 2 of the tile, so a thread's keys are exactly one MX block of P.  The kParts threads of a row
// exchange their block maxima through shared memory (one bounded mbarrier per quadrant, one arrival per
// warp); everything else is private.
template <int DCH, int KV_STAGES, bool SOFTCAP, bool DUMP>
__device__ __forceinline__ void softmax_rows(const PrefillParams& p, uint8_t* smem, uint64_t* bars, uint32_t tmem_base,
                                             volatile int* abort_flag, int qt, int bh, int n_tiles, int j0) {
  using L = SmemLayout<DCH, KV_STAGES>;
  uint64_t* s_full = bars + 1 + 4 * KV_STAGES;
  uint64_t* s_empty = s_full + 1;
  uint64_t* p_full = s_empty + 1;     // [2]
  uint64_t* pv_done = p_full + 2;     // [2]
  uint64_t* quadbar = pv_done + 3;    // [4]: the kParts warps of a lane quadrant meet here (bounded, unlike bar.sync)
  float* xchg = reinterpret_cast<float*>(smem + L::xchg_off);   // [3][kParts][128 rows]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int quad = warp & 3, part = warp >> 2;             // TMEM lane quadrant, 32-key block of the tile
  const int row = quad * 32 + lane;
  const uint32_t lane_addr = ((uint32_t)(quad * 32)) << 16;
  const int q_row = qt * kBlockM + row;
  const int q_pos = p.q_pos0 + q_row;
  const float NEG_INF = __int_as_float(0xff800000);
  constexpr int kOCols = DCH * 128 / kParts;               // O columns this thread rescales (32 or 64)

  float m_run = NEG_INF;   // running max, log2 domain (score * log2 e)
  float l_run = 0.0f;      // this thread's share of the row sum
  bool ok = true;

  // The body of a key tile exists twice: PLAIN for tiles no row of which needs a mask, and the general one with the
  // mask code.  The loop over plain tiles runs nearly all the time and is kept small and contiguous (the softmax
  // warps stall on instruction fetch; code inside the loop costs time even when it is jumped over).
  auto tile = [&](const int j, auto plain_tag) -> bool {
    constexpr bool PLAIN = decltype(plain_tag)::value;
    const int pb = j & 1;
    const int sslot = (warp == 0) ? 0 : (warp == 15 ? 1 : 7);
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 0);
    if (!__all_sync(0xffffffffu, mbar_wait(s_full, j & 1, abort_flag, p.status, 101))) return false;
    tc_fence_after();
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 1);

    // mask bounds relative to the tile's first key: key column c is masked iff c > hi || c <= lo
    const int key0 = (j + j0) * kBlockN;                      // first key of this tile (j counts from the first tile inside the window)
    const bool tail = (key0 + kBlockN > p.S_kv);
    const bool diag = p.causal && (key0 + kBlockN - 1 > p.q_pos0 + qt * kBlockM);
    const bool need_mask = !PLAIN && (tail || diag || (p.window > 0));
    int hi = p.S_kv - 1 - key0;
    if (p.causal) hi = min(hi, q_pos - key0);
    const int lo = (p.window > 0) ? (q_pos - p.window - key0) : -1;

    float s[32];
    tmem_ld32(tmem_base + lane_addr + kColS + part * 32, reinterpret_cast<uint32_t*>(s));
    tc_wait_ld();
    float mx_others = NEG_INF;
    if (!SOFTCAP) {
      // Row max without talking to the other warps: read the row's other three 32-key blocks as well
      // (TMEM reads are cheap) and reduce them here.  The warps of a row then never wait for each other.
#pragma unroll 1
      for (int o = 1; o < kParts; ++o) {
        const int blk = (part + o) & (kParts - 1);
        float t[32];
        tmem_ld32(tmem_base + lane_addr + kColS + blk * 32, reinterpret_cast<uint32_t*>(t));
        tc_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) t[c] = (blk * 32 + c > hi || blk * 32 + c <= lo) ? NEG_INF : t[c];
        }
        float b0 = fmax3(t[0], t[1], t[2]), b1 = fmax3(t[3], t[4], t[5]);
#pragma unroll
        for (int c = 6; c < 30; c += 4) { b0 = fmax3(b0, t[c], t[c + 1]); b1 = fmax3(b1, t[c + 2], t[c + 3]); }
        mx_others = fmax3(mx_others, fmax3(b0, b1, t[30]), t[31]);
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(s_empty);        // one arrival per warp: S may be overwritten once all 16 have read
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 2);

    if (DUMP && p.dbg && qt == p.n_q_tiles - 1 && bh == 0 && j == 0) {
#pragma unroll
      for (int c = 0; c < 32; ++c) p.dbg[row * 128 + part * 32 + c] = s[c];
    }

    // ---- (soft-cap,) mask, block max ---------------------------------------------------------------
    // Without a cap the max is taken on the raw scores (the scale is positive) and the scale is folded
    // into the exponent's FMA; with a cap s[] is replaced by the capped score in the log2 domain.
    if (SOFTCAP) softcap_scores(s, p.scale_log2, p.cap_log2, p.inv_cap_scale);   // cap * tanh(s * scale / cap), pre-multiplied by log2 e
    if (need_mask) {
#pragma unroll
      for (int c = 0; c < 32; ++c) s[c] = (part * 32 + c > hi || part * 32 + c <= lo) ? NEG_INF : s[c];
    }
    float a0 = fmax3(s[0], s[1], s[2]), a1 = fmax3(s[3], s[4], s[5]);
#pragma unroll
    for (int c = 6; c < 30; c += 4) { a0 = fmax3(a0, s[c], s[c + 1]); a1 = fmax3(a1, s[c + 2], s[c + 3]); }
    const float bmax = fmax3(a0, a1, fmaxf(s[30], s[31]));     // this block's max (raw / capped domain)
    float mx = fmaxf(bmax, mx_others);
    if (SOFTCAP) {
      // the capped scores cost two MUFU ops each, so here the four threads of a row exchange block maxima
      xchg[(pb * kParts + part) * 128 + row] = bmax;
      __syncwarp();
      if (lane == 0) mbar_arrive(&quadbar[quad]);
      if (!__all_sync(0xffffffffu, mbar_wait(&quadbar[quad], j & 1, abort_flag, p.status, 104))) return false;
#pragma unroll
      for (int o = 1; o < kParts; ++o) mx = fmaxf(mx, xchg[(pb * kParts + ((part + o) & (kParts - 1))) * 128 + row]);
    }
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 3);
    const float sc_mul = SOFTCAP ? 1.0f : p.scale_log2;
    const float m_new = fmaxf(m_run, mx * sc_mul);            // -inf * positive stays -inf
    // The exponent is formed as fma(s, scale, -m): for the row-max element that leaves the rounding
    // residue of s*scale (up to half an ulp of m) instead of exactly 0, and a p a hair below 1 would
    // drop the block scale by a binade.  Lowering the subtracted max by 2^-21 |m| keeps that p in
    // [1, 1 + 1e-5); the common factor cancels in O = sum(p v) / sum(p).
    const float m_use = (m_new == NEG_INF) ? 0.0f : (SOFTCAP ? m_new : fmaf(-fabsf(m_new), 4.76837158203125e-7f, m_new));
    const float corr = (m_run == NEG_INF) ? 1.0f : ex2_approx(m_run - m_new);
    m_run = m_new;

    // ---- p = 2^(x - m), row sum from the unquantised p, requant of this 32-key block ---------------
    uint8_t* p_tile = smem + L::p_off + pb * kTileBytes + row * 128;
    float ls0 = 0.0f, ls1 = 0.0f, ls2 = 0.0f, ls3 = 0.0f;
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
      // two packed FMAs form the four exponents; the exponentials themselves go to the MUFU one by one
      float x0, x1, x2, x3;
      fma2(s[c + 0], s[c + 1], sc_mul, -m_use, x0, x1);
      fma2(s[c + 2], s[c + 3], sc_mul, -m_use, x2, x3);
      const float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
      s[c + 0] = p0; s[c + 1] = p1; s[c + 2] = p2; s[c + 3] = p3;
      add2(ls0, ls1, p0, p1);
      add2(ls2, ls3, p2, p3);
    }
    // block max of p = 2^(block max of x - m): exp2 is monotone, so it is the p of the arg-max element
    const float pmax = ex2_approx(fmaf(bmax, sc_mul, -m_use));
    // E8M0 code = exponent field of the block max (se = floor(log2 pmax) <= 0; an all-zero block gives 0)
    int sc = (int)(__float_as_uint(pmax) >> 23);
    sc = min(sc, 127);
    uint32_t w[8];
    {
      // y = p * 2^(7-sc) has exponent field E - se + 7 = the E4M3 exponent field and keeps the mantissa,
      // so the truncated code is y's bits [20,27); .ftz zeroes everything below 2^-6 of the block scale.
      // ex2.approx.ftz never returns a subnormal, so this holds whatever sc is (a block whose maximum lies
      // below 2^-120 needs no other path: its non-zero elements all lie within 2^6 of that maximum).
      const float f = __uint_as_float((uint32_t)(134 - sc) << 23);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float y0, y1, y2, y3;
        mul2_ftz(s[q * 4 + 0], s[q * 4 + 1], f, y0, y1);
        mul2_ftz(s[q * 4 + 2], s[q * 4 + 3], f, y2, y3);
        w[q] = pack_u8x2(__float_as_uint(y1) >> 20, __float_as_uint(y0) >> 20,
                         pack_u8x2(__float_as_uint(y3) >> 20, __float_as_uint(y2) >> 20, 0u));
      }
    }
    {
      // two 16-byte chunks of this row, 128-byte swizzle: chunk index XOR (row % 8)
      const int c0 = (2 * part) ^ (row & 7), c1 = (2 * part + 1) ^ (row & 7);
      *reinterpret_cast<uint4*>(p_tile + c0 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(p_tile + c1 * 16) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    l_run = l_run * corr + ((ls0 + ls1) + (ls2 + ls3));
    smem[L::sfp_off + pb * kSfAtomBytes + (row & 31) * 16 + (row >> 5) * 4 + part] = (uint8_t)sc;

    if (DUMP && p.dbg && qt == p.n_q_tiles - 1 && bh == 0 && j == 0) {
      // P codes as written (un-swizzled view) and the scale bytes, after the 128x128 S dump
      uint32_t* d32 = reinterpret_cast<uint32_t*>(p.dbg + 128 * 128);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int lc = part * 2 + c;
        const uint4 v4 = *reinterpret_cast<const uint4*>(p_tile + ((lc ^ (row & 7)) * 16));
        d32[row * 32 + lc * 4 + 0] = v4.x; d32[row * 32 + lc * 4 + 1] = v4.y;
        d32[row * 32 + lc * 4 + 2] = v4.z; d32[row * 32 + lc * 4 + 3] = v4.w;
      }
      reinterpret_cast<uint8_t*>(d32 + 128 * 32)[row * 4 + part] = (uint8_t)sc;
    }

    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 4);
    // ---- rescale this thread's share of O in TMEM once the previous PV has landed (it had the whole
    //      exp/requant phase above to finish, so this wait is normally free) ----------------------------
    if (j > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, 102))) return false;
      tc_fence_after();
      if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int ch = 0; ch < kOCols / 32; ++ch) {
          uint32_t r[32];
          const uint32_t addr = tmem_base + lane_addr + kColO + part * kOCols + ch * 32;
          tmem_ld32(addr, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) mul2_ftz_inplace(r[i], r[i + 1], corr);
          tmem_st32(addr, r);
        }
        tc_wait_st();
      }
    }
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 5);
    fence_proxy_async_smem();   // make the st.shared P tile + scales visible to the tensor-core (async) proxy
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&p_full[pb]);
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 6);
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

  // ---- epilogue: O / l -> bf16, each thread d / kParts of the columns -------------------------------
  float l_tot = l_run;
  if (ok) {
    xchg[(2 * kParts + part) * 128 + row] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(&quadbar[quad]);
    ok = __all_sync(0xffffffffu, mbar_wait(&quadbar[quad], SOFTCAP ? (n_tiles & 1) : 0, abort_flag, p.status, 105));
    if (ok) {
#pragma unroll
      for (int o = 1; o < kParts; ++o) l_tot += xchg[(2 * kParts + ((part + o) & (kParts - 1))) * 128 + row];
    }
  }
  if (ok) {
    const int last = n_tiles - 1;
    ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[last & 1], (last >> 1) & 1, abort_flag, p.status, 103));
  }
  if (ok) {
    tc_fence_after();
    const float inv_l = (l_tot > 0.0f) ? 1.0f / l_tot : 1.0f;
    const bool live = q_row < p.S_q;
    __nv_bfloat16* orow = p.o + ((size_t)bh * p.S_q + q_row) * p.d;
    const int ncols = p.d / kParts;                 // 16, 32 or 64 output columns per thread
    if (DUMP && p.dbg && qt == p.n_q_tiles - 1 && bh == 0 && part == 0) {
      p.dbg[128 * 128 + 128 * 32 + 128 + row * 2 + 0] = m_run;
      p.dbg[128 * 128 + 128 * 32 + 128 + row * 2 + 1] = l_tot;
    }
#pragma unroll 1
    for (int c16 = 0; c16 < ncols / 16; ++c16) {
      uint32_t r[16];
      const int col0 = part * ncols + c16 * 16;
      tmem_ld16(tmem_base + lane_addr + kColO + col0, r);
      tc_wait_ld();
      if (live) {
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
          packed[i] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        uint4* dst = reinterpret_cast<uint4*>(orow + col0);
        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      }
    }
    if (p.lse && live && part == 0)
      p.lse[(size_t)bh * p.S_q + q_row] = (l_tot > 0.0f) ? m_run * 0.6931471805599453f + logf(l_tot) : NEG_INF;
  }
  tc_fence_before();
}

// ---- the kernel ---------------------------------------------------------------------------------
template <int DCH, int KV_STAGES, bool SOFTCAP, bool DUMP>
__global__ void __launch_bounds__(kNumThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p, const uint32_t idesc_qk,
               const uint32_t idesc_pv) {
  using L = SmemLayout<DCH, KV_STAGES>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + L::misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc_off + 4);

  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_full = v_empty + KV_STAGES;
  uint64_t* s_empty = s_full + 1;
  uint64_t* p_full = s_empty + 1;
  uint64_t* pv_done = p_full + 2;
  uint64_t* drain = pv_done + 2;
  uint64_t* drain2 = drain + 5;       // after the four pair barriers

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // an earlier launch on this device gave up on a wait: do nothing until the host has read the status
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;
  // heavy (late) query tiles first within a head; heads adjacent so a KV head's tiles share L2
  // work order: see PrefillParams::head_group (heaviest query tiles of a whole group of heads first)
  const int n_bh = p.B * p.H;
  const int per_group = p.n_q_tiles * p.head_group;
  const int grp_i = (int)blockIdx.x / per_group, r = (int)blockIdx.x % per_group;
  const int heads_here = min(p.head_group, n_bh - grp_i * p.head_group);
  const int qt = p.n_q_tiles - 1 - r / heads_here;
  const int bh_lin = grp_i * p.head_group + r % heads_here;
  const int h = bh_lin % p.H, b = bh_lin / p.H;
  const int bh = b * p.H + h;
  const int bhkv = b * p.H_kv + h / (p.H / p.H_kv);

  // key tiles this query tile needs: causal tiles wholly above the diagonal are never touched
  // (blocks_used, kernels/flash_attention_mx_gqa/flash_attention_model.py:182-186)
  int n_tiles = p.n_kv_tiles;
  if (p.causal) {
    const int max_qpos = p.q_pos0 + min(qt * kBlockM + kBlockM, p.S_q) - 1;
    n_tiles = max_qpos < 0 ? 0 : min(n_tiles, max_qpos / kBlockN + 1);
  }
  // sliding window: key tiles wholly below the window of the tile's first row are masked for every row of it
  int j0 = 0;
  if (p.window > 0) {
    const int first_key = p.q_pos0 + qt * kBlockM - p.window + 1;      // lowest key the first row may see
    j0 = min(max(first_key, 0) / kBlockN, max(n_tiles - 1, 0));
    n_tiles -= j0;                                                      // tiles j0 .. j0 + n_tiles - 1 are visited
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(s_empty, kNumSoftmaxWarps);
    mbar_init(&p_full[0], kNumSoftmaxWarps); mbar_init(&p_full[1], kNumSoftmaxWarps);
    mbar_init(&pv_done[0], 1); mbar_init(&pv_done[1], 1);
    mbar_init(drain, 1); mbar_init(drain2, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&drain[1 + i], kParts);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kNumSoftmaxWarps + 1) { tmem_alloc(tmem_ptr, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (n_tiles == 0) {
    // no visible key: O = 0 (the l <= 0 guard of finalize_O, kernels/flash_attention_mx_gemma/flash_mx_impl.hpp:554-560)
    if (warp < 4) {
      const int q_row = qt * kBlockM + threadIdx.x;
      if (q_row < p.S_q) {
        __nv_bfloat16* orow = p.o + ((size_t)bh * p.S_q + q_row) * p.d;
        for (int c = 0; c < p.d; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        if (p.lse) p.lse[(size_t)bh * p.S_q + q_row] = __int_as_float(0xff800000);
      }
    }
  } else if (warp < kNumSoftmaxWarps) {
    softmax_rows<DCH, KV_STAGES, SOFTCAP, DUMP>(p, smem, bars, tmem_base, abort_flag, qt, bh, n_tiles, j0);
  } else if (warp == kNumSoftmaxWarps) {
    // ================= TMA producer =================
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(q_full, DCH * (p.q_tile_tx + kSfAtomBytes));
      for (int ch = 0; ch < DCH; ++ch) {
        tma_load_3d(smem + L::q_off + ch * kTileBytes, &tmap_q, q_full, ch * 128, qt * kBlockM, bh);
        bulk_load_1d(smem + L::sfq_off + ch * kSfAtomBytes,
                     p.q_sf + (((size_t)bh * p.n_q_tiles + qt) * DCH + ch) * kSfAtomBytes, kSfAtomBytes, q_full);
      }
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % KV_STAGES, use = j / KV_STAGES;
        if (use > 0) ok = mbar_wait(&k_empty[st], (use - 1) & 1, abort_flag, p.status, 201);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[st], DCH * (p.kv_tile_tx + kSfAtomBytes));
        for (int ch = 0; ch < DCH; ++ch) {
          tma_load_3d(smem + L::k_off + (st * DCH + ch) * kTileBytes, &tmap_k, &k_full[st], ch * 128, (j + j0) * kBlockN, bhkv);
          bulk_load_1d(smem + L::sfk_off + (st * DCH + ch) * kSfAtomBytes,
                       p.k_sf + (((size_t)bhkv * p.n_kv_tiles + j + j0) * DCH + ch) * kSfAtomBytes, kSfAtomBytes, &k_full[st]);
        }
        if (use > 0) ok = mbar_wait(&v_empty[st], (use - 1) & 1, abort_flag, p.status, 202);
        if (!ok) break;
        mbar_arrive_expect_tx(&v_full[st], DCH * (p.kv_tile_tx + kSfAtomBytes));
        for (int ch = 0; ch < DCH; ++ch) {
          if (p.v_transposed)
            tma_load_3d(smem + L::v_off + (st * DCH + ch) * kTileBytes, &tmap_v, &v_full[st], (j + j0) * kBlockN, ch * 128, bhkv);
          else
            tma_load_3d(smem + L::v_off + (st * DCH + ch) * kTileBytes, &tmap_v, &v_full[st], ch * 128, (j + j0) * kBlockN, bhkv);
          bulk_load_1d(smem + L::sfv_off + (st * DCH + ch) * kSfAtomBytes,
                       p.v_sf + (((size_t)bhkv * p.n_kv_tiles + j + j0) * DCH + ch) * kSfAtomBytes, kSfAtomBytes, &v_full[st]);
        }
      }
    }
  } else if (warp == kNumSoftmaxWarps + 1) {
    // ================= issuer of S = Q K^T =================
    // One thread issues; what it runs per key tile is kept short (a lone thread executes one instruction every few
    // cycles): descriptors are built once, a tile's descriptor is the base plus an offset in its low word.
    if (lane == 0) {
      const uint64_t dq = make_smem_desc(smem_u32(smem + L::q_off), 16, 1024, kLayoutSw128);
      const uint64_t dk = make_smem_desc(smem_u32(smem + L::k_off), 16, 1024, kLayoutSw128);
      const uint64_t dsfq = make_smem_desc(smem_u32(smem + L::sfq_off), 0, 128, kLayoutNone);
      const uint64_t dsfk = make_smem_desc(smem_u32(smem + L::sfk_off), 0, 128, kLayoutNone);
      uint32_t idesc_kk[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) idesc_kk[kk] = idesc_with_sf(idesc_qk, kk, kk);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 301);
      if (ok) {
#pragma unroll
        for (int ch = 0; ch < DCH; ++ch) tc_cp_32x128b_warpx4(tmem_base + kColSfQ + ch * 4, dsfq + (uint32_t)(ch * (kSfAtomBytes >> 4)));
      }
      int st = 0, use_par = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        RK_STAMP(2, j, 0);
        ok = mbar_wait(&k_full[st], use_par, abort_flag, p.status, 302);
        RK_STAMP(2, j, 1);
        if (ok && j > 0) ok = mbar_wait(s_empty, (j - 1) & 1, abort_flag, p.status, 305);
        if (!ok) break;
        tc_fence_after();
        RK_STAMP(2, j, 2);
#pragma unroll
        for (int ch = 0; ch < DCH; ++ch)
          tc_cp_32x128b_warpx4(tmem_base + kColSfK + st * 8 + ch * 4, dsfk + (uint32_t)((st * DCH + ch) * (kSfAtomBytes >> 4)));
#pragma unroll
        for (int ch = 0; ch < DCH; ++ch) {
          const uint64_t dqt = dq + (uint32_t)(ch * (kTileBytes >> 4));
          const uint64_t dkt = dk + (uint32_t)((st * DCH + ch) * (kTileBytes >> 4));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_mxf8f6f4_ss(tmem_base + kColS, dqt + kk * 2, dkt + kk * 2, idesc_kk[kk], tmem_base + kColSfQ + ch * 4,
                            tmem_base + kColSfK + st * 8 + ch * 4, (ch > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(s_full);
        RK_STAMP(2, j, 3);
        if (++st == KV_STAGES) { st = 0; use_par ^= 1; }
      }
      // make sure nothing issued from this thread is still running before TMEM is released
      tc_commit(drain);
      mbar_wait(drain, 0, abort_flag, p.status, 306);
    }
    __syncwarp();
  } else {
    // ================= issuer of O += P V =================
    if (lane == 0) {
      const uint64_t dp = make_smem_desc(smem_u32(smem + L::p_off), 16, 1024, kLayoutSw128);
      // B = V tile, MN-major (d contiguous): 32 keys = 32 rows of 128 bytes; a 6-bit V is stored transposed,
      // [d][keys], and is K-major like the K tile of QK^T
      const uint64_t dv = p.v_transposed ? make_smem_desc(smem_u32(smem + L::v_off), 16, 1024, kLayoutSw128)
                                         : make_smem_desc(smem_u32(smem + L::v_off), kTileBytes, 1024, kLayoutSw128);
      const uint32_t v_kk = p.v_transposed ? 2u : (uint32_t)(4096 >> 4);
      const uint64_t dsfp = make_smem_desc(smem_u32(smem + L::sfp_off), 0, 128, kLayoutNone);
      const uint64_t dsfv = make_smem_desc(smem_u32(smem + L::sfv_off), 0, 128, kLayoutNone);
      uint32_t idesc_kk[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) idesc_kk[kk] = idesc_with_sf(idesc_pv, kk, kk);
      bool ok = true;
      int st = 0, use_par = 0;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int pb = i & 1;
        ok = mbar_wait(&v_full[st], use_par, abort_flag, p.status, 303) &&
             mbar_wait(&p_full[pb], (i >> 1) & 1, abort_flag, p.status, 304);
        if (!ok) break;
        tc_fence_after();
        tc_cp_32x128b_warpx4(tmem_base + kColSfP + pb * 4, dsfp + (uint32_t)(pb * (kSfAtomBytes >> 4)));
#pragma unroll
        for (int ch = 0; ch < DCH; ++ch)
          tc_cp_32x128b_warpx4(tmem_base + kColSfV + st * 8 + ch * 4, dsfv + (uint32_t)((st * DCH + ch) * (kSfAtomBytes >> 4)));
        const uint64_t dpt = dp + (uint32_t)(pb * (kTileBytes >> 4));
#pragma unroll
        for (int ch = 0; ch < DCH; ++ch) {
          const uint64_t dvt = dv + (uint32_t)((st * DCH + ch) * (kTileBytes >> 4));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_mxf8f6f4_ss(tmem_base + kColO + ch * 128, dpt + kk * 2, dvt + kk * v_kk, idesc_kk[kk],
                            tmem_base + kColSfP + pb * 4, tmem_base + kColSfV + st * 8 + ch * 4, (i > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&v_empty[st]);
        tc_commit(&pv_done[pb]);
        if (++st == KV_STAGES) { st = 0; use_par ^= 1; }
      }
      tc_commit(drain2);
      mbar_wait(drain2, 0, abort_flag, p.status, 308);
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kNumSoftmaxWarps + 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

// ---- host side ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// [BH][S][d] bytes, box = 128 bytes of d x 128 rows x 1, 128-byte swizzle, rows/cols past the edge read as 0
int make_tmap_u8_3d(CUtensorMap* m, const void* base, int64_t BH, int64_t S, int64_t d) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return RK_ERR_NO_DEVICE;
  cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)d, (cuuint64_t)(S * d)};
  cuuint32_t box[3] = {128, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RK_OK : RK_ERR_BAD_SHAPE;
}

// Packed 6-bit tensor [BH][rows][cols_padded codes], cols_padded a multiple of 128; a box is 128 codes x 128 rows
// and lands in shared memory as 128 bytes per row (16 codes in 12 bytes + 4 bytes of padding, 128-byte swizzle).
// bits = 4: the same with 16 codes in 8 bytes + 8 bytes of padding (16U4_ALIGN16B).
int make_tmap_sub8_3d(CUtensorMap* m, const void* base, int64_t BH, int64_t rows, int64_t cols_padded, int bits) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return RK_ERR_NO_DEVICE;
  const cuuint64_t row_bytes = (cuuint64_t)cols_padded * bits / 8;
  cuuint64_t dims[3] = {(cuuint64_t)cols_padded, (cuuint64_t)rows, (cuuint64_t)BH};
  cuuint64_t strides[2] = {row_bytes, row_bytes * (cuuint64_t)rows};
  cuuint32_t box[3] = {128, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, bits == 4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RK_OK : RK_ERR_BAD_SHAPE;
}

template <int DCH, int KV_STAGES, bool SOFTCAP, bool DUMP>
static int launch_cfg(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                      uint32_t idesc_qk, uint32_t idesc_pv, dim3 grid, cudaStream_t st) {
  using L = SmemLayout<DCH, KV_STAGES>;
  const int smem_bytes = L::total + 1024;
  auto kern = prefill_kernel<DCH, KV_STAGES, SOFTCAP, DUMP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_before, st);
  kern<<<grid, kNumThreads, smem_bytes, st>>>(tq, tk, tv, p, idesc_qk, idesc_pv);
  if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_after, st);
  return (int)cudaGetLastError();
}

float* g_prefill_dbg = nullptr;   // set by rk_debug_set_prefill_dump (tests only)
int g_prefill_perturb = 0;

int launch_prefill(const rk_prefill_args& a, const uint8_t* q_codes, const uint8_t* k_codes, const uint8_t* v_codes,
                   const uint8_t* q_sf, const uint8_t* k_sf, const uint8_t* v_sf, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  int rc;
  const bool q6 = a.q_fmt >= RK_FMT_E2M3, kv6 = a.kv_fmt >= RK_FMT_E2M3;                  // packed sub-byte operands
  const int qbits = a.q_fmt == RK_FMT_E2M1 ? 4 : 6, kvbits = a.kv_fmt == RK_FMT_E2M1 ? 4 : 6;
  const int64_t dp = (a.d + 127) / 128 * 128, skp = ((int64_t)a.S_kv + 127) / 128 * 128;
  rc = q6 ? make_tmap_sub8_3d(&tq, q_codes, (int64_t)a.B * a.H, a.S_q, dp, qbits) : make_tmap_u8_3d(&tq, q_codes, (int64_t)a.B * a.H, a.S_q, a.d);
  if (rc != RK_OK) return rc;
  rc = kv6 ? make_tmap_sub8_3d(&tk, k_codes, (int64_t)a.B * a.H_kv, a.S_kv, dp, kvbits) : make_tmap_u8_3d(&tk, k_codes, (int64_t)a.B * a.H_kv, a.S_kv, a.d);
  if (rc != RK_OK) return rc;
  rc = kv6 ? make_tmap_sub8_3d(&tv, v_codes, (int64_t)a.B * a.H_kv, a.d, skp, kvbits) : make_tmap_u8_3d(&tv, v_codes, (int64_t)a.B * a.H_kv, a.S_kv, a.d);
  if (rc != RK_OK) return rc;

  PrefillParams p;
  p.q_sf = q_sf; p.k_sf = k_sf; p.v_sf = v_sf;
  p.o = reinterpret_cast<__nv_bfloat16*>(a.o);
  p.lse = a.lse;
  p.status = device_status_word();
  if (!p.status) return RK_ERR_NO_DEVICE;
  p.dbg = g_prefill_dbg;
  p.B = a.B; p.H = a.H; p.H_kv = a.H_kv; p.S_q = a.S_q; p.S_kv = a.S_kv; p.d = a.d;
  {
    // heads whose K and V (shared by the query heads of a KV head) fit in about 100 MB of L2, in equal groups
    const double per_head = 2.0 * a.S_kv * a.d * ((double)a.H_kv / a.H);
    const int n_bh = a.B * a.H;
    const int fit = (int)std::max(8.0, 100.0e6 / std::max(per_head, 1.0));
    const int ngroups = (n_bh + fit - 1) / fit;
    p.head_group = (n_bh + ngroups - 1) / ngroups;
  }
  p.n_q_tiles = (a.S_q + kBlockM - 1) / kBlockM;
  p.n_kv_tiles = (a.S_kv + kBlockN - 1) / kBlockN;
  p.q_pos0 = a.q_pos0; p.causal = a.causal; p.window = a.window;
  p.v_transposed = kv6 ? 1 : 0;
  p.perturb = g_prefill_perturb;
  p.q_tile_tx = q6 ? kTileBytes * qbits / 8 : kTileBytes;
  p.kv_tile_tx = kv6 ? kTileBytes * kvbits / 8 : kTileBytes;
  const float scale = a.softmax_scale > 0.0f ? a.softmax_scale : 1.0f / sqrtf((float)a.d);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.cap_log2 = a.softcap * 1.4426950408889634f;
  p.inv_cap_scale = a.softcap > 0.0f ? scale / a.softcap : 0.0f;

  const uint32_t idesc_qk = make_idesc(a.q_fmt, a.kv_fmt, false, false, 128, 128);
  const uint32_t idesc_pv = make_idesc(RK_FMT_E4M3, a.kv_fmt, false, /*B MN-major*/ !kv6, 128, 128);
  dim3 grid(p.n_q_tiles * a.H * a.B, 1, 1);
  const bool cap = a.softcap > 0.0f;
  if (a.d <= 128) return launch_prefill2c(tq, tk, tv, p, idesc_qk, idesc_pv, cap, a.B, st);   // two query tiles per CTA
  if (p.dbg)      // the stage dump lives in instantiations of its own: the kernels that ship carry none of its code
    return cap ? launch_cfg<2, 2, true, true>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st)
               : launch_cfg<2, 2, false, true>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st);
  return cap ? launch_cfg<2, 2, true, false>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st)
             : launch_cfg<2, 2, false, false>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st);
}

}  // namespace rk
