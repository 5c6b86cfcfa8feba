// MX flash-attention prefill, two 128-row query tiles per CTA (head dim <= 128).
//
// Same stages as rk_prefill.cu (TMA -> tcgen05 block-scaled QK^T -> fp32 online softmax
// -> P re-quantized to E4M3/E8M0 per 32 keys -> block-scaled PV into TMEM), following
// fa_entry, kernels/flash_attention_mx_gqa/kernel.cpp:91-184.  What differs is the
// schedule: the tile loop of one query tile is a chain of latencies (S ready -> TMEM
// load -> row max -> exp/requant -> P visible -> PV -> O rescale), so a CTA now carries
// two independent query tiles, "A" and "B", each with its own 8 softmax warps, O
// accumulator, P buffers and barriers.  While one group waits on a latency the other
// one computes, and every K/V tile brought in by TMA serves both (half the L2 traffic).
// The S accumulator in TMEM is shared: a group copies its S rows to registers at once and
// hands the columns back, so the MMA warp alternates QK_A, QK_B on one 128-column region.
//
// 576 threads: warps 0-7 softmax of tile A, 8-15 softmax of tile B (two threads per row,
// 64 keys each), warp 16 TMA producer, warp 17 MMA issuer + TMEM allocation.
#include "rk_prefill.cuh"

namespace rk {

namespace q2 {
constexpr int kStages = 3;
constexpr int kGroupWarps = 8;
constexpr int kThreads = (2 * kGroupWarps + 2) * 32;
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
              bPF = 17 /* + g*2+pb */, bPV = 21 /* + g*2+pb */, bPAIR = 25 /* + g*4+quad */, bDRAIN = 33, nBars = 34;
constexpr int misc_off = bar_off + nBars * 8;
constexpr int xchg_off = misc_off + 16;                    // [2 groups][3][2 halves][128] floats
constexpr int total = xchg_off + 2 * 3 * 2 * 128 * 4;
}  // namespace q2

template <bool SOFTCAP>
__device__ __forceinline__ void softmax_group(const PrefillParams& p, uint8_t* smem, uint64_t* bars, uint32_t tmem_base,
                                              volatile int* abort_flag, int grp, int qt, int bh, int n_tiles, int j0) {
  using namespace q2;
  uint64_t* s_full = bars + bSF + grp;
  uint64_t* s_empty = bars + bSE + grp;
  uint64_t* p_full = bars + bPF + grp * 2;
  uint64_t* pv_done = bars + bPV + grp * 2;
  uint64_t* pair = bars + bPAIR + grp * 4;
  float* xchg = reinterpret_cast<float*>(smem + xchg_off) + grp * (3 * 2 * 128);

  const int gwarp = (threadIdx.x >> 5) - grp * kGroupWarps;   // 0..7 within the group
  const int lane = threadIdx.x & 31;
  const int quad = gwarp & 3, half = gwarp >> 2;
  const int row = quad * 32 + lane;
  const uint32_t lane_addr = ((uint32_t)(quad * 32)) << 16;
  const int q_row = qt * kBlockM + row;
  const int q_pos = p.q_pos0 + q_row;
  const float NEG_INF = __int_as_float(0xff800000);
  const bool dump = p.dbg && qt == p.n_q_tiles - 1 && bh == 0;
  const uint32_t o_col = cO + grp * 128 + half * 64;         // this thread's 64 columns of O

  float m_run = NEG_INF, l_run = 0.0f;
  bool ok = true;

  for (int j = 0; j < n_tiles && ok; ++j) {
    const int pb = j & 1;
    const int sslot = (gwarp == 0) ? grp : 7;
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 0);
    ok = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1, abort_flag, p.status, 101));
    if (!ok) break;
    tc_fence_after();
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 1);

    float s[64];
    tmem_ld32(tmem_base + lane_addr + cS + half * 64, reinterpret_cast<uint32_t*>(s));
    tmem_ld32(tmem_base + lane_addr + cS + half * 64 + 32, reinterpret_cast<uint32_t*>(s) + 32);
    tc_wait_ld();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(s_empty);       // hand the S columns back: the other query tile's QK^T may use them
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 2);

    if (dump && j == 0) {
#pragma unroll
      for (int c = 0; c < 64; ++c) p.dbg[row * 128 + half * 64 + c] = s[c];
    }

    // ---- (soft-cap,) mask, block maxima ----------------------------------------------------------------
    const int key0 = (j + j0) * kBlockN;                      // first key of this tile (j counts from the first tile inside the window)
    const bool tail = (key0 + kBlockN > p.S_kv);
    const bool diag = p.causal && (key0 + kBlockN - 1 > p.q_pos0 + qt * kBlockM);
    const bool need_mask = tail || diag || (p.window > 0);
    if (SOFTCAP) {
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float e = ex2_approx(s[c] * (2.0f * 1.4426950408889634f * p.inv_cap_scale));
        s[c] = p.cap_log2 * fmaf(-2.0f, rcp_approx(1.0f + e), 1.0f);
      }
    }
    if (need_mask) {
      const int kb = key0 + half * 64;
      int hi = p.S_kv - 1 - kb;                               // masked iff c > hi || c <= lo
      if (p.causal) hi = min(hi, q_pos - kb);
      const int lo = (p.window > 0) ? (q_pos - p.window - kb) : -1;
#pragma unroll
      for (int c = 0; c < 64; ++c) s[c] = (c > hi || c <= lo) ? NEG_INF : s[c];
    }
    float bmax[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      float a0 = fmax3(s[g * 32 + 0], s[g * 32 + 1], s[g * 32 + 2]);
      float a1 = fmax3(s[g * 32 + 3], s[g * 32 + 4], s[g * 32 + 5]);
#pragma unroll
      for (int c = 6; c < 30; c += 4) { a0 = fmax3(a0, s[g * 32 + c], s[g * 32 + c + 1]); a1 = fmax3(a1, s[g * 32 + c + 2], s[g * 32 + c + 3]); }
      bmax[g] = fmax3(a0, a1, fmaxf(s[g * 32 + 30], s[g * 32 + 31]));
    }
    float mx = fmaxf(bmax[0], bmax[1]);
    // the other 64 keys of the row belong to the partner warp of this lane quadrant
    xchg[(pb * 2 + half) * 128 + row] = mx;
    __syncwarp();
    if (lane == 0) mbar_arrive(&pair[quad]);
    ok = __all_sync(0xffffffffu, mbar_wait(&pair[quad], j & 1, abort_flag, p.status, 104));
    if (!ok) break;
    mx = fmaxf(mx, xchg[(pb * 2 + (half ^ 1)) * 128 + row]);
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 3);
    const float sc_mul = SOFTCAP ? 1.0f : p.scale_log2;
    const float m_new = fmaxf(m_run, mx * sc_mul);
    // exponent = fma(s, scale, -m): lowering m by 2^-21 |m| keeps the row-max p in [1, 1 + 1e-5) in spite of
    // the rounding residue of s*scale; the common factor cancels in O = sum(p v) / sum(p).
    const float m_use = (m_new == NEG_INF) ? 0.0f : (SOFTCAP ? m_new : fmaf(-fabsf(m_new), 4.76837158203125e-7f, m_new));
    const float corr = (m_run == NEG_INF) ? 1.0f : ex2_approx(m_run - m_new);
    m_run = m_new;

    // ---- p = 2^(x - m), row sum from the unquantised p, requant per 32-key block ---------------------
    uint8_t* p_tile = smem + p_off + (grp * 2 + pb) * kTileBytes + row * 128;
    float ls0 = 0.0f, ls1 = 0.0f, ls2 = 0.0f, ls3 = 0.0f;
    uint32_t scale_half = 0;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        float x0, x1, x2, x3;
        fma2(s[g * 32 + c + 0], s[g * 32 + c + 1], sc_mul, -m_use, x0, x1);
        fma2(s[g * 32 + c + 2], s[g * 32 + c + 3], sc_mul, -m_use, x2, x3);
        const float p0 = ex2_approx(x0), p1 = ex2_approx(x1), p2 = ex2_approx(x2), p3 = ex2_approx(x3);
        s[g * 32 + c + 0] = p0; s[g * 32 + c + 1] = p1; s[g * 32 + c + 2] = p2; s[g * 32 + c + 3] = p3;
        add2(ls0, ls1, p0, p1);
        add2(ls2, ls3, p2, p3);
      }
      const float pmax = ex2_approx(fmaf(bmax[g], sc_mul, -m_use));   // p of the block's arg-max element
      int sc = (int)(__float_as_uint(pmax) >> 23);                    // E8M0 code: se = floor(log2 pmax) <= 0
      sc = min(sc, 127);
      scale_half |= (uint32_t)sc << (8 * g);
      uint32_t w[8];
      if (sc >= 7) {
        // y = p * 2^(7-sc): exponent field = E4M3 exponent field, mantissa kept, so the truncated code is
        // y's bits [20,27); .ftz zeroes everything below 2^-6 of the block scale.
        const float f = __uint_as_float((uint32_t)(134 - sc) << 23);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float y0, y1, y2, y3;
          mul2_ftz(s[g * 32 + q * 4 + 0], s[g * 32 + q * 4 + 1], f, y0, y1);
          mul2_ftz(s[g * 32 + q * 4 + 2], s[g * 32 + q * 4 + 3], f, y2, y3);
          w[q] = pack_u8x2(__float_as_uint(y1) >> 20, __float_as_uint(y0) >> 20,
                           pack_u8x2(__float_as_uint(y3) >> 20, __float_as_uint(y2) >> 20, 0u));
        }
      } else {
        const int sub = (sc - 7) * 8;                                 // block max below 2^-120: exact integer form
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint32_t word = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t bits = __float_as_uint(s[g * 32 + q * 4 + e]);
            int t = (int)(bits >> 20) - sub;
            t = (t >= 8 && bits >= 0x00800000u) ? t : 0;
            word |= (uint32_t)t << (8 * e);
          }
          w[q] = word;
        }
      }
      const int blk = half * 2 + g;
      const int c0 = (2 * blk) ^ (row & 7), c1 = (2 * blk + 1) ^ (row & 7);     // 128-byte swizzle
      *reinterpret_cast<uint4*>(p_tile + c0 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(p_tile + c1 * 16) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    l_run = l_run * corr + ((ls0 + ls1) + (ls2 + ls3));
    *reinterpret_cast<uint16_t*>(smem + sfp_off + (grp * 2 + pb) * kSfAtomBytes + (row & 31) * 16 + (row >> 5) * 4 + half * 2) =
        (uint16_t)scale_half;

    if (dump && j == 0) {
      uint32_t* d32 = reinterpret_cast<uint32_t*>(p.dbg + 128 * 128);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int lc = half * 4 + c;
        const uint4 v4 = *reinterpret_cast<const uint4*>(p_tile + ((lc ^ (row & 7)) * 16));
        d32[row * 32 + lc * 4 + 0] = v4.x; d32[row * 32 + lc * 4 + 1] = v4.y;
        d32[row * 32 + lc * 4 + 2] = v4.z; d32[row * 32 + lc * 4 + 3] = v4.w;
      }
      reinterpret_cast<uint16_t*>(d32 + 128 * 32)[row * 2 + half] = (uint16_t)scale_half;
    }
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 4);

    // ---- rescale this thread's half of O once the previous PV has landed ---------------------------------
    if (j > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, 102));
      if (!ok) break;
      tc_fence_after();
      if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_addr + o_col + ch * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) mul2_ftz_inplace(r[i], r[i + 1], corr);
          tmem_st32(tmem_base + lane_addr + o_col + ch * 32, r);
        }
        tc_wait_st();
      }
    }
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 5);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&p_full[pb]);
    if (lane == 0 && sslot < 2) RK_STAMP(sslot, j, 6);
  }

  // ---- epilogue --------------------------------------------------------------------------------------------
  float l_tot = l_run;
  if (ok) {
    xchg[(2 * 2 + half) * 128 + row] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(&pair[quad]);
    ok = __all_sync(0xffffffffu, mbar_wait(&pair[quad], n_tiles & 1, abort_flag, p.status, 105));
    if (ok) l_tot += xchg[(2 * 2 + (half ^ 1)) * 128 + row];
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
    const int ncols = p.d / 2;                      // 32 or 64 output columns per thread
    if (dump && half == 0) {
      p.dbg[128 * 128 + 128 * 32 + 128 + row * 2 + 0] = m_run;
      p.dbg[128 * 128 + 128 * 32 + 128 + row * 2 + 1] = l_tot;
    }
#pragma unroll 1
    for (int c16 = 0; c16 < ncols / 16; ++c16) {
      uint32_t r[16];
      const int col0 = half * ncols + c16 * 16;
      tmem_ld16(tmem_base + lane_addr + cO + grp * 128 + col0, r);
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
    if (p.lse && live && half == 0)
      p.lse[(size_t)bh * p.S_q + q_row] = (l_tot > 0.0f) ? m_run * 0.6931471805599453f + logf(l_tot) : NEG_INF;
  }
  tc_fence_before();
}

template <bool SOFTCAP>
__global__ void __launch_bounds__(q2::kThreads, 1)
prefill2q_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p, const uint32_t idesc_qk,
                 const uint32_t idesc_pv) {
  using namespace q2;
  extern __shared__ __align__(1024) uint8_t smem_raw2[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw2) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + bar_off);
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc_off + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;   // an earlier launch gave up on a wait
  const int n_pairs = (p.n_q_tiles + 1) / 2;
  // Work order over the 1-D grid: (batch, head) pairs are taken in groups of p.head_group; inside a group the
  // heaviest (latest) query-tile pairs of all its heads come first and the lightest last, so the grid ends on
  // short CTAs (measured on B8 H16 S4096: 9 % faster than head after head), while a group's K/V still fits in L2.
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

  if (threadIdx.x == 0) {
    mbar_init(&bars[bQ], 1);
    for (int i = 0; i < kStages; ++i) { mbar_init(&bars[bKF + i], 1); mbar_init(&bars[bKE + i], 1); mbar_init(&bars[bVF + i], 1); mbar_init(&bars[bVE + i], 1); }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&bars[bSF + g], 1); mbar_init(&bars[bSE + g], kGroupWarps);
      for (int i = 0; i < 2; ++i) { mbar_init(&bars[bPF + g * 2 + i], kGroupWarps); mbar_init(&bars[bPV + g * 2 + i], 1); }
      for (int i = 0; i < 4; ++i) mbar_init(&bars[bPAIR + g * 4 + i], 2);
    }
    mbar_init(&bars[bDRAIN], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 2 * kGroupWarps + 1) { tmem_alloc(tmem_ptr, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp < 2 * kGroupWarps) {
    const int grp = warp / kGroupWarps;
    const int qt = 2 * qp + grp;
    if (nt[grp] > 0) {
      softmax_group<SOFTCAP>(p, smem, bars, tmem_base, abort_flag, grp, qt, bh, nt[grp], j0);
    } else if (qt < p.n_q_tiles) {
      // no visible key: O = 0 (the l <= 0 guard of finalize_O, kernels/flash_attention_mx_gemma/flash_mx_impl.hpp:554-560)
      const int t = threadIdx.x - grp * kGroupWarps * 32;
      if (t < 128) {
        const int q_row = qt * kBlockM + t;
        if (q_row < p.S_q) {
          __nv_bfloat16* orow = p.o + ((size_t)bh * p.S_q + q_row) * p.d;
          for (int c = 0; c < p.d; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
          if (p.lse) p.lse[(size_t)bh * p.S_q + q_row] = __int_as_float(0xff800000);
        }
      }
    }
  } else if (warp == 2 * kGroupWarps) {
    // ================= TMA producer =================
    if (lane == 0 && n_all > 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      const int nq = (2 * qp + 1 < p.n_q_tiles) ? 2 : 1;
      mbar_arrive_expect_tx(&bars[bQ], nq * (p.q_tile_tx + kSfAtomBytes));
      for (int g = 0; g < nq; ++g) {
        tma_load_3d(smem + q_off + g * kTileBytes, &tmap_q, &bars[bQ], 0, (2 * qp + g) * kBlockM, bh);
        bulk_load_1d(smem + sfq_off + g * kSfAtomBytes, p.q_sf + ((size_t)bh * p.n_q_tiles + 2 * qp + g) * kSfAtomBytes,
                     kSfAtomBytes, &bars[bQ]);
      }
      bool ok = true;
      for (int j = 0; j < n_all && ok; ++j) {
        const int st = j % kStages, use = j / kStages;
        if (use > 0) ok = mbar_wait(&bars[bKE + st], (use - 1) & 1, abort_flag, p.status, 201);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[bKF + st], p.kv_tile_tx + kSfAtomBytes);
        tma_load_3d(smem + k_off + st * kTileBytes, &tmap_k, &bars[bKF + st], 0, (j + j0) * kBlockN, bhkv);
        bulk_load_1d(smem + sfk_off + st * kSfAtomBytes, p.k_sf + ((size_t)bhkv * p.n_kv_tiles + j + j0) * kSfAtomBytes,
                     kSfAtomBytes, &bars[bKF + st]);
        if (use > 0) ok = mbar_wait(&bars[bVE + st], (use - 1) & 1, abort_flag, p.status, 202);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[bVF + st], p.kv_tile_tx + kSfAtomBytes);
        if (p.v_transposed) tma_load_3d(smem + v_off + st * kTileBytes, &tmap_v, &bars[bVF + st], (j + j0) * kBlockN, 0, bhkv);
        else tma_load_3d(smem + v_off + st * kTileBytes, &tmap_v, &bars[bVF + st], 0, (j + j0) * kBlockN, bhkv);
        bulk_load_1d(smem + sfv_off + st * kSfAtomBytes, p.v_sf + ((size_t)bhkv * p.n_kv_tiles + j + j0) * kSfAtomBytes,
                     kSfAtomBytes, &bars[bVF + st]);
      }
    }
  } else {
    // ================= MMA issuer =================
    if (lane == 0 && n_all > 0) {
      const uint32_t q_addr = smem_u32(smem + q_off), k_addr = smem_u32(smem + k_off);
      const uint32_t v_addr = smem_u32(smem + v_off), pt_addr = smem_u32(smem + p_off);
      bool ok = mbar_wait(&bars[bQ], 0, abort_flag, p.status, 301);
      if (ok) {
        for (int g = 0; g < 2; ++g)
          tc_cp_32x128b_warpx4(tmem_base + cSfQ + g * 4, make_smem_desc(smem_u32(smem + sfq_off + g * kSfAtomBytes), 0, 128, kLayoutNone));
      }
      int s_user_g = -1, s_user_j = 0;       // who read the shared S columns last
      auto issue_qk = [&](int g, int j, int st) -> bool {
        if (s_user_g >= 0 && !mbar_wait(&bars[bSE + s_user_g], s_user_j & 1, abort_flag, p.status, 305)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t adesc = make_smem_desc(q_addr + g * kTileBytes + kk * 32, 16, 1024, kLayoutSw128);
          const uint64_t bdesc = make_smem_desc(k_addr + st * kTileBytes + kk * 32, 16, 1024, kLayoutSw128);
          mma_mxf8f6f4_ss(tmem_base + cS, adesc, bdesc, idesc_with_sf(idesc_qk, kk, kk), tmem_base + cSfQ + g * 4,
                          tmem_base + cSfK + st * 4, kk > 0 ? 1u : 0u);
        }
        tc_commit(&bars[bSF + g]);
        s_user_g = g; s_user_j = j;
        return true;
      };
      auto issue_pv = [&](int g, int i, bool first_of_tile, bool last_of_tile) -> bool {
        const int pb = i & 1, st = i % kStages, use = i / kStages;
        if (first_of_tile) {
          if (!mbar_wait(&bars[bVF + st], use & 1, abort_flag, p.status, 303)) return false;
          tc_cp_32x128b_warpx4(tmem_base + cSfV + st * 4, make_smem_desc(smem_u32(smem + sfv_off + st * kSfAtomBytes), 0, 128, kLayoutNone));
        }
        if (!mbar_wait(&bars[bPF + g * 2 + pb], (i >> 1) & 1, abort_flag, p.status, 304)) return false;
        tc_fence_after();
        tc_cp_32x128b_warpx4(tmem_base + cSfP + (g * 2 + pb) * 4,
                             make_smem_desc(smem_u32(smem + sfp_off + (g * 2 + pb) * kSfAtomBytes), 0, 128, kLayoutNone));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t adesc = make_smem_desc(pt_addr + (g * 2 + pb) * kTileBytes + kk * 32, 16, 1024, kLayoutSw128);
          // V tile [keys][d] is the MN-major B operand; a 6-bit V is stored transposed and is K-major like K
          const uint64_t bdesc = p.v_transposed ? make_smem_desc(v_addr + st * kTileBytes + kk * 32, 16, 1024, kLayoutSw128)
                                                : make_smem_desc(v_addr + st * kTileBytes + kk * 4096, kTileBytes, 1024, kLayoutSw128);
          mma_mxf8f6f4_ss(tmem_base + cO + g * 128, adesc, bdesc, idesc_with_sf(idesc_pv, kk, kk),
                          tmem_base + cSfP + (g * 2 + pb) * 4, tmem_base + cSfV + st * 4, (i > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&bars[bPV + g * 2 + pb]);
        if (last_of_tile) tc_commit(&bars[bVE + st]);
        return true;
      };
      // PVs of tile i: group 0 first, then group 1; flags tell which one opens / closes the V stage
      auto pv_flags = [&](int g, int i, bool& first, bool& last) {
        const bool a = i < nt[0], bb = i < nt[1];
        first = (g == 0) ? true : !a;
        last = (g == 1) ? true : !bb;
      };
      for (int j = 0; j < n_all && ok; ++j) {
        const int st = j % kStages, use = j / kStages;
        ok = mbar_wait(&bars[bKF + st], use & 1, abort_flag, p.status, 302);
        if (!ok) break;
        tc_cp_32x128b_warpx4(tmem_base + cSfK + st * 4, make_smem_desc(smem_u32(smem + sfk_off + st * kSfAtomBytes), 0, 128, kLayoutNone));
        bool f, l;
        if (j < nt[0]) ok = issue_qk(0, j, st);
        if (ok && j > 0 && j - 1 < nt[0]) { pv_flags(0, j - 1, f, l); ok = issue_pv(0, j - 1, f, l); }
        if (ok && j < nt[1]) ok = issue_qk(1, j, st);
        if (ok) tc_commit(&bars[bKE + st]);
        if (ok && j > 0 && j - 1 < nt[1]) { pv_flags(1, j - 1, f, l); ok = issue_pv(1, j - 1, f, l); }
      }
      if (ok) {
        bool f, l;
        const int i = n_all - 1;
        if (i < nt[0]) { pv_flags(0, i, f, l); ok = issue_pv(0, i, f, l); }
        if (ok && i < nt[1]) { pv_flags(1, i, f, l); ok = issue_pv(1, i, f, l); }
      }
      tc_commit(&bars[bDRAIN]);
      mbar_wait(&bars[bDRAIN], 0, abort_flag, p.status, 306);
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2 * kGroupWarps + 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

template <bool SOFTCAP>
static int launch2q_cfg(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                        uint32_t idesc_qk, uint32_t idesc_pv, dim3 grid, cudaStream_t st) {
  const int smem_bytes = q2::total + 1024;
  auto kern = prefill2q_kernel<SOFTCAP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_before, st);
  kern<<<grid, q2::kThreads, smem_bytes, st>>>(tq, tk, tv, p, idesc_qk, idesc_pv);
  if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_after, st);
  return (int)cudaGetLastError();
}

int launch_prefill2q(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                     uint32_t idesc_qk, uint32_t idesc_pv, bool softcap, int B, cudaStream_t st) {
  dim3 grid(((p.n_q_tiles + 1) / 2) * p.H * B, 1, 1);
  return softcap ? launch2q_cfg<true>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st)
                 : launch2q_cfg<false>(tq, tk, tv, p, idesc_qk, idesc_pv, grid, st);
}

}  // namespace rk
