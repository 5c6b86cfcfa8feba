// Split-KV decode attention over an MXFP8 KV cache on the 5th-generation tensor cores.
//
// Same semantics and same partial format as rk_decode.cu (prefill at S_q = 1, GQA head map
// kernels/flash_attention_mx_gqa/kernel.cpp:109-115; K and V decoded exactly, fp32 softmax state, no P
// requant in the reference sense), but the raw E4M3 bytes of K and V go from shared memory straight into
// tcgen05 block-scaled MMAs, so no thread ever converts a cache byte:
//
//   S^T[key][n]   = K_tile[128 keys x 128 d] . Qterms^T          A = K tile as TMA wrote it (K-major, SW128),
//                                                                scale-factor A = the tile's E8M0 key scales,
//                                                                B = the query heads as 2 MXFP8 terms each
//                                                                (q = hi + lo exactly: bf16 has 8 significant
//                                                                bits, an E4M3 term 4), N = 16
//   O^T[d][n]    += V_tile^T[128 d x 128 keys] . Pterms^T        A = V tile as TMA wrote it (MN-major), unit
//                                                                scales; B = P, per (head, 32-column group g of
//                                                                d, term): p * 2^(sv[key][g]) as 2 MXFP8 terms
//                                                                with one E8M0 scale per 32 keys, N = 32
//
// V's scale belongs to (key, 32-column group of d); a block-scaled MMA has one scale per (row, 32 keys), so the
// scale is folded into P: column (h, g) of B carries p[h][key] * 2^(sv[key][g] - svmax[g]) and its block scale
// carries svmax[g] (the largest V scale among the block's 32 keys) and the exponent of the block's largest p.
// Row d of O^T only uses the columns of its own group g = d / 32.
//
// One CTA = (batch, KV head, split): 4 worker warps (thread = key for S and P, thread = column d for O), one
// TMA warp, one MMA warp; a stage holds 128 keys.  The running maximum is CTA-wide per head; O is rescaled in
// TMEM only when a maximum grew by more than 2^8 since the last rescale (p stays below 2^8 in between, which the
// block scales absorb), so the common tile touches O not at all.
//
// Included by rk_decode.cu (one translation unit: both kernels share the combine kernel and the launcher).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

namespace dtc {
constexpr int kWorkers = 4;                       // worker warps
constexpr int kThreads = (kWorkers + 2) * 32;     // + TMA warp + MMA warp
constexpr int kTile = 128;                        // keys per stage
constexpr int kD = 128;
#ifndef RK_X_DTC_STAGES
#define RK_X_DTC_STAGES 3
#endif
constexpr int kStages = RK_X_DTC_STAGES;
constexpr int kCtasPerSm = kStages <= 3 ? 2 : 1;
constexpr int kMaxGrp = 8;                        // query heads per KV head handled by this kernel (HH = 4 or 8 rows of capacity)
constexpr int kNq = 16;                           // B rows of the QK^T MMA: term * HH + h (rows past 2 HH stay zero)
constexpr int kTileBytes = kTile * kD;            // 16384
constexpr int kStageBytes = 2 * kTileBytes + 2 * 512;   // K, V, K scales [128][4], V scales [128][4]
constexpr float kLazyLog2 = 8.0f;                 // rescale O when a running maximum grew by more than this

// Per head capacity HH: B rows of the PV MMA = term * 4 HH + h * 4 + g; with 8 heads one P buffer instead of two keeps
// the CTA inside the shared memory that lets two CTAs share an SM.
template <int HH> struct Lay {
  static constexpr int kNp = 8 * HH;
  static constexpr int kPBufs = HH == 4 ? 2 : 1;
  static constexpr int kPBytes = kNp * 128;       // one P tile: [kNp rows][128 B], K-major SW128
  // shared-memory map (offsets from a 1024-byte aligned base)
  static constexpr int stage_off = 0;
  static constexpr int p_off = kStages * kStageBytes;
  static constexpr int q_off = p_off + kPBufs * kPBytes;       // [16 rows][128 B], K-major SW128
  static constexpr int sfp_off = q_off + 2048;                 // 2 x 512-byte scale atoms for P
  static constexpr int sfq_off = sfp_off + 2 * 512;            // scale atom of the query terms
  static constexpr int one_off = sfq_off + 512;                // scale atom of ones (code 127) for V
  static constexpr int xchg_off = one_off + 512;               // [2][4 warps][8 heads] floats (tile maxima)
  static constexpr int bar_off = xchg_off + 2 * 32 * 4;
  static constexpr int misc_off = bar_off + 32 * 8;            // tmem base, abort flag
  static constexpr int total = misc_off + 16;
  static_assert(kStageBytes % 1024 == 0 && p_off % 1024 == 0 && q_off % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};
enum { bFull = 0, bEmpty = bFull + kStages, bSF = bEmpty + kStages, bSE = bSF + 2, bPF = bSE + 2, bPV = bPF + 2,
       bMX = bPV + 2, bDrain = bMX + 2, nBars = bDrain + 1 };
static_assert(nBars <= 32, "barrier slots");

// TMEM columns
constexpr uint32_t cS = 0;          // 2 x 16
constexpr uint32_t cO = 32;         // up to 64
constexpr uint32_t cSfK = 96;       // 4 per stage
constexpr uint32_t cSfQ = cSfK + 4 * kStages;
constexpr uint32_t cSfP = cSfQ + 4; // 2 x 4
constexpr uint32_t cSfOne = cSfP + 8;
constexpr uint32_t kTmemCols = 128;
static_assert(cSfOne + 4 <= kTmemCols, "TMEM map");
}  // namespace dtc

struct DecodeTcParams {
  const __nv_bfloat16* q;
  const uint8_t* k_scale;
  const uint8_t* v_scale;
  const int32_t* kv_len;
  float* part_o;    // [B*H][nsplit][128]
  float* part_ml;   // [B*H][nsplit][2]   (reference maximum in the log2 domain, l)
  int* status;
  int B, H, H_kv, L, grp, nsplit;
  float scale_log2;
};

// two fp32 -> two E4M3 codes, RNE, saturating: bits 15:8 = code(hi), bits 7:0 = code(lo)
RK_DEVINL uint32_t cvt_e4m3x2(float hi, float lo) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// the two codes back to fp32 (exact)
RK_DEVINL void e4m3x2_to_f32(uint32_t codes, float& hi, float& lo) {
  uint32_t h2;
  asm("{\n\t.reg .b16 c;\n\tcvt.u16.u32 c, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, c;\n\t}" : "=r"(h2) : "r"(codes));
  const __half2 v = *reinterpret_cast<const __half2*>(&h2);
  lo = __low2float(v);
  hi = __high2float(v);
}
RK_DEVINL uint32_t redux_max_u32(uint32_t v) {
  uint32_t r;
  asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
  return r;
}
// byte offset of (row n, byte x) in a K-major tile with 128-byte rows and the 128-byte swizzle
RK_DEVINL int sw128(int n, int x) { return n * 128 + ((((x >> 4) ^ (n & 7))) << 4) + (x & 15); }

// order-preserving map fp32 -> u32 (for integer max reductions) and back
RK_DEVINL uint32_t f32_to_ordered(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
RK_DEVINL float ordered_to_f32(uint32_t u) { return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u); }
// 2^e as fp32 for an integer e; below the normal range the result is 0, above it the largest power of two
RK_DEVINL float pow2i(int e) {
  const int f = e + 127;
  return __uint_as_float(f <= 0 ? 0u : ((uint32_t)(f > 254 ? 254 : f) << 23));
}

template <int HH>
__global__ void __launch_bounds__(dtc::kThreads, dtc::kCtasPerSm)
decode_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                 const DecodeTcParams p, const uint32_t idesc_qk, const uint32_t idesc_pv) {
  using namespace dtc;
  using L = Lay<HH>;
  extern __shared__ __align__(1024) uint8_t dtc_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dtc_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc_off + 4);
  float* xchg = reinterpret_cast<float*>(smem + L::xchg_off);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;   // an earlier launch gave up on a wait
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int bhkv = b * p.H_kv + hkv;
  const int len = p.kv_len ? min(max(p.kv_len[b], 0), p.L) : p.L;
  const int n_tiles_all = (len + kTile - 1) / kTile;
  const int tiles_per_split = (n_tiles_all + p.nsplit - 1) / p.nsplit;
  const int tile0 = split * tiles_per_split;
  const int n_tiles = max(0, min(n_tiles_all, tile0 + tiles_per_split) - tile0);
  const float NEG_INF = __int_as_float(0xff800000);

  // ---- set-up: barriers, TMEM, constant shared-memory regions, the query terms ------------------------------
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bEmpty + i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[bSF + i], 1); mbar_init(&bars[bSE + i], kWorkers); mbar_init(&bars[bPF + i], kWorkers);
      mbar_init(&bars[bPV + i], 1); mbar_init(&bars[bMX + i], kWorkers);
    }
    mbar_init(&bars[bDrain], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kWorkers + 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  if (warp < kWorkers) {
    const int t = threadIdx.x;                                    // 0..127
    // P tiles: rows of heads that do not exist stay zero for ever; scale atoms start as ones (code 127)
    for (int i = t; i < L::kPBufs * L::kPBytes / 16; i += 128) reinterpret_cast<uint4*>(smem + L::p_off)[i] = make_uint4(0u, 0u, 0u, 0u);
    for (int i = t; i < 2048 / 16; i += 128) reinterpret_cast<uint4*>(smem + L::sfp_off)[i] = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
    // rows of the query tile that no head writes below stay zero
    reinterpret_cast<uint4*>(smem + L::q_off)[t] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("bar.sync 1, 128;" ::: "memory");                  // fills done before the query terms land in them
    // query heads h = warp, warp + 4 as two MXFP8 terms each: q = hi + lo (lib/golden block rule on q, then on the residual)
#pragma unroll
    for (int h = warp; h < HH; h += kWorkers) {
      float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (h < p.grp) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p.q + ((size_t)b * p.H + hkv * p.grp + h) * kD + lane * 4);
        x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xFFFF0000u);
      }
#pragma unroll
      for (int term = 0; term < 2; ++term) {
        float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));   // the 8 lanes of one 32-wide block of d
        uint32_t code = 127u;
        float p2 = 1.0f;
        if (amax > 0.0f && amax < 3.0e38f) block_scale<0>(amax, code, p2);
        const float back = e8m0_to_f32(code);
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t c = encode_rne<0>(x[e] * p2);
          word |= c << (8 * e);
          x[e] -= decode_elem<0>(c) * back;                          // residual, exact
        }
        const int n = term * HH + h;
        *reinterpret_cast<uint32_t*>(smem + L::q_off + sw128(n, lane * 4)) = word;
        if ((lane & 7) == 0) smem[L::sfq_off + n * 16 + (lane >> 3)] = (uint8_t)code;
      }
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == kWorkers) {
    // ================= TMA producer =================
    if (lane == 0) {
      prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kStages;
        if (j >= kStages && !mbar_wait<20000>(&bars[bEmpty + st], ((j / kStages) - 1) & 1, abort_flag, p.status, 511)) break;
        uint8_t* sb = smem + L::stage_off + st * kStageBytes;
        const int key0 = (tile0 + j) * kTile;
        // scale rows past L are not read: the copy is clipped to the cache extent (L % 4 == 0 keeps it a 16-byte multiple)
        const uint32_t sbytes = (uint32_t)min(kTile, p.L - key0) * 4u;
        mbar_arrive_expect_tx(&bars[bFull + st], 2u * kTileBytes + 2u * sbytes);
        tma_load_3d(sb, &tmap_k, &bars[bFull + st], 0, key0, bhkv);
        tma_load_3d(sb + kTileBytes, &tmap_v, &bars[bFull + st], 0, key0, bhkv);
        bulk_load_1d(sb + 2 * kTileBytes, p.k_scale + ((size_t)bhkv * p.L + key0) * 4, sbytes, &bars[bFull + st]);
        bulk_load_1d(sb + 2 * kTileBytes + 512, p.v_scale + ((size_t)bhkv * p.L + key0) * 4, sbytes, &bars[bFull + st]);
      }
    }
  } else if (warp == kWorkers + 1) {
    // ================= MMA issuer (all lanes re-tile the key scales, lane 0 issues) =================
    const uint32_t q_addr = smem_u32(smem + L::q_off), p_addr = smem_u32(smem + L::p_off);
    auto issue_pv = [&](int i) -> bool {                            // lane 0 only
      const int buf = i & 1, sti = i % kStages;
      if (!mbar_wait(&bars[bPF + buf], (i >> 1) & 1, abort_flag, p.status, 523)) return false;
      tc_fence_after();
      tc_cp_32x128b_warpx4(tmem_base + cSfP + buf * 4, make_smem_desc(smem_u32(smem + L::sfp_off + buf * 512), 0, 128, kLayoutNone));
      const uint32_t v_addr = smem_u32(smem + L::stage_off + sti * kStageBytes + kTileBytes);
      const int pbuf = L::kPBufs == 2 ? buf : 0;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        // A = V tile [keys][d]: d is the contiguous (M) dimension, 32 keys per instruction
        const uint64_t adesc = make_smem_desc(v_addr + kk * 4096, kTileBytes, 1024, kLayoutSw128);
        const uint64_t bdesc = make_smem_desc(p_addr + pbuf * L::kPBytes + kk * 32, 16, 1024, kLayoutSw128);
        mma_mxf8f6f4_ss(tmem_base + cO, adesc, bdesc, idesc_with_sf(idesc_pv, kk, kk), tmem_base + cSfOne,
                        tmem_base + cSfP + buf * 4, (i > 0 || kk > 0) ? 1u : 0u);
      }
      tc_commit(&bars[bPV + buf]);
      tc_commit(&bars[bEmpty + sti]);
      return true;
    };
    if (lane == 0 && n_tiles > 0) {
      tc_cp_32x128b_warpx4(tmem_base + cSfQ, make_smem_desc(smem_u32(smem + L::sfq_off), 0, 128, kLayoutNone));
      tc_cp_32x128b_warpx4(tmem_base + cSfOne, make_smem_desc(smem_u32(smem + L::one_off), 0, 128, kLayoutNone));
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kStages;
      uint8_t* sb = smem + L::stage_off + st * kStageBytes;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars[bFull + st], (j / kStages) & 1, abort_flag, p.status, 521));
      if (!ok) break;
      // key scales [key][4] -> scale atom: word (key % 32) * 4 + key / 32
      uint32_t* ks = reinterpret_cast<uint32_t*>(sb + 2 * kTileBytes);
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) w[q] = ks[q * 32 + lane];
      __syncwarp();
      *reinterpret_cast<uint4*>(ks + lane * 4) = make_uint4(w[0], w[1], w[2], w[3]);
      fence_proxy_async_smem();
      __syncwarp();
      int good = 1;
      if (lane == 0) {
        tc_cp_32x128b_warpx4(tmem_base + cSfK + st * 4, make_smem_desc(smem_u32(ks), 0, 128, kLayoutNone));
        if (j >= 2 && !mbar_wait(&bars[bSE + (j & 1)], ((j - 2) >> 1) & 1, abort_flag, p.status, 522)) good = 0;
        if (good) {
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sb);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adesc = make_smem_desc(k_addr + kk * 32, 16, 1024, kLayoutSw128);
            const uint64_t bdesc = make_smem_desc(q_addr + kk * 32, 16, 1024, kLayoutSw128);
            mma_mxf8f6f4_ss(tmem_base + cS + (j & 1) * 16, adesc, bdesc, idesc_with_sf(idesc_qk, kk, kk),
                            tmem_base + cSfK + st * 4, tmem_base + cSfQ, kk > 0 ? 1u : 0u);
          }
          tc_commit(&bars[bSF + (j & 1)]);
          if (j >= 1 && !issue_pv(j - 1)) good = 0;
        }
      }
      ok = __shfl_sync(0xffffffffu, good, 0) != 0;
    }
    if (lane == 0 && n_tiles > 0) {
      if (ok) ok = issue_pv(n_tiles - 1);
      tc_commit(&bars[bDrain]);
      mbar_wait(&bars[bDrain], 0, abort_flag, p.status, 524);
    }
    __syncwarp();
  }
  else {
    // ================= workers: thread = key kt of the tile (S, P), thread = column d = kt (O) =================
    const int kt = warp * 32 + lane;
    const uint32_t lane_addr = ((uint32_t)(warp * 32)) << 16;
    float m_ref[HH], m_run[HH], l_part[HH];
#pragma unroll
    for (int h = 0; h < HH; ++h) { m_ref[h] = NEG_INF; m_run[h] = NEG_INF; l_part[h] = 0.0f; }

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1, st = j % kStages;
      uint8_t* sb = smem + L::stage_off + st * kStageBytes;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars[bSF + buf], (j >> 1) & 1, abort_flag, p.status, 501));
      if (!ok) break;
      tc_fence_after();
      uint32_t c[16];
      tmem_ld16(tmem_base + lane_addr + cS + buf * 16, c);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[bSE + buf]);

      const int key = (tile0 + j) * kTile + kt;
      const bool valid = key < len;
      const bool tail = (tile0 + j + 1) * kTile > len;
      float s[HH];
      float* xw = xchg + (buf * kWorkers + warp) * HH;
#pragma unroll
      for (int h = 0; h < HH; ++h) {
        s[h] = valid ? (__uint_as_float(c[h]) + __uint_as_float(c[HH + h])) * p.scale_log2 : NEG_INF;   // log2 domain
        const uint32_t wmax = redux_max_u32(f32_to_ordered(s[h]));
        if (lane == 0) xw[h] = ordered_to_f32(wmax);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[bMX + buf]);
      ok = __all_sync(0xffffffffu, mbar_wait(&bars[bMX + buf], (j >> 1) & 1, abort_flag, p.status, 504));
      if (!ok) break;
      float m_new[HH];
      // every thread of the CTA holds the same m_run / m_ref / m_new, so the decision below is CTA-uniform
      bool bump = (j == 0);
#pragma unroll
      for (int h = 0; h < HH; ++h) {
        const float* xr = xchg + buf * kWorkers * HH + h;
        m_new[h] = fmaxf(m_run[h], fmaxf(fmaxf(xr[0], xr[HH]), fmaxf(xr[2 * HH], xr[3 * HH])));
        bump = bump || (m_new[h] > m_ref[h] + kLazyLog2);
        m_run[h] = m_new[h];
      }
      if (bump) {
        if (j > 0) {
          // rescale O (this thread's row d = kt, all columns) once the previous PV has landed
          ok = __all_sync(0xffffffffu, mbar_wait(&bars[bPV + ((j - 1) & 1)], ((j - 1) >> 1) & 1, abort_flag, p.status, 502));
          if (!ok) break;
          tc_fence_after();
          float corr[HH];
#pragma unroll
          for (int h = 0; h < HH; ++h) { corr[h] = ex2_approx(m_ref[h] - m_new[h]); l_part[h] *= corr[h]; }
#pragma unroll
          for (int part = 0; part < L::kNp / 32; ++part) {
            uint32_t o[32];
            tmem_ld32(tmem_base + lane_addr + cO + part * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int n = 0; n < 32; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * corr[((part * 32 + n) % (4 * HH)) >> 2]);
            tmem_st32(tmem_base + lane_addr + cO + part * 32, o);
          }
          tc_wait_st();
        }
#pragma unroll
        for (int h = 0; h < HH; ++h) m_ref[h] = m_new[h];
      }

      // ---- p, row sums, block exponents -------------------------------------------------------------------
      float ph[HH];
      uint32_t eh[HH];     // biased exponent of the largest p of this warp's 32 keys, per head
      uint32_t emin = 255u, emax = 0u;
#pragma unroll
      for (int h = 0; h < HH; ++h) {
        const float pr = ex2_approx(s[h] - m_ref[h]);            // <= 2^8; masked keys give 0
        l_part[h] += pr;
        eh[h] = redux_max_u32(__float_as_uint(pr)) >> 23;
        ph[h] = pr * pow2i(134 - (int)eh[h]);
        emin = min(emin, eh[h]); emax = max(emax, eh[h]);
      }
      const uint32_t svw = valid ? *reinterpret_cast<const uint32_t*>(sb + 2 * kTileBytes + 512 + kt * 4) : 0u;
      uint32_t svmax[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) svmax[g] = redux_max_u32((svw >> (8 * g)) & 0xFFu);
      // element (h, g) = p * 2^(sv[g] - svmax[g]) * 2^(7 - (eh - 127)) <= 2^8 under the block scale code
      // svmax[g] + eh[h] - 134 (kept >= 4 so that the low term's code, 4 less, exists)
      float fg[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) fg[g] = pow2i((int)((svw >> (8 * g)) & 0xFFu) - (int)svmax[g]);
      const uint32_t smin = min(min(svmax[0], svmax[1]), min(svmax[2], svmax[3]));
      const uint32_t smax = max(max(svmax[0], svmax[1]), max(svmax[2], svmax[3]));
      const bool plain = (smin + emin >= 138u) && (smax + emax <= 388u);      // every code in [4, 254]

      // the P buffer is free once the PV that read it has completed: two tiles ago with two buffers, the last one with one
      if (j >= L::kPBufs) {
        const int i = j - L::kPBufs;
        ok = __all_sync(0xffffffffu, mbar_wait(&bars[bPV + (i & 1)], (i >> 1) & 1, abort_flag, p.status, 503));
        if (!ok) break;
      }
      uint8_t* pt = smem + L::p_off + (L::kPBufs == 2 ? buf : 0) * L::kPBytes;
#pragma unroll
      for (int h = 0; h < HH; ++h) {
#pragma unroll
        for (int g = 0; g < 4; g += 2) {
          float v0 = ph[h] * fg[g], v1 = ph[h] * fg[g + 1];
          if (!plain) {     // block scale code clamped: move the difference into the elements
            const int r0 = (int)svmax[g] + (int)eh[h] - 134, r1 = (int)svmax[g + 1] + (int)eh[h] - 134;
            v0 *= pow2i(r0 - min(max(r0, 4), 254));
            v1 *= pow2i(r1 - min(max(r1, 4), 254));
          }
          const uint32_t hi = cvt_e4m3x2(v1, v0);
          float a1, a0;
          e4m3x2_to_f32(hi, a1, a0);
          const uint32_t lo = cvt_e4m3x2((v1 - a1) * 16.0f, (v0 - a0) * 16.0f);
          const int n = h * 4 + g;
          pt[sw128(n, kt)] = (uint8_t)hi;
          pt[sw128(n + 1, kt)] = (uint8_t)(hi >> 8);
          pt[sw128(4 * HH + n, kt)] = (uint8_t)lo;
          pt[sw128(4 * HH + n + 1, kt)] = (uint8_t)(lo >> 8);
        }
      }
#pragma unroll
      for (int part = 0; part < L::kNp / 32; ++part) {   // block scale of column n for this warp's 32 keys (k-block = warp)
        const int n = part * 32 + lane;
        const int term = n / (4 * HH), hh = (n >> 2) % HH, gg = n & 3;
        const uint32_t sv_s = gg == 0 ? svmax[0] : gg == 1 ? svmax[1] : gg == 2 ? svmax[2] : svmax[3];
        uint32_t eh_s = eh[0];
#pragma unroll
        for (int h = 1; h < HH; ++h) eh_s = (hh == h) ? eh[h] : eh_s;
        const int code = min(max((int)sv_s + (int)eh_s - 134, 4), 254) - 4 * term;
        smem[L::sfp_off + buf * 512 + (n & 31) * 16 + (n >> 5) * 4 + warp] = (uint8_t)code;
      }
      if (tail && !valid) {   // a key past kv_len: its V row may hold anything; 0 * NaN must not reach the accumulator
        uint4* vrow = reinterpret_cast<uint4*>(sb + kTileBytes + kt * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) vrow[i] = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[bPF + buf]);
    }

    // ---- epilogue: O^T row d = kt, the columns of group g = warp -------------------------------------------
    float oh[HH];
#pragma unroll
    for (int h = 0; h < HH; ++h) oh[h] = 0.0f;
    if (ok && n_tiles > 0) {
      const int last = n_tiles - 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars[bPV + (last & 1)], (last >> 1) & 1, abort_flag, p.status, 505));
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int part = 0; part < L::kNp / 32; ++part) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_addr + cO + part * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int n = 0; n < 32; ++n) {
            const int col = part * 32 + n;                       // = term * 4 HH + h * 4 + g: both terms add up
            if ((col & 3) == warp) oh[(col % (4 * HH)) >> 2] += __uint_as_float(o[n]);
          }
        }
      }
    }
    float* lsum = reinterpret_cast<float*>(smem + L::p_off);        // [HH heads][128 threads]: the P tiles are free now
#pragma unroll
    for (int h = 0; h < HH; ++h) lsum[h * 128 + kt] = l_part[h];
    asm volatile("bar.sync 1, 128;" ::: "memory");                  // workers only; every worker reaches this point
    if (ok) {
#pragma unroll
      for (int h = 0; h < HH; ++h) {
        if (h < p.grp) {
          const size_t bh = (size_t)b * p.H + hkv * p.grp + h;
          p.part_o[(bh * p.nsplit + split) * 128 + kt] = oh[h];
        }
      }
      if (kt < p.grp) {
        float l = 0.0f;
        for (int i = 0; i < 128; ++i) l += lsum[kt * 128 + i];
        float mr = m_ref[0];
#pragma unroll
        for (int h = 1; h < HH; ++h) mr = (kt == h) ? m_ref[h] : mr;
        const size_t bh = (size_t)b * p.H + hkv * p.grp + kt;
        p.part_ml[(bh * p.nsplit + split) * 2] = mr;
        p.part_ml[(bh * p.nsplit + split) * 2 + 1] = l;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == dtc::kWorkers + 1) { tc_fence_after(); tmem_dealloc(tmem_base, dtc::kTmemCols); }
}

}  // namespace rk
