// Split-KV decode attention over an MXFP8 KV cache (one query token per
// sequence, GQA), HBM-bound: every byte of K/V codes and scales is read once.
//
// No decode attention kernel exists in the reference; the semantics are its
// prefill path (kernels/flash_attention_mx_gqa/kernel.cpp:91-184) at S_q = 1
// with the GQA head map h -> h / grp (:109-115): K and V decoded exactly, fp32
// softmax state, no P requant.
//
// Work unit = (batch, KV head, split of the keys).  The `grp` query heads that
// share a KV head are the M rows of the tensor-core tiles, so K and V are
// streamed once per group.  Per CTA, 4 consumer warps + 1 TMA warp; a stage holds 128 keys (K 16 KB +
// V 16 KB as 128-byte-swizzled TMA tiles, plus 2 x 512 B of E8M0 scales); each
// warp owns 32 keys of a stage and keeps private (m, l, O) state that is merged
// through shared memory at the end.  Partials (m, l, O) go to the workspace and
// a second kernel does the log-sum-exp combine.
//
// Math per warp and 16 keys (legacy mma.sync: the kernel is memory bound, the
// tensor pipe only has to keep up with HBM):
//   S[head][key]  = sum over the 4 scale blocks of d: 2^(sk-127) * (Q . K_codes)   m16n8k16 f16
//                   (E4M3 -> f16 is exact; Q is pre-scaled per head by a power of two into f16 range)
//   O[head][d]   += (P * 2^(sv-vref)) . V_codes                                    m16n8k16 bf16
//                   (E4M3 -> bf16 by bit placement, exact up to a 2^120 factor folded into P; vref is the warp's
//                   running reference V scale code, at least 127 and at least every code seen so far: when a larger
//                   code turns up the accumulator is rescaled by the exact power of two, like the running maximum,
//                   so no V scale code can overflow the folded factor)
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32 + 32;   // 4 consumer warps + 1 TMA producer warp
constexpr int kDecTileKeys = 128;
constexpr int kDecStages = 3;
constexpr int kDecD = 128;
constexpr int kDecStageBytes = 2 * kDecTileKeys * kDecD + 2 * kDecTileKeys * 4;   // K, V, K scales, V scales
constexpr int kDecSmemBytes = kDecStages * kDecStageBytes + 64 + 1024;

struct DecodeParams {
  const __nv_bfloat16* q;
  const uint8_t* k_scale;
  const uint8_t* v_scale;
  const int32_t* kv_len;
  float* part_o;    // [B*H][nsplit][128]
  float* part_ml;   // [B*H][nsplit][2]   (m in log2 domain, l)
  int* status;
  int B, H, H_kv, L, grp, nsplit;
  float scale_log2;
};

RK_DEVINL void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
RK_DEVINL void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// E8M0 byte `blk` of the packed scale word -> 2^(code-127) as fp32 (code 0 -> 0: such a block holds zeros only)
RK_DEVINL float e8m0_byte_to_f32(uint32_t word, int blk) {
  const uint32_t sh = blk < 3 ? (word << (23 - 8 * blk)) : (word >> 1);
  return __uint_as_float(sh & 0x7F800000u);
}
// Element formats of the cache, one code per byte (FMT = RK_FMT_*).  EB / MB: exponent and mantissa bits; F = 127 - bias.
template <int FMT> struct DecFmt;
template <> struct DecFmt<0> { static constexpr int EB = 4, MB = 3, F = 120; };   // E4M3
template <> struct DecFmt<1> { static constexpr int EB = 5, MB = 2, F = 112; };   // E5M2
template <> struct DecFmt<2> { static constexpr int EB = 2, MB = 3, F = 126; };   // E2M3
template <> struct DecFmt<3> { static constexpr int EB = 3, MB = 2, F = 124; };   // E3M2
template <> struct DecFmt<4> { static constexpr int EB = 2, MB = 1, F = 126; };   // E2M1
// four codes of a word -> f16x2 of codes 0,1 (HI = false) or 2,3 (HI = true), exact: one hardware conversion per
// pair.  An E2M1 code (s ee m) is the E2M3 code (s ee m00) of the same value.
template <int FMT, bool HI> RK_DEVINL uint32_t codes_to_f16x2(uint32_t x) {
  uint32_t r;
  if (FMT == 4) x = ((x & 0x08080808u) << 2) | ((x & 0x07070707u) << 2);
  if (FMT == 0) {
    if (HI) asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, hi;\n\t}" : "=r"(r) : "r"(x));
    else    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(x));
  } else if (FMT == 1) {
    if (HI) asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e5m2x2 %0, hi;\n\t}" : "=r"(r) : "r"(x));
    else    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e5m2x2 %0, lo;\n\t}" : "=r"(r) : "r"(x));
  } else if (FMT == 3) {
    if (HI) asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e3m2x2 %0, hi;\n\t}" : "=r"(r) : "r"(x));
    else    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e3m2x2 %0, lo;\n\t}" : "=r"(r) : "r"(x));
  } else {
    if (HI) asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e2m3x2 %0, hi;\n\t}" : "=r"(r) : "r"(x));
    else    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e2m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(x));
  }
  return r;
}
// z holds two codes in bytes 1 and 3 (bytes 0 and 2 arbitrary): each code c becomes the bf16 whose exponent
// field starts with c's exponent field and whose mantissa starts with c's mantissa, i.e. value(c) * 2^-F
// (normals and subnormals alike; for E4M3: sign | (c & 0x7F) << 4).
template <int FMT> RK_DEVINL uint32_t hi_bytes_to_bf16x2_scaled(uint32_t z) {
  using D = DecFmt<FMT>;
  constexpr uint32_t kMag = (((1u << (D::EB + D::MB)) - 1u) << 8) * 0x00010001u;
  const uint32_t mag = (z & kMag) >> (D::MB + 1);
  const uint32_t sgn = z << (7 - D::EB - D::MB);          // the sign bit to bit 15 of its half
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(sgn), "r"(0x80008000u), "r"(mag));   // (sgn & C) | mag
  return r;
}
RK_DEVINL uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel)); return r;
}
RK_DEVINL uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
RK_DEVINL uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}
// two E8M0 codes (bytes 0,1 of x) -> bf16x2 of 2^(code-127)
RK_DEVINL uint32_t ue8m0x2_to_bf16x2(uint32_t x) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.bf16x2.ue8m0x2 %0, lo;\n\t}" : "=r"(r) : "r"(x));
  return r;
}

template <int FMT>
__global__ void __launch_bounds__(kDecThreads, 2)
decode_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, const DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t dsmem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dsmem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kDecStages * kDecStageBytes);
  uint64_t* empty = full + kDecStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kDecStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;   // an earlier launch gave up on a wait
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int bhkv = b * p.H_kv + hkv;
  const int len = p.kv_len ? min(max(p.kv_len[b], 0), p.L) : p.L;
  const int n_tiles_all = (len + kDecTileKeys - 1) / kDecTileKeys;
  const int tiles_per_split = (n_tiles_all + p.nsplit - 1) / p.nsplit;
  const int tile0 = split * tiles_per_split;
  const int tile1 = min(n_tiles_all, tile0 + tiles_per_split);
  const int n_tiles = max(0, tile1 - tile0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDecStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kDecWarps); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  auto issue_stage = [&](int j) {
    const int st = j % kDecStages;
    uint8_t* sb = smem + st * kDecStageBytes;
    const int key0 = (tile0 + j) * kDecTileKeys;
    // scale rows past L are not read: the copy is clipped to the cache extent (L % 4 == 0 keeps it a 16-byte multiple)
    const uint32_t sbytes = (uint32_t)min(kDecTileKeys, p.L - key0) * 4u;
    mbar_arrive_expect_tx(&full[st], 2u * kDecTileKeys * kDecD + 2u * sbytes);
    tma_load_3d(sb, &tmap_k, &full[st], 0, key0, bhkv);
    tma_load_3d(sb + kDecTileKeys * kDecD, &tmap_v, &full[st], 0, key0, bhkv);
    bulk_load_1d(sb + 2 * kDecTileKeys * kDecD, p.k_scale + ((size_t)bhkv * p.L + key0) * 4, sbytes, &full[st]);
    bulk_load_1d(sb + 2 * kDecTileKeys * kDecD + kDecTileKeys * 4, p.v_scale + ((size_t)bhkv * p.L + key0) * 4, sbytes, &full[st]);
  };
  if (warp == kDecWarps) {
    // ================= TMA producer warp =================
    if (lane == 0) {
      prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      for (int j = 0; j < n_tiles; ++j) {
        if (j >= kDecStages &&
            !mbar_wait<20000>(&empty[j % kDecStages], ((j / kDecStages) - 1) & 1, abort_flag, p.status, 402)) break;
        issue_stage(j);
      }
    }
  }

  const float NEG_INF = __int_as_float(0xff800000);
  float m_run = NEG_INF, l_part = 0.0f;
  int vref = 127;          // reference V scale code of this warp's accumulator: oacc = sum(p v) * 2^(127 - vref)
  float oacc[4][4][4];   // [32-col group][e][c-frag]; c0,c1 = head g, cols 32grp+8t+e, +4; c2,c3 = unused rows
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int e = 0; e < 4; ++e) { oacc[a][e][0] = oacc[a][e][1] = oacc[a][e][2] = oacc[a][e][3] = 0.0f; }
  bool ok = true;

  if (warp < kDecWarps) {   // consumer warps (the producer warp must not join their warp-wide shuffles)
    // ---- Q fragments: head g of the group (rows 8..15 of the MMA tile stay zero) ------------------
    // contraction order inside a 16-wide k-step i: logical k = 2t,2t+1 -> d = 16i+4t+{0,1}; k = 2t+8,2t+9 -> d = 16i+4t+{2,3}
    uint32_t qa[8][2];
    float qscale = 0.0f;     // softmax_scale * log2(e) * 2^(e_h): undoes the per-head power-of-two pre-scale
    {
      const int h = hkv * p.grp + g;
      float qv[8][4];
      float amax = 0.0f;
      if (g < p.grp) {
        const __nv_bfloat16* qrow = p.q + ((size_t)b * p.H + h) * kDecD;
  #pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint2 raw = *reinterpret_cast<const uint2*>(qrow + 16 * i + 4 * t);
          qv[i][0] = __uint_as_float(raw.x << 16); qv[i][1] = __uint_as_float(raw.x & 0xFFFF0000u);
          qv[i][2] = __uint_as_float(raw.y << 16); qv[i][3] = __uint_as_float(raw.y & 0xFFFF0000u);
  #pragma unroll
          for (int e = 0; e < 4; ++e) amax = fmaxf(amax, fabsf(qv[i][e]));
        }
      } else {
  #pragma unroll
        for (int i = 0; i < 8; ++i) { qv[i][0] = qv[i][1] = qv[i][2] = qv[i][3] = 0.0f; }
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      int eh = (int)((__float_as_uint(amax) >> 23) & 0xFF);        // biased exponent of the head's largest |q|
      eh = max(1, min(eh, 253));
      const float down = __uint_as_float((uint32_t)(254 - eh) << 23);   // 2^-(eh-127): largest |q| lands in [1,2)
      const float up = __uint_as_float((uint32_t)eh << 23);
      qscale = p.scale_log2 * up;
  #pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __half2 lo = __floats2half2_rn(qv[i][0] * down, qv[i][1] * down);
        const __half2 hi = __floats2half2_rn(qv[i][2] * down, qv[i][3] * down);
        qa[i][0] = *reinterpret_cast<const uint32_t*>(&lo);
        qa[i][1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
    }

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kDecStages;
      ok = __all_sync(0xffffffffu, mbar_wait<20000>(&full[st], (j / kDecStages) & 1, abort_flag, p.status, 401));
      if (!ok) break;
      const uint8_t* sk = smem + st * kDecStageBytes;
      const uint8_t* sv = sk + kDecTileKeys * kDecD;
      const uint8_t* sks = sv + kDecTileKeys * kDecD;
      const uint8_t* svs = sks + kDecTileKeys * 4;
      const int wkey0 = warp * 32;                              // this warp's 32 keys inside the stage
      const int gkey0 = (tile0 + j) * kDecTileKeys + wkey0;     // global index of the first of them

      if (gkey0 < len) {
        // ---------------- S = Q K^T for 32 keys: 4 n-tiles of 8 keys ----------------
        float sacc[4][2];
  #pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int krow = wkey0 + nt * 8 + g;                  // B fragment: key n = g of this n-tile
          const uint8_t* rowp = sk + krow * 128;
          const uint32_t ksc = *reinterpret_cast<const uint32_t*>(sks + (wkey0 + nt * 8 + 2 * t) * 4);       // key col 2t
          const uint32_t ksc1 = *reinterpret_cast<const uint32_t*>(sks + (wkey0 + nt * 8 + 2 * t + 1) * 4);  // key col 2t+1
          float s0 = 0.0f, s1 = 0.0f;
  #pragma unroll
          for (int blk = 0; blk < 4; ++blk) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  #pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int i = blk * 2 + hh;
              const uint32_t w = *reinterpret_cast<const uint32_t*>(rowp + ((i ^ (krow & 7)) << 4) + 4 * t);
              mma_f16_16816(c, qa[i][0], 0u, qa[i][1], 0u, codes_to_f16x2<FMT, false>(w), codes_to_f16x2<FMT, true>(w));
            }
            s0 = fmaf(c[0], e8m0_byte_to_f32(ksc, blk), s0);
            s1 = fmaf(c[1], e8m0_byte_to_f32(ksc1, blk), s1);
          }
          sacc[nt][0] = s0 * qscale;     // log2 domain
          sacc[nt][1] = s1 * qscale;
        }
        // ---------------- mask the tail, online softmax over these 32 keys ----------------
        const bool tail = gkey0 + 32 > len;
        float mx = NEG_INF;
  #pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          if (tail) {
            const int kk = gkey0 + nt * 8 + 2 * t;
            if (kk >= len) sacc[nt][0] = NEG_INF;
            if (kk + 1 >= len) sacc[nt][1] = NEG_INF;
          }
          mx = fmaxf(mx, fmaxf(sacc[nt][0], sacc[nt][1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);          // finite: key gkey0 is valid for every head row
        const float corr = (m_run == NEG_INF) ? 1.0f : ex2_approx(m_run - m_new);
        m_run = m_new;
        float pr[4][2];
  #pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          pr[nt][0] = ex2_approx(sacc[nt][0] - m_new);
          pr[nt][1] = ex2_approx(sacc[nt][1] - m_new);
        }
        l_part = l_part * corr + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]) + (pr[2][0] + pr[2][1]) + (pr[3][0] + pr[3][1]));
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
  #pragma unroll
          for (int a = 0; a < 4; ++a)
  #pragma unroll
            for (int e = 0; e < 4; ++e) { oacc[a][e][0] *= corr; oacc[a][e][1] *= corr; }
        }
        // ---------------- V scale words of this lane's 8 keys; the warp's reference scale code ----------------
        uint32_t vsw[2][4];
  #pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          const int r0 = wkey0 + ks * 16 + 2 * t;               // V rows 2t, 2t+1, 2t+8, 2t+9 of this k-step
          vsw[ks][0] = *reinterpret_cast<const uint32_t*>(svs + (r0) * 4);
          vsw[ks][1] = *reinterpret_cast<const uint32_t*>(svs + (r0 + 1) * 4);
          vsw[ks][2] = *reinterpret_cast<const uint32_t*>(svs + (r0 + 8) * 4);
          vsw[ks][3] = *reinterpret_cast<const uint32_t*>(svs + (r0 + 9) * 4);
          if (tail) {                                            // scales of keys past the end are not data
            const int kk = gkey0 + ks * 16 + 2 * t;
            if (kk >= len) vsw[ks][0] = 0u;
            if (kk + 1 >= len) vsw[ks][1] = 0u;
            if (kk + 8 >= len) vsw[ks][2] = 0u;
            if (kk + 9 >= len) vsw[ks][3] = 0u;
          }
        }
        {
          uint32_t mw = __vmaxu4(__vmaxu4(__vmaxu4(vsw[0][0], vsw[0][1]), __vmaxu4(vsw[0][2], vsw[0][3])),
                                 __vmaxu4(__vmaxu4(vsw[1][0], vsw[1][1]), __vmaxu4(vsw[1][2], vsw[1][3])));
          mw = __vmaxu4(mw, mw >> 16);
          const int vloc = (int)__reduce_max_sync(0xffffffffu, max(mw & 0xFFu, (mw >> 8) & 0xFFu));
          if (vloc > vref) {                                     // warp-uniform
            const int dn = vloc - vref;                          // accumulator *= 2^-dn, exact (or 0 below fp32 range)
            const float f = dn < 127 ? __uint_as_float((uint32_t)(127 - dn) << 23) : 0.0f;
  #pragma unroll
            for (int a = 0; a < 4; ++a)
  #pragma unroll
              for (int e = 0; e < 4; ++e) { oacc[a][e][0] *= f; oacc[a][e][1] *= f; }
            vref = vloc;
          }
        }
        // bf16x2 of 2^(F + 127 - vref), F = 120 for E4M3: undoes the bit placement of V and moves P * 2^(sv-127) to the
        // reference scale
        const uint32_t two120 = ((uint32_t)(254 + DecFmt<FMT>::F - vref) << 7) * 0x00010001u;
        // ---------------- O += P V, two k-steps of 16 keys ----------------
  #pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          // A fragment rows = head g; k = 2t,2t+1 <- n-tile 2ks (keys 16ks+2t,+1); k = 2t+8,2t+9 <- n-tile 2ks+1
          const uint32_t p01 = pack_bf16x2(pr[2 * ks][0], pr[2 * ks][1]);
          const uint32_t p89 = pack_bf16x2(pr[2 * ks + 1][0], pr[2 * ks + 1][1]);
          const int r0 = wkey0 + ks * 16 + 2 * t;               // V rows 2t, 2t+1, 2t+8, 2t+9 of this k-step
          const uint32_t vs0 = vsw[ks][0], vs1 = vsw[ks][1], vs8 = vsw[ks][2], vs9 = vsw[ks][3];
  #pragma unroll
          for (int grp = 0; grp < 4; ++grp) {
            // P * 2^(sv-127) * 2^(247-vref) per (key, 32-col group)
            uint32_t a0 = bf16x2_mul(bf16x2_mul(p01, ue8m0x2_to_bf16x2(prmt(vs0, vs1, 0x0040u + 0x11u * grp))), two120);
            uint32_t a2 = bf16x2_mul(bf16x2_mul(p89, ue8m0x2_to_bf16x2(prmt(vs8, vs9, 0x0040u + 0x11u * grp))), two120);
            if (tail) {
              const int kk = gkey0 + ks * 16 + 2 * t;
              if (kk >= len) a0 &= 0xFFFF0000u;
              if (kk + 1 >= len) a0 &= 0x0000FFFFu;
              if (kk + 8 >= len) a2 &= 0xFFFF0000u;
              if (kk + 9 >= len) a2 &= 0x0000FFFFu;
            }
            const int chunk = 2 * grp + (g >> 2);                // 16-byte chunk holding cols 32grp+4g..+3
            const int wo = (g & 3) * 4;
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(sv + (r0) * 128 + ((chunk ^ ((r0) & 7)) << 4) + wo);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(sv + (r0 + 1) * 128 + ((chunk ^ ((r0 + 1) & 7)) << 4) + wo);
            const uint32_t w8 = *reinterpret_cast<const uint32_t*>(sv + (r0 + 8) * 128 + ((chunk ^ ((r0 + 8) & 7)) << 4) + wo);
            const uint32_t w9 = *reinterpret_cast<const uint32_t*>(sv + (r0 + 9) * 128 + ((chunk ^ ((r0 + 9) & 7)) << 4) + wo);
  #pragma unroll
            for (int e = 0; e < 4; ++e) {
              // bytes e of the two rows -> byte 1 and byte 3 of the fragment register
              const uint32_t sel = 0x4000u * 0 + ((4u + e) << 12) + ((uint32_t)e << 4);   // {b3,b2,b1,b0} = {w1[e], x, w0[e], x}
              const uint32_t b0 = hi_bytes_to_bf16x2_scaled<FMT>(prmt(w0, w1, sel));
              const uint32_t b1 = hi_bytes_to_bf16x2_scaled<FMT>(prmt(w8, w9, sel));
              mma_bf16_16816(oacc[grp][e], a0, 0u, a2, 0u, b0, b1);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);   // the producer warp refills the stage once all 4 warps let go
    }

  }

  // ---- merge the 4 warps through shared memory, write the split's partial ------------------------
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem);             // [warp][8 heads][132]: 128 O values, m, l
  if (warp < kDecWarps) {
    float l_row = l_part;
    l_row += __shfl_xor_sync(0xffffffffu, l_row, 1);
    l_row += __shfl_xor_sync(0xffffffffu, l_row, 2);
    float* mine = red + (warp * 8 + g) * 132;
    const float vback = __uint_as_float((uint32_t)vref << 23);   // 2^(vref-127): back to the true scale
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mine[32 * a + 8 * t + e] = oacc[a][e][0] * vback;
        mine[32 * a + 8 * t + 4 + e] = oacc[a][e][1] * vback;
      }
    if (t == 0) { mine[128] = m_run; mine[129] = l_row; }
  }
  __syncthreads();
  if (ok || !*abort_flag) {
    for (int idx = threadIdx.x; idx < p.grp * 128; idx += kDecThreads) {
      const int hg = idx >> 7, c = idx & 127;
      float m = NEG_INF;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, red[(w * 8 + hg) * 132 + 128]);
      float o = 0.0f, l = 0.0f;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float mw = red[(w * 8 + hg) * 132 + 128];
        const float f = (mw == NEG_INF) ? 0.0f : ex2_approx(mw - m);
        o += f * red[(w * 8 + hg) * 132 + c];
        l += f * red[(w * 8 + hg) * 132 + 129];
      }
      const size_t bh = (size_t)b * p.H + hkv * p.grp + hg;
      p.part_o[(bh * p.nsplit + split) * 128 + c] = o;
      if (c == 0) { p.part_ml[(bh * p.nsplit + split) * 2] = m; p.part_ml[(bh * p.nsplit + split) * 2 + 1] = l; }
    }
  }
}

// log-sum-exp combine of the split partials: one warp per (b, h); lane owns 4 columns.
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nsplit,
                                      int BH, __nv_bfloat16* __restrict__ o, float* __restrict__ lse) {
  const int bh = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (bh >= BH) return;
  const float NEG_INF = __int_as_float(0xff800000);
  float m = NEG_INF;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[((size_t)bh * nsplit + s) * 2]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.0f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[((size_t)bh * nsplit + s) * 2];
    const float f = (ms == NEG_INF) ? 0.0f : exp2f(ms - m);
    l += f * part_ml[((size_t)bh * nsplit + s) * 2 + 1];
    const float4 v = *reinterpret_cast<const float4*>(part_o + ((size_t)bh * nsplit + s) * 128 + lane * 4);
    acc[0] += f * v.x; acc[1] += f * v.y; acc[2] += f * v.z; acc[3] += f * v.w;
  }
  const float inv = l > 0.0f ? 1.0f / l : 1.0f;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
  uint2 out;
  out.x = *reinterpret_cast<const uint32_t*>(&lo);
  out.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(o + (size_t)bh * 128 + lane * 4) = out;
  if (lse && lane == 0) lse[bh] = l > 0.0f ? m * 0.6931471805599453f + logf(l) : NEG_INF;
}

int make_tmap_u8_3d(CUtensorMap* m, const void* base, int64_t BH, int64_t S, int64_t d);   // defined beside the prefill kernel

}  // namespace rk
#include "rk_decode_tc.cuh"
namespace rk {

// Which kernel serves a call: the tcgen05 kernel handles d = 128 with up to 4 query heads per KV head; everything
// else (and a forced choice through the test hook: 1 = mma.sync kernel, 2 = tcgen05 kernel) takes the mma.sync kernel.
int g_decode_path = 0;
bool decode_uses_tc(const rk_decode_args& a) {
  // 6-bit and 4-bit caches hold one code per byte, which the tensor core does not read: the mma.sync kernel converts them
  const bool can = a.d == 128 && a.H_kv > 0 && a.H / a.H_kv <= dtc::kMaxGrp && a.kv_fmt <= RK_FMT_E5M2;
  if (g_decode_path == 1) return false;
  return can;
}
int decode_ctas_per_sm(const rk_decode_args& a) { return decode_uses_tc(a) ? dtc::kCtasPerSm : 2; }

int launch_decode(const rk_decode_args& a, int nsplit, cudaStream_t st) {
  CUtensorMap tk, tv;
  int rc;
  if ((rc = make_tmap_u8_3d(&tk, a.k, (int64_t)a.B * a.H_kv, a.L, a.d)) != RK_OK) return rc;
  if ((rc = make_tmap_u8_3d(&tv, a.v, (int64_t)a.B * a.H_kv, a.L, a.d)) != RK_OK) return rc;
  DecodeParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.k_scale = a.k_scale; p.v_scale = a.v_scale; p.kv_len = a.kv_len;
  const size_t BH = (size_t)a.B * a.H;
  p.part_o = reinterpret_cast<float*>(a.workspace);
  p.part_ml = p.part_o + BH * nsplit * 128;
  p.status = device_status_word();
  if (!p.status) return RK_ERR_NO_DEVICE;
  p.B = a.B; p.H = a.H; p.H_kv = a.H_kv; p.L = a.L; p.grp = a.H / a.H_kv; p.nsplit = nsplit;
  const float scale = a.softmax_scale > 0.0f ? a.softmax_scale : 1.0f / sqrtf((float)a.d);
  p.scale_log2 = scale * 1.4426950408889634f;
  cudaError_t e;
  dim3 grid(nsplit, a.H_kv, a.B);
  if (decode_uses_tc(a)) {
    DecodeTcParams t;
    t.q = p.q; t.k_scale = p.k_scale; t.v_scale = p.v_scale; t.kv_len = p.kv_len;
    t.part_o = p.part_o; t.part_ml = p.part_ml; t.status = p.status;
    t.B = p.B; t.H = p.H; t.H_kv = p.H_kv; t.L = p.L; t.grp = p.grp; t.nsplit = p.nsplit; t.scale_log2 = p.scale_log2;
    const bool eight = p.grp > 4;                        // head capacity 4 (two P buffers) or 8 (one)
    const int smem_bytes = (eight ? dtc::Lay<8>::total : dtc::Lay<4>::total) + 1024;
    auto kern = eight ? decode_tc_kernel<8> : decode_tc_kernel<4>;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes)) != cudaSuccess) return (int)e;
    // A = the cache tile in its own 8-bit format (E4M3 or E5M2: no thread decodes a cache byte, so the format is
    // one field of the instruction descriptor), B = the MXFP8 terms of Q / P, always E4M3
    const uint32_t idesc_qk = make_idesc(a.kv_fmt, RK_FMT_E4M3, false, false, 128, dtc::kNq);
    const uint32_t idesc_pv = make_idesc(a.kv_fmt, RK_FMT_E4M3, true, false, 128, eight ? dtc::Lay<8>::kNp : dtc::Lay<4>::kNp);
    if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_before, st);
    kern<<<grid, dtc::kThreads, smem_bytes, st>>>(tk, tv, t, idesc_qk, idesc_pv);
    if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_after, st);
  } else {
    auto kern = a.kv_fmt == RK_FMT_E5M2 ? decode_kernel<1> : a.kv_fmt == RK_FMT_E2M3 ? decode_kernel<2> :
                a.kv_fmt == RK_FMT_E3M2 ? decode_kernel<3> : a.kv_fmt == RK_FMT_E2M1 ? decode_kernel<4> : decode_kernel<0>;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes)) != cudaSuccess) return (int)e;
    if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_before, st);
    kern<<<grid, kDecThreads, kDecSmemBytes, st>>>(tk, tv, p);
    if (g_ev_before && g_ev_after) cudaEventRecord(g_ev_after, st);
  }
  if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  const int warps_per_cta = 4;
  decode_combine_kernel<<<(int)((BH + warps_per_cta - 1) / warps_per_cta), warps_per_cta * 32, 0, st>>>(
      p.part_o, p.part_ml, nsplit, (int)BH, reinterpret_cast<__nv_bfloat16*>(a.o), a.lse);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// Decode without any allocation.  Some hosts may not allocate device memory where they call us: a
// serving loop that runs inside a memory pool it does not own, a plugin loaded into a process whose
// allocator is locked while a step is in flight, or code that must not perturb a caching allocator's
// bookkeeping.  For them the split partials live in a fixed array that is part of the library image
// on every GPU that loads it, instead of in a caller-provided workspace.
constexpr size_t kNoAllocScratchFloats = RK_DECODE_NOALLOC_SCRATCH_BYTES / sizeof(float);   // e.g. batch 64 x 32 heads x 4 splits x 130 floats
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
static __device__ int g_noalloc_status;               // zero at load; a kernel's bounded wait records its code here

namespace {
struct NoAllocDev { bool ready = false; float* scratch = nullptr; int* status = nullptr; int sms = 0; };
NoAllocDev g_noalloc_dev[64];
std::mutex g_noalloc_mu;
}  // namespace

// Set-up of the no-allocation path for the current device (once per device): in host code the array's name is
// only a stand-in, the device address comes from the runtime, with that device current.
static int noalloc_dev(NoAllocDev& out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  NoAllocDev& slot = g_noalloc_dev[dev & 63];
  if (!slot.ready) {
    void* ptr = nullptr;
    if ((e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch)) != cudaSuccess) return (int)e;
    slot.scratch = static_cast<float*>(ptr);
    if ((e = cudaGetSymbolAddress(&ptr, g_noalloc_status)) != cudaSuccess) return (int)e;
    slot.status = static_cast<int*>(ptr);
    if ((e = cudaDeviceGetAttribute(&slot.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    slot.ready = true;
  }
  out = slot;
  return RK_OK;
}

// Status word of the no-allocation path on the current device: synchronises the device, returns the recorded code
// (0 = clean) and clears it.  Plain copies to and from an address inside the library image: nothing is allocated.
int noalloc_status_read_clear() {
  NoAllocDev nd;
  int rc = noalloc_dev(nd);
  if (rc != RK_OK) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  int v = 0;
  if ((e = cudaMemcpy(&v, nd.status, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess) return (int)e;
  if (v != 0) {
    const int zero = 0;
    if ((e = cudaMemcpy(nd.status, &zero, sizeof(int), cudaMemcpyHostToDevice)) != cudaSuccess) return (int)e;
  }
  return v;
}

// Test hook: one CTA waits on an mbarrier nobody arrives at, with the bounded wait every kernel here uses.
__global__ void wait_runs_out_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag = 0; fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, status, 901, limit_ns);
  __syncthreads();
}

int launch_wait_runs_out(int limit_us, bool noalloc, cudaStream_t st) {
  if (limit_us <= 0 || limit_us > 1000000) return RK_ERR_BAD_SHAPE;     // at most one second
  int* status = nullptr;
  if (noalloc) {
    NoAllocDev nd;
    int rc = noalloc_dev(nd);
    if (rc != RK_OK) return rc;
    status = nd.status;
  } else {
    status = device_status_word();
    if (!status) return RK_ERR_NO_DEVICE;
  }
  wait_runs_out_kernel<<<1, 32, 0, st>>>(status, (unsigned long long)limit_us * 1000ull);
  return (int)cudaGetLastError();
}

int launch_decode_noalloc(const rk_decode_args& a, cudaStream_t st) {
  NoAllocDev nd;
  {
    int rc0 = noalloc_dev(nd);
    if (rc0 != RK_OK) return rc0;
  }
  cudaError_t e;
  // split count: the caller's, or the one that fills whole waves of 2 CTAs per SM best, shrunk to fit the array
  const int tiles = (a.L + kDecTileKeys - 1) / kDecTileKeys;
  const size_t BH = (size_t)a.B * a.H;
  int nsplit;
  if (a.num_splits > 0) {
    nsplit = a.num_splits < tiles ? a.num_splits : tiles;
    if (BH * nsplit * 130 > kNoAllocScratchFloats) return RK_ERR_TOO_LARGE;
  } else {
    const long slots = 2L * nd.sms, units = (long)a.B * a.H_kv;
    nsplit = 1; double best_eff = -1.0;
    for (int s = 1; s <= 64 && (s == 1 || tiles / s >= 4) && BH * s * 130 <= kNoAllocScratchFloats; ++s) {
      const long ctas = units * s, waves = (ctas + slots - 1) / slots;
      const double eff = (double)ctas / (double)(waves * slots);
      if (eff > best_eff + 0.02) { best_eff = eff; nsplit = s; }
    }
    if (BH * nsplit * 130 > kNoAllocScratchFloats) return RK_ERR_TOO_LARGE;
  }
  CUtensorMap tk, tv;
  int rc;
  if ((rc = make_tmap_u8_3d(&tk, a.k, (int64_t)a.B * a.H_kv, a.L, a.d)) != RK_OK) return rc;
  if ((rc = make_tmap_u8_3d(&tv, a.v, (int64_t)a.B * a.H_kv, a.L, a.d)) != RK_OK) return rc;
  DecodeParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(a.q);
  p.k_scale = a.k_scale; p.v_scale = a.v_scale; p.kv_len = a.kv_len;
  p.part_o = nd.scratch;
  p.part_ml = nd.scratch + BH * nsplit * 128;
  p.status = nd.status;
  p.B = a.B; p.H = a.H; p.H_kv = a.H_kv; p.L = a.L; p.grp = a.H / a.H_kv; p.nsplit = nsplit;
  const float scale = a.softmax_scale > 0.0f ? a.softmax_scale : 1.0f / sqrtf((float)a.d);
  p.scale_log2 = scale * 1.4426950408889634f;
  if ((e = cudaFuncSetAttribute(decode_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes)) != cudaSuccess) return (int)e;
  decode_kernel<0><<<dim3(nsplit, a.H_kv, a.B), kDecThreads, kDecSmemBytes, st>>>(tk, tv, p);
  if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  decode_combine_kernel<<<(int)((BH + 3) / 4), 128, 0, st>>>(p.part_o, p.part_ml, nsplit, (int)BH,
                                                            reinterpret_cast<__nv_bfloat16*>(a.o), a.lse);
  return (int)cudaGetLastError();
}

}  // namespace rk
