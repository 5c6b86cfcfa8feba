// Definitions shared by the two prefill kernels (one 128-row query tile per CTA / two of them).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kTileBytes = 128 * 128;      // one [128 rows][128 B] swizzled tile
constexpr int kSfAtomBytes = 512;
constexpr int kParts = 4;                       // threads per query row (each owns 128 / kParts keys of a tile)
constexpr int kNumSoftmaxWarps = 4 * kParts;
constexpr int kNumThreads = (kNumSoftmaxWarps + 3) * 32;   // + TMA producer, Q K^T issuer, P V issuer
constexpr uint32_t kTmemCols = 512;

// TMEM column map
constexpr uint32_t kColS = 0;
constexpr uint32_t kColO = 128;
constexpr uint32_t kColSfQ = 384;                 // + ch*4
constexpr uint32_t kColSfK = 392;                 // + stage*8 + ch*4   (<= 3 stages)
constexpr uint32_t kColSfP = 416;                 // + pbuf*4
constexpr uint32_t kColSfV = 424;                 // + stage*8 + ch*4

struct PrefillParams {
  const uint8_t* q_sf;
  const uint8_t* k_sf;
  const uint8_t* v_sf;
  __nv_bfloat16* o;
  float* lse;
  int* status;
  float* dbg;          // optional stage dump of CTA (0,0,0), first key tile
  int B, H, H_kv, S_q, S_kv, d;
  int n_q_tiles, n_kv_tiles;
  int head_group;      // (batch, head) pairs per work-order group: the heaviest query tiles of a whole group run first
  int q_pos0, causal, window;
  int q_tile_tx, kv_tile_tx;   // bytes one Q / K / V tile load adds to its mbarrier: 16384, 12288 for 6-bit, 8192 for 4-bit tensors
                               // (the transaction counts the packed source bytes, not the padded shared-memory image)
  int v_transposed;    // V tiles are [d][keys] (K-major B operand; 6-bit V) instead of [keys][d]
  int perturb;         // test hook: warp role that sleeps a little at every key tile (0 = none)
  float scale_log2;    // softmax_scale * log2(e)
  float cap_log2;      // softcap * log2(e)
  float inv_cap_scale; // softmax_scale / softcap
};

RK_DEVINL float fmax3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
// packed fp32 pairs (two lanes per instruction on the FMA pipe)
RK_DEVINL void fma2(float a0, float a1, float b, float c, float& d0, float& d1) {      // d = a * b + c
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}" : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
RK_DEVINL void add2(float& a0, float& a1, float b0, float b1) {                          // a += b
  asm("{\n\t.reg .b64 ra, rb;\n\tmov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %3};\n\tadd.rn.f32x2 ra, ra, rb;\n\tmov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(a0), "+f"(a1) : "f"(b0), "f"(b1));
}
RK_DEVINL void mul2_ftz_inplace(uint32_t& a0, uint32_t& a1, float b) {                 // a *= b on two fp32 bit patterns, in their registers
  asm("{\n\t.reg .b64 ra, rb;\n\tmov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %2};\n\tmul.rn.ftz.f32x2 ra, ra, rb;\n\tmov.b64 {%0, %1}, ra;\n\t}"
      : "+r"(a0), "+r"(a1) : "f"(b));
}
RK_DEVINL void mul2_ftz(float a0, float a1, float b, float& d0, float& d1) {           // d = a * b, subnormal results -> 0
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmul.rn.ftz.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b));
}
// The same packed operations on values that stay in 64-bit registers (two fp32 lanes each): a broadcast operand is
// packed once by the caller instead of once per instruction.
RK_DEVINL uint64_t pack2(float lo, float hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
RK_DEVINL void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
RK_DEVINL void unpack2u(uint64_t v, uint32_t& lo, uint32_t& hi) { asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v)); }
RK_DEVINL uint64_t fma2p(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
RK_DEVINL uint64_t add2p(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
RK_DEVINL uint64_t mul2p_ftz(uint64_t a, uint64_t b) { uint64_t d; asm("mul.rn.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
// Soft cap of two scores in the log2 domain: cap_log2 * tanh(s * scale / cap), tanh(y) = 1 - 2 / (1 + e^(2y)).
// The exponential is the one special-function instruction; the reciprocal is three Newton steps on the FMA pipe from
// an integer first guess (error 0.12 -> 1.4e-2 -> 2e-4 -> 4e-8), because the special-function unit is what bounds
// the capped kernels (it also has the softmax exponential to do).  k2 = 2 log2(e) scale / cap; the exponent is
// clamped so that 1 + e stays finite.
RK_DEVINL void softcap_pair(float& s0, float& s1, float k2, uint64_t one2, uint64_t m2cap2, uint64_t cap2) {
  const float e0 = ex2_approx(fminf(s0 * k2, 126.0f)), e1 = ex2_approx(fminf(s1 * k2, 126.0f));
  const uint64_t z = add2p(pack2(e0, e1), one2);                       // 1 + e in [1, 2^126]
  uint32_t z0, z1;
  unpack2u(z, z0, z1);
  uint64_t r = pack2(__uint_as_float(0x7EF311C7u - z0), __uint_as_float(0x7EF311C7u - z1));
  const uint64_t nz = z ^ 0x8000000080000000ull;                       // -z
#pragma unroll
  for (int it = 0; it < 3; ++it) r = fma2p(r, fma2p(nz, r, one2), r);   // r += r * (1 - z r)
  unpack2(fma2p(r, m2cap2, cap2), s0, s1);                              // cap_log2 * (1 - 2 r)
}

RK_DEVINL float fmin3(float a, float b, float c) { float d; asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
RK_DEVINL uint64_t mul2p(uint64_t a, uint64_t b) { uint64_t d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// The soft cap of a whole set of scores, in place: s <- cap_log2 * tanh(s * scale / cap).
// While every |s * scale / cap| of the warp's scores is at most 1/8 (logits of a model that caps at 50 are two orders
// of magnitude below that) tanh is its series y - y^3/3 + 2 y^5/15 - 17 y^7/315 (next term below 1.4e-9 of y),
// evaluated in s^2 with the constants folded into the coefficients: five packed FMA-pipe operations per pair of
// scores and no special-function operation, against an exponential and a Newton reciprocal per score in
// softcap_pair, which is kept for the scores that are not small (the decision is per warp and per key tile).
template <int N>
RK_DEVINL void softcap_scores(float (&s)[N], float scale_log2, float cap_log2, float inv_cap_scale) {
  static_assert(N % 2 == 0 && N >= 4, "pairs");
  float hi = fmax3(s[0], s[1], s[2]), lo = fmin3(s[0], s[1], s[2]);
#pragma unroll
  for (int c = 3; c + 1 < N; c += 2) { hi = fmax3(hi, s[c], s[c + 1]); lo = fmin3(lo, s[c], s[c + 1]); }
  hi = fmaxf(hi, s[N - 1]); lo = fminf(lo, s[N - 1]);
  const bool small = fmaxf(hi, -lo) * inv_cap_scale <= 0.125f;          // false for NaN
  if (__all_sync(0xffffffffu, small)) {
    const float q = inv_cap_scale * inv_cap_scale;
    const float c1 = -0.3333333333f * q * scale_log2, c2 = 0.1333333333f * q * q * scale_log2,
                c3 = -0.05396825397f * q * q * q * scale_log2;
    const uint64_t k1 = pack2(c1, c1), k2 = pack2(c2, c2), k3 = pack2(c3, c3), a2 = pack2(scale_log2, scale_log2);
#pragma unroll
    for (int c = 0; c < N; c += 2) {
      const uint64_t v = pack2(s[c], s[c + 1]);
      const uint64_t z = mul2p(v, v);
      uint64_t t = fma2p(z, k3, k2);
      t = fma2p(z, t, k1);
      t = fma2p(z, t, a2);
      unpack2(mul2p(v, t), s[c], s[c + 1]);
    }
  } else {
    const float k2 = 2.0f * 1.4426950408889634f * inv_cap_scale;
    const uint64_t one2 = pack2(1.0f, 1.0f), m2cap2 = pack2(-2.0f * cap_log2, -2.0f * cap_log2), cap2 = pack2(cap_log2, cap_log2);
#pragma unroll
    for (int c = 0; c < N; c += 2) softcap_pair(s[c], s[c + 1], k2, one2, m2cap2, cap2);
  }
}

// two ints (0..255 each) into bytes 1:0 of the result, bytes 3:2 taken from the low half of c
RK_DEVINL uint32_t pack_u8x2(uint32_t hi, uint32_t lo, uint32_t c) {
  uint32_t d; asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(c)); return d;
}

#ifdef RK_X_STAMPS
// Timeline stamps (measurement builds only): clock64 of chosen events of one CTA, written into the dump buffer.
// The CTA is RK_X_STAMP_BLOCK, or the block index b when the perturbation hook is set to 1000 + b (+ 100000 * (s + 1)
// to pick the s-th work item of a persistent CTA).
#ifndef RK_X_STAMP_BLOCK
#define RK_X_STAMP_BLOCK 0
#endif
#define RK_STAMP_CTA ((int)blockIdx.x == (p.perturb % 100000 >= 1000 ? p.perturb % 100000 - 1000 : RK_X_STAMP_BLOCK))
#define RK_STAMP(slot, j, k) do { if (p.dbg && RK_STAMP_CTA && (j) < 32) \
    reinterpret_cast<unsigned*>(p.dbg)[24576 + (slot) * 512 + (j) * 8 + (k)] = (unsigned)clock64(); } while (0)
#define RK_STAMP_RAW(idx) do { if (p.dbg && RK_STAMP_CTA) \
    reinterpret_cast<unsigned*>(p.dbg)[24576 + 2048 + (idx)] = (unsigned)clock64(); } while (0)
#else
#define RK_STAMP(slot, j, k) do {} while (0)
#define RK_STAMP_RAW(idx) do {} while (0)
#endif


int make_tmap_u8_3d(CUtensorMap* m, const void* base, int64_t BH, int64_t S, int64_t d);
int make_tmap_sub8_3d(CUtensorMap* m, const void* base, int64_t BH, int64_t rows, int64_t cols_padded, int bits);
extern float* g_prefill_dbg;

// Two query tiles per CTA, one thread per row, correction warps (d <= 128); defined in rk_prefill2c.cu.
int launch_prefill2c(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                     uint32_t idesc_qk, uint32_t idesc_pv, bool softcap, int B, cudaStream_t st);
extern int g_prefill_perturb;   // test hook: PrefillParams::perturb of the next launches

}  // namespace rk
