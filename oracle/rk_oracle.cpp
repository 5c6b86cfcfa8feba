// CPU oracle for the MX attention path.  TEST INFRASTRUCTURE ONLY: this file is
// the checker the GPU kernels are compared with (and the timed CPU baseline of
// the benchmark); nothing in the shipped library calls it.
//
// It restates, in plain C++17 with fp32 arithmetic, the algorithm of the
// radiance-kernels MXFP8 flash-attention path.  Each function cites the
// reference file:line it follows (paths relative to the reference tree).
//
// Parity status
//   * codecs + block quantizer: PINNED.  Checked bit for bit against the
//     reference's own lib/golden/mx_fp_math.h (compiled from the reference
//     tree) and against golden vectors produced by the reference's
//     lib/golden/golden.py and kernels/simt_quant/gen_quant.py.
//   * RoPE (rko_rope_rows) and the tanh soft-cap: PINNED against vectors made by
//     importing rope_caches / rope_apply / softcap from lib/golden/golden.py.
//   * the P requantization rule (p_block_scale_code, p_code): PINNED against the
//     reference attention kernel's own helpers bf16_floor_log2 /
//     bf16_to_e4m3_scaled (kernels/flash_attention_mx_gqa/flash_mx_impl.hpp:53-77)
//     compiled from the reference tree, over every non-negative finite bf16 p.
//   * the fp32 attention reference (rko_attn_fp32_ref: causal mask with a query
//     offset, GQA head map, soft-cap before the mask, sliding window): PINNED
//     against the reference's own attention_reference_causal_gqa /
//     attention_reference_gemma (golden vectors made by importing its model files).
//   * the MX attention composition (prefill, decode): PARITY UNPINNED.  The
//     reference commits no MX attention golden vectors and the MX half of its
//     Python model calls into a module (fp8_matmul_model, from the un-vendored
//     submodule lib/mxgemmini -> Rakanic/gemmini-rocc-tests, no pinned revision)
//     that is absent.  Every rule the composition uses is pinned above; the
//     structure below follows the reference model line by line; the matmuls are
//     fp32-accumulated over exactly decoded operands and the softmax state is
//     fp32, as the build target asks.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

namespace {

inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// ---------------------------------------------------------------------------
// Element formats.  ebits/mbits/bias and the largest finite magnitude
// (1 + max_mant/2^mbits) * 2^emax.  E4M3 follows lib/golden/mx_fp_math.h:205-236
// (no inf, top code 0x7E = 448).  E5M2 / E2M3 / E3M2 / E2M1 generalise the same
// encoder; E3M2 decode follows lib/golden/mx_fp_math.h:256-264, E2M1 (FP4)
// decode lib/golden/mx_fp_math.h:238-246.
// ---------------------------------------------------------------------------
struct Fmt { int ebits, mbits, bias, emax_unb, max_mant; uint32_t scale_thresh; };
// scale_thresh: mantissa threshold of block_exp (lib/golden/golden.py:161-165),
// i.e. the fp32 mantissa of the format's largest finite value.
const Fmt kFmt[5] = {
    /*E4M3*/ {4, 3, 7, 8, 6, 0x600000u},    // 448   = 1.75  * 2^8
    /*E5M2*/ {5, 2, 15, 15, 3, 0x600000u},  // 57344 = 1.75  * 2^15
    /*E2M3*/ {2, 3, 1, 2, 7, 0x700000u},    // 7.5   = 1.875 * 2^2
    /*E3M2*/ {3, 2, 3, 4, 3, 0x600000u},    // 28    = 1.75  * 2^4
    /*E2M1*/ {2, 1, 1, 2, 1, 0x400000u},    // 6     = 1.5   * 2^2
};

inline float fmt_max(const Fmt& f) {
  return std::ldexp(1.0f + (float)f.max_mant / (float)(1 << f.mbits), f.emax_unb);
}

// decode: lib/golden/mx_fp_math.h:227-236 (E4M3), :256-264 (E3M2); same form
// for the other two.  Codes 0x7F/0xFF of E4M3 decode to +-480 exactly as the
// reference does (it has no NaN case).  E5M2 inf/NaN codes decode as numbers
// too; the quantizer never emits them.
inline float decode_elem(uint8_t code, const Fmt& f) {
  const int nb = 1 + f.ebits + f.mbits;
  const int s = (code >> (nb - 1)) & 1;
  const int e = (code >> f.mbits) & ((1 << f.ebits) - 1);
  const int m = code & ((1 << f.mbits) - 1);
  const float frac = (float)m / (float)(1 << f.mbits);
  float v = (e == 0) ? frac * std::ldexp(1.0f, 1 - f.bias)
                     : (1.0f + frac) * std::ldexp(1.0f, e - f.bias);
  return s ? -v : v;
}

// round-half-to-even of v >> sh: lib/golden/golden.py:118-126,
// kernels/simt_quant/kernel.cpp:44-54 (sh >= 32 underflows to 0).
inline uint32_t round_shift(uint32_t v, int sh) {
  if (sh >= 32) return 0u;
  const uint32_t mask = (1u << sh) - 1u, low = v & mask, half = 1u << (sh - 1);
  uint32_t q = v >> sh;
  if (low > half || (low == half && (q & 1u))) q++;
  return q;
}

// fp32 -> element code, RNE, saturating to the largest finite magnitude, sign
// kept on zero.  For E4M3 this is fp8_code_rshift (lib/golden/golden.py:129-158)
// == f32_to_e4m3 (kernels/simt_quant/kernel.cpp:56-81); the other formats use
// the same integer round-shift with their own widths.
inline uint8_t encode_elem_rne(float xf, const Fmt& f) {
  const int nb = 1 + f.ebits + f.mbits;
  const uint32_t x = f32_bits(xf);
  const uint32_t sign = (x >> 31) & 1u;
  const uint32_t absx = x & 0x7FFFFFFFu;
  const uint32_t s = sign << (nb - 1);
  const uint32_t sat = (uint32_t)((((f.emax_unb + f.bias) << f.mbits) | f.max_mant));
  if (absx == 0u) return (uint8_t)s;
  if (bits_f32(absx) >= fmt_max(f)) return (uint8_t)(s | sat);   // also inf / NaN payloads
  const int e = (int)((absx >> 23) & 0xFFu) - 127;
  const uint32_t sig = (1u << 23) | (absx & 0x7FFFFFu);   // value = sig * 2^(e-23)
  const int emin = 1 - f.bias;
  const uint32_t one = 1u << f.mbits;
  uint32_t out;
  if (e < emin) {                                          // subnormal target
    const uint32_t q = round_shift(sig, (23 - f.mbits) + (emin - e));
    out = (q >= one) ? (one | (q - one)) : q;              // may round up to min normal
  } else {
    uint32_t r = round_shift(sig, 23 - f.mbits);           // in [one, 2*one]
    int E = e;
    if (r == 2 * one) { r = one; E += 1; }
    const int expf = E + f.bias;
    const uint32_t mant = r - one;
    const int expf_max = f.emax_unb + f.bias;
    if (expf > expf_max || (expf == expf_max && (int)mant > f.max_mant)) return (uint8_t)(s | sat);
    out = ((uint32_t)expf << f.mbits) | mant;
  }
  return (uint8_t)(s | out);
}

// E8M0: lib/golden/mx_fp_math.h:249-252 (0xFF -> NaN).  Code 0 is 2^-127, a
// denormal fp32; it is built from its bit pattern so no libm call rounds it.
inline float e8m0_decode(uint8_t c) {
  if (c == 0xFF) return std::numeric_limits<float>::quiet_NaN();
  return c == 0 ? bits_f32(0x00400000u) : bits_f32((uint32_t)c << 23);
}

// One 32-element (or shorter, ragged tail) block under the lib/golden rule:
//   e = ceil(log2(amax / FMT_MAX)) from the fp32 exponent field
//   (lib/golden/golden.py:161-165), scale code clamp(e+127, 0, 254), elements
//   x * 2^-e encoded RNE (kernels/simt_quant/kernel.cpp:95-129,
//   kernels/simt_quant/gen_quant.py:51-70).  `stride` lets the block run along
//   a non-contiguous axis.
inline uint8_t quantize_block(const float* x, int n, int64_t stride, const Fmt& f,
                              uint8_t* codes, int64_t cstride) {
  float amax = 0.0f;
  for (int j = 0; j < n; j++) {
    const float av = bits_f32(f32_bits(x[j * stride]) & 0x7FFFFFFFu);
    if (av > amax) amax = av;
  }
  if (!(amax > 0.0f)) {
    // all-zero block: scale code 0; codes keep only the sign bit, as
    // f32_to_e4m3(+-0 * 1.0) does (kernels/simt_quant/kernel.cpp:110,60).
    for (int j = 0; j < n; j++) codes[j * cstride] = encode_elem_rne(x[j * stride], f);
    return 0;
  }
  const uint32_t ab = f32_bits(amax);
  const int e = ((int)((ab >> 23) & 0xFFu) - 127 - f.emax_unb) + ((ab & 0x7FFFFFu) > f.scale_thresh ? 1 : 0);
  int sc = e + 127;
  sc = sc < 0 ? 0 : (sc > 254 ? 254 : sc);
  const float pow2 = bits_f32((uint32_t)(127 - e) << 23);  // 2^-e (lib/golden/golden.py:168-170)
  for (int j = 0; j < n; j++) codes[j * cstride] = encode_elem_rne(x[j * stride] * pow2, f);
  return (uint8_t)sc;
}

void parallel_for(int64_t n, int nthreads, const std::function<void(int64_t)>& fn) {
  if (nthreads <= 1 || n <= 1) { for (int64_t i = 0; i < n; i++) fn(i); return; }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> th;
  const int nt = (int)std::min<int64_t>(nthreads, n);
  for (int t = 0; t < nt; t++)
    th.emplace_back([&]() { for (;;) { int64_t i = next.fetch_add(1); if (i >= n) break; fn(i); } });
  for (auto& t : th) t.join();
}

// P-tile requant of the attention kernels
// (kernels/flash_attention_mx_gqa/flash_mx_impl.hpp:53-77 bf16_to_e4m3_scaled,
//  :356-387 the per-block scale and store): per 32 keys,
//   se = floor(log2(max p)) clamped to <= 0 (an all-zero block gives se = -127),
//   scale code se + 127, element = p * 2^-se TRUNCATED to 3 mantissa bits,
//   zero when p has a zero exponent field or lands below 2^-6 (no subnormals).
// Restated on the fp32 bit pattern of p instead of the reference's bf16 one.
inline uint8_t p_block_scale_code(float pmax) {
  int se = (int)((f32_bits(pmax) >> 23) & 0xFFu) - 127;
  if (se > 0) se = 0;
  return (uint8_t)(se + 127);
}
inline uint8_t p_code(float p, uint8_t scale_code) {
  const uint32_t b = f32_bits(p);
  const int expf = (int)((b >> 23) & 0xFFu);
  const int se = (int)scale_code - 127;
  int E = expf - 127 - se;
  int m3 = (int)((b >> 20) & 7u);
  if (E > 8) { E = 8; m3 = 6; }
  if (E == 8 && m3 > 6) m3 = 6;
  if (expf == 0 || E < -6) return 0;
  return (uint8_t)(((E + 7) << 3) | m3);
}

inline float bf16_round_to_f32(float x, uint16_t* bits_out) {
  // lib/golden/mx_fp_math.h:11-28 (RNE, -0 and underflow-to-zero canonicalised to +0)
  uint16_t out;
  if (x == 0.0f) out = 0;
  else {
    const uint32_t bits = f32_bits(x);
    if (((bits >> 23) & 0xFF) == 0xFF) {
      uint32_t bf = bits >> 16;
      if ((bits & 0x7FFFFFu) && !(bf & 0x40)) bf |= 0x40;
      out = (uint16_t)bf;
    } else {
      const uint32_t lsb = (bits >> 16) & 1;
      out = (uint16_t)((bits + 0x7FFF + lsb) >> 16);
      if ((out & 0x7FFF) == 0) out = 0;
    }
  }
  if (bits_out) *bits_out = out;
  return bits_f32((uint32_t)out << 16);
}

// fp32 dot product with 16 independent partial sums (lets the compiler
// vectorise; the summation order is part of the oracle's definition only to
// within fp32 reassociation, which the attention tolerance absorbs).
inline float dot_f32(const float* a, const float* b, int n) {
  float acc[16] = {0};
  int i = 0;
  for (; i + 16 <= n; i += 16)
    for (int j = 0; j < 16; j++) acc[j] += a[i + j] * b[i + j];
  float s = 0.0f;
  for (int j = 0; j < 16; j++) s += acc[j];
  for (; i < n; i++) s += a[i] * b[i];
  return s;
}

}  // namespace

extern "C" {

// ------------------------------ codecs -------------------------------------
float rko_decode_elem(uint8_t code, int fmt) { return decode_elem(code, kFmt[fmt]); }
uint8_t rko_encode_elem_rne(float x, int fmt) { return encode_elem_rne(x, kFmt[fmt]); }
float rko_e8m0_decode(uint8_t c) { return e8m0_decode(c); }
uint16_t rko_f32_to_bf16(float x) { uint16_t b; bf16_round_to_f32(x, &b); return b; }
uint8_t rko_p_block_scale_code(float pmax) { return p_block_scale_code(pmax); }
uint8_t rko_p_code(float p, uint8_t sc) { return p_code(p, sc); }

// ------------------------------ quantizer ----------------------------------
// x fp32 [rows][cols] row-major; blocks of 32 along cols (ragged tail allowed).
// codes u8 [rows][cols]; scales u8 [rows][ceil(cols/32)].
void rko_quantize_rows(const float* x, int64_t rows, int64_t cols, int fmt,
                       uint8_t* codes, uint8_t* scales, int nthreads) {
  const Fmt& f = kFmt[fmt];
  const int64_t nb = (cols + 31) / 32;
  parallel_for(rows, nthreads, [&](int64_t r) {
    for (int64_t b = 0; b < nb; b++) {
      const int n = (int)std::min<int64_t>(32, cols - b * 32);
      scales[r * nb + b] = quantize_block(x + r * cols + b * 32, n, 1, f, codes + r * cols + b * 32, 1);
    }
  });
}

// Blocks of 32 along rows (the key axis): scales u8 [ceil(rows/32)][cols].
// This is how the reference quantizes V (kernels/flash_attention_mx/gen_data.py:77,
// kernels/flash_attention_mx_gqa/fa_gen_data.py:106-108: V transposed, then
// quantized per row, i.e. groups run along the keys).
void rko_quantize_cols(const float* x, int64_t rows, int64_t cols, int fmt,
                       uint8_t* codes, uint8_t* scales, int nthreads) {
  const Fmt& f = kFmt[fmt];
  const int64_t nb = (rows + 31) / 32;
  parallel_for(nb, nthreads, [&](int64_t b) {
    const int n = (int)std::min<int64_t>(32, rows - b * 32);
    for (int64_t c = 0; c < cols; c++)
      scales[b * cols + c] = quantize_block(x + b * 32 * cols + c, n, cols, f, codes + b * 32 * cols + c, cols);
  });
}

// codes [rows][cols] + scales [rows][cols/32] -> fp32 (code * 2^(s-127), one fp32 multiply)
// The other quantization rule of the reference, the requant post-pass of its hardware-semantics matmul golden
// (lib/golden/mx_golden.cpp:146-200 with fp8_e4m3_to_code, lib/golden/mx_fp_math.h:205-225), kept as a
// selectable oracle mode; it is NOT the rule of the attention path.  Per 32 values of a row:
//   scale code = floor(log2(amax)) - 8 + 127 (0 for an all-zero block), so the scaled maximum lands in
//   [256, 512) and saturates to 448; element = value / 2^(code-127) rounded to nearest-even on the 3-bit
//   mantissa, exponents below -6 flushed to 0 (no subnormals), zero keeps no sign, above 2^8 -> 448.
// Restated on fp32 bit fields; the reference takes floor(log2f(.)), which agrees with the exponent field
// for the bf16-valued inputs this pass sees.
static uint8_t e4m3_code_mxgolden(float v) {
  const uint32_t b = f32_bits(v);
  const int expf = (int)((b >> 23) & 0xFFu);
  if (expf == 0 || expf == 0xFF) return 0;            // zero, fp32 denormal (far below 2^-6), inf, NaN
  const uint32_t s = b >> 31;
  int E = expf - 127;
  if (E < -6) return 0;
  uint32_t mant;
  if (E > 8) { E = 8; mant = 6; }
  else {
    const uint32_t m23 = b & 0x7FFFFFu;
    uint32_t k = m23 >> 20;
    const uint32_t rem = m23 & 0xFFFFFu, half = 0x80000u;
    if (rem > half || (rem == half && (k & 1u))) k++;
    if (k >= 8) { E += 1; k = 0; if (E > 8) { E = 8; k = 6; } }
    else if (E == 8 && k > 6) k = 6;
    mant = k;
  }
  return (uint8_t)((s << 7) | ((uint32_t)((E + 7) & 0xF) << 3) | (mant & 7u));
}

void rko_quantize_rows_mxgolden(const float* x, int64_t rows, int64_t cols, uint8_t* codes, uint8_t* scales) {
  const int64_t nb = cols / 32;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t bi = 0; bi < nb; bi++) {
      const float* v = x + r * cols + bi * 32;
      float amax = 0.0f;
      for (int j = 0; j < 32; j++) amax = std::max(amax, std::fabs(v[j]));
      int sc = 0;
      if (amax != 0.0f) {
        sc = (int)((f32_bits(amax) >> 23) & 0xFFu) - 8;          // floor(log2 amax) - 8 + 127
        sc = std::min(std::max(sc, 0), 254);
      }
      scales[r * nb + bi] = (uint8_t)sc;
      const float scale = e8m0_decode((uint8_t)sc);
      for (int j = 0; j < 32; j++) codes[r * cols + bi * 32 + j] = e4m3_code_mxgolden(v[j] / scale);
    }
}

// RoPE, HF Llama rotate-half form with half-width caches (lib/golden/golden.py:229-236, rope_apply):
// out[:, :half] = c0 * cos - c1 * sin, out[:, half:] = c1 * cos + c0 * sin, every product and sum rounded to
// fp32 on its own (numpy float32 arithmetic: no fused multiply-add).  Row r uses cache row pos[r].
void rko_rope_rows(const float* x, int64_t rows, int64_t d, const int32_t* pos, const float* cos_h,
                   const float* sin_h, float* out) {
  const int64_t half = d / 2;
  for (int64_t r = 0; r < rows; r++) {
    const float* c = cos_h + (int64_t)pos[r] * half;
    const float* s = sin_h + (int64_t)pos[r] * half;
    for (int64_t i = 0; i < half; i++) {
      const volatile float c0 = x[r * d + i], c1 = x[r * d + half + i];
      const volatile float a = c0 * c[i], b = c1 * s[i], e = c1 * c[i], f = c0 * s[i];   // volatile: no contraction
      out[r * d + i] = a - b;
      out[r * d + half + i] = e + f;
    }
  }
}

// Row RMSNorm in the reference's fp32 path, lib/golden/golden.py:203-216 (rmsnorm): the sum of squares is
// accumulated in index order, every product and sum rounded to fp32 on its own; mean = ss / K;
// rms = 1 / sqrt(mean + eps) with the square root correctly rounded to fp32 (the golden takes it in double and
// rounds, which gives the same fp32) and a correctly rounded fp32 division; out = (x * rms) * gamma, two roundings.
void rko_rmsnorm_rows(const float* x, int64_t rows, int64_t K, const float* gamma, float eps, float* out) {
  for (int64_t r = 0; r < rows; r++) {
    const float* row = x + r * K;
    volatile float ss = 0.0f;                      // volatile: no contraction, no reassociation
    for (int64_t k = 0; k < K; k++) { const volatile float sq = row[k] * row[k]; ss = ss + sq; }
    const volatile float mean = ss / (float)K;
    const volatile float me = mean + eps;
    const volatile float root = (float)std::sqrt((double)me);
    const volatile float rms = 1.0f / root;
    for (int64_t k = 0; k < K; k++) { const volatile float t = row[k] * rms; out[r * K + k] = t * gamma[k]; }
  }
}

void rko_dequant_rows(const uint8_t* codes, const uint8_t* scales, int64_t rows, int64_t cols,
                      int fmt, float* out) {
  const Fmt& f = kFmt[fmt];
  const int64_t nb = (cols + 31) / 32;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++)
      out[r * cols + c] = decode_elem(codes[r * cols + c], f) * e8m0_decode(scales[r * nb + c / 32]);
}
void rko_dequant_cols(const uint8_t* codes, const uint8_t* scales, int64_t rows, int64_t cols,
                      int fmt, float* out) {
  const Fmt& f = kFmt[fmt];
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++)
      out[r * cols + c] = decode_elem(codes[r * cols + c], f) * e8m0_decode(scales[(r / 32) * cols + c]);
}

// Re-block V from scales along d to scales along the keys: decode every element
// exactly (code * 2^(s-127)), then apply the lib/golden block rule down each
// column.  This is what lets a V that was quantized "block-32 along d" feed a
// P.V contraction whose block scales must run along the keys, as the reference's
// own V does.  in: codes [S][d], scales [S][d/32]; out: codes [S][d], scales [ceil(S/32)][d].
void rko_rebase_v(const uint8_t* codes, const uint8_t* scales, int64_t S, int64_t d, int fmt,
                  uint8_t* out_codes, uint8_t* out_scales) {
  std::vector<float> tmp((size_t)(S * d));
  rko_dequant_rows(codes, scales, S, d, fmt, tmp.data());
  rko_quantize_cols(tmp.data(), S, d, fmt, out_codes, out_scales, 1);
}

// ------------------------------ MX matmul, hardware accumulate semantics --------------------------
// The reference's golden for the MX-Gemmini matmul models the mesh itself (lib/golden/mx_golden.cpp:114-144): per
// 16-deep K step the partial sum flows down a systolic column whose accumulator widens as it goes (ACC_E / ACC_M,
// :44-48), every product is truncated to 3 fraction bits and saturated at 448 (mx_product_quantize_trunc,
// lib/golden/mx_fp_math.h:44-71), both addends are re-rounded to the stage's format before an exact add that is
// rounded again (fp_quantize_rne / fp_add_exact, :120-189); after 16 stages the sum is scaled by the two E8M0 codes
// of the 32-element K group and added into a bf16 accumulator.  Restated here in integer form; pinned against the
// reference's own program built under oracle/_ref (tests/test_oracle_golden.py).

// x rounded to the nearest value of a float format with `ebits` exponent and `mbits` fraction bits (ties to even),
// gradual underflow, overflow to infinity; zero results are +0 (mx_fp_math.h:120-172).
static float quantize_rne_fmt(float x, int ebits, int mbits) {
  if (x != x) return std::numeric_limits<float>::quiet_NaN();
  if (std::isinf(x) || x == 0.0f) return x == 0.0f ? 0.0f : x;
  uint32_t b; std::memcpy(&b, &x, 4);
  const bool neg = (b >> 31) != 0;
  const int e_raw = (int)((b >> 23) & 0xFF);
  const uint64_t sig = e_raw ? ((b & 0x7FFFFFu) | 0x800000u) : (b & 0x7FFFFFu);   // |x| = sig * 2^ex
  const int ex = (e_raw ? e_raw : 1) - 150;
  const int top = 63 - __builtin_clzll(sig);
  const int bias = (1 << (ebits - 1)) - 1, emin = 1 - bias, emax = bias;
  const int E = ex + top;                                    // floor(log2 |x|)
  const int qexp = std::max(E, emin) - mbits;                // exponent of the format's quantum at this magnitude
  const int sh = qexp - ex;
  uint64_t q;
  if (sh <= 0) q = sig << (-sh);
  else if (sh >= 40) q = 0;
  else {
    const uint64_t rem = sig & ((1ull << sh) - 1), half = 1ull << (sh - 1);
    q = sig >> sh;
    if (rem > half || (rem == half && (q & 1))) ++q;
  }
  if (q == 0) return 0.0f;
  const int qtop = 63 - __builtin_clzll(q);
  if (qtop + qexp > emax) return neg ? -std::numeric_limits<float>::infinity() : std::numeric_limits<float>::infinity();
  const float r = std::ldexp((float)q, qexp);
  return neg ? -r : r;
}

static float add_then_round(float x, float y, int ebits, int mbits) {     // fp_add_exact, mx_fp_math.h:179-189
  if (x != x || y != y) return std::numeric_limits<float>::quiet_NaN();
  if (std::isinf(x) || std::isinf(y)) {
    if (std::isinf(x) && std::isinf(y) && std::signbit(x) != std::signbit(y)) return std::numeric_limits<float>::quiet_NaN();
    return std::isinf(x) ? x : y;
  }
  if (x == 0.0f) return y;
  if (y == 0.0f) return x;
  return quantize_rne_fmt(x + y, ebits, mbits);
}

// bf16 rounding as the reference does it: zero magnitudes come out as +0 (mx_fp_math.h:11-35)
static float bf16_round_ref(float x) {
  uint16_t bits;
  const float r = bf16_round_to_f32(x, &bits);
  return (r == 0.0f) ? 0.0f : r;
}

// A codes [M][K], B codes [K][N] (E4M3), SA [K/32][M], SB [K/32][N] (E8M0) -> C bf16 bits [M][N].
// M, N, K multiples of 16, K of 32.  A NaN comes out as 0x7FC0.
void rko_mx_gemm_hw(const uint8_t* A, const uint8_t* B, const uint8_t* SA, const uint8_t* SB, int M, int N, int K,
                    uint16_t* C, int nthreads) {
  static const int kAccE[16] = {4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 8};
  static const int kAccM[16] = {4, 4, 4, 4, 4, 4, 4, 4, 5, 5, 6, 6, 6, 6, 6, 7};
  const Fmt& f8 = kFmt[0];
  parallel_for((int64_t)M * N, nthreads, [&](int64_t idx) {
    const int m = (int)(idx / N), n = (int)(idx % N);
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 16) {
      float ct = 0.0f;
      for (int kk = 0; kk < 16; kk++) {
        const float prod = decode_elem(A[(size_t)m * K + k0 + kk], f8) * decode_elem(B[(size_t)(k0 + kk) * N + n], f8);
        float pq;
        if (prod == 0.0f) pq = 0.0f;
        else {
          uint32_t pb; std::memcpy(&pb, &prod, 4);
          pb &= 0xFFF00000u;                                   // truncate to 3 fraction bits
          std::memcpy(&pq, &pb, 4);
          if (std::fabs(pq) > 448.0f) pq = std::signbit(pq) ? -448.0f : 448.0f;
        }
        const int ae = kAccE[kk], am = kAccM[kk];
        const float cq = (ae == 8) ? bf16_round_ref(ct) : quantize_rne_fmt(ct, ae, am);
        const float pr = (ae == 8) ? bf16_round_ref(pq) : quantize_rne_fmt(pq, ae, am);
        ct = add_then_round(cq, pr, ae, am);
      }
      const int g = k0 / 32;
      int e = (int)SA[(size_t)g * M + m] + (int)SB[(size_t)g * N + n] - 127;
      e = e < 0 ? 0 : (e > 254 ? 254 : e);
      const float scaled = bf16_round_ref(ct * e8m0_decode((uint8_t)e));
      acc = bf16_round_ref(add_then_round(bf16_round_ref(acc), bf16_round_ref(scaled), 8, 7));
    }
    uint16_t bits;
    const float r = bf16_round_to_f32(acc, &bits);
    if (r != r) bits = 0x7FC0;
    else if (r == 0.0f) bits = 0;
    C[idx] = bits;
  });
}

// ------------------------------ prefill attention --------------------------
struct rko_prefill_args {
  const uint8_t* q;        // [B][H][Sq][d] codes
  const uint8_t* k;        // [B][Hkv][Skv][d]
  const uint8_t* v;        // [B][Hkv][Skv][d]
  const uint8_t* q_scale;  // [B][H][Sq][d/32]
  const uint8_t* k_scale;  // [B][Hkv][Skv][d/32]
  const uint8_t* v_scale;  // axis d: [B][Hkv][Skv][d/32]; axis keys: [B][Hkv][ceil(Skv/32)][d]
  int32_t B, H, Hkv, Sq, Skv, d;
  int32_t q_pos0, causal, window;   // window 0 = off
  float softcap;                    // 0 = off
  float softmax_scale;
  int32_t q_fmt, kv_fmt;
  int32_t v_scale_axis;             // 0 = keys (reference layout), 1 = d (re-based first)
  int32_t block_n;                  // keys per online-softmax step
  int32_t nthreads;
  int64_t slice_begin, slice_end;   // flattened (b*H+h) range to compute, end<=0 = all
  float* o_f32;                     // [B][H][Sq][d] or null
  uint16_t* o_bf16;                 // [B][H][Sq][d] or null
  float* lse;                       // [B][H][Sq] natural-log LSE, or null
  // optional stage dumps for one (b,h) slice = dump_slice (tests only)
  int64_t dump_slice;
  float* dump_s;                    // [Sq][Skv] scaled (+capped, masked=-inf) scores
  uint8_t* dump_p_codes;            // [Sq][Skv]
  uint8_t* dump_p_scales;           // [Sq][Skv/32]
  float* dump_m;                    // [Sq] final running max
  float* dump_l;                    // [Sq] final l
  // Where the numbers are rounded.  0 (the build target): fp32 softmax state, exp and accumulation, one bf16 rounding
  // of O at the end.  1: every intermediate re-rounded to bf16 where the reference's model does it (q_bf16 of
  // kernels/flash_attention_mx_gqa/flash_attention_model.py:222-246): the matmul results S and P.V, S * scale, corr,
  // p, the block's sum of p, l, the O accumulator after every key block, and O / l.
  int32_t bf16_faithful;
};

// Streaming MX attention for one (b,h) slice.  Structure:
//   kernels/flash_attention_mx_gqa/flash_attention_model.py:205-248 (causal GQA),
//   kernels/flash_attention_mx_gemma/flash_attention_model.py:317-372 (cap before
//   mask and max; sliding window; masked p forced to 0),
//   P requant kernels/flash_attention_mx_gqa/flash_mx_impl.hpp:356-387,
//   l accumulated from the unquantised p (:380), deferred 1/l with the l<=0
//   guard (flash_attention_model.py:244-246).
// Deliberate deviations (asked for by the build target): softmax state, exp and
// both contractions in fp32 instead of bf16 / the mesh's reduced precision.
static void prefill_slice(const rko_prefill_args& a, int64_t slice) {
  const int b = (int)(slice / a.H), h = (int)(slice % a.H);
  const int grp = a.H / a.Hkv, kv = h / grp;     // flash_attention_model.py:213-215
  const int Sq = a.Sq, Skv = a.Skv, d = a.d, nbd = d / 32;
  const Fmt& fq = kFmt[a.q_fmt];
  const Fmt& fkv = kFmt[a.kv_fmt];
  const int64_t qoff = ((int64_t)b * a.H + h) * Sq, koff = ((int64_t)b * a.Hkv + kv) * Skv;

  std::vector<float> Q((size_t)Sq * d), K((size_t)Skv * d), V((size_t)Skv * d);
  for (int i = 0; i < Sq; i++)
    for (int c = 0; c < d; c++)
      Q[(size_t)i * d + c] = decode_elem(a.q[(qoff + i) * d + c], fq) * e8m0_decode(a.q_scale[(qoff + i) * nbd + c / 32]);
  for (int i = 0; i < Skv; i++)
    for (int c = 0; c < d; c++)
      K[(size_t)i * d + c] = decode_elem(a.k[(koff + i) * d + c], fkv) * e8m0_decode(a.k_scale[(koff + i) * nbd + c / 32]);
  {
    const int64_t nkb = (Skv + 31) / 32;
    if (a.v_scale_axis == 1) {
      std::vector<uint8_t> vc((size_t)Skv * d), vs((size_t)nkb * d);
      rko_rebase_v(a.v + koff * d, a.v_scale + koff * nbd, Skv, d, a.kv_fmt, vc.data(), vs.data());
      rko_dequant_cols(vc.data(), vs.data(), Skv, d, a.kv_fmt, V.data());
    } else {
      rko_dequant_cols(a.v + koff * d, a.v_scale + ((int64_t)b * a.Hkv + kv) * nkb * d, Skv, d, a.kv_fmt, V.data());
    }
  }

  const bool dump = (a.dump_slice == slice);
  const bool bf = a.bf16_faithful != 0;
  auto rb = [bf](float x) { uint16_t bits; return bf ? bf16_round_to_f32(x, &bits) : x; };   // q_bf16 in faithful mode
  const int bn = a.block_n;
  const float NEG_INF = -std::numeric_limits<float>::infinity();
  std::vector<float> s(bn), p(bn), pq(bn), o(d);
  for (int i = 0; i < Sq; i++) {
    const int q_pos = a.q_pos0 + i;
    std::fill(o.begin(), o.end(), 0.0f);
    float m_run = NEG_INF, l_run = 0.0f;
    // blocks wholly above the diagonal are skipped (flash_attention_model.py:182-186);
    // per row that is every block whose first key is past q_pos.
    for (int k0 = 0; k0 < Skv; k0 += bn) {
      const int nk = std::min(bn, Skv - k0);
      if (a.causal && k0 > q_pos) {
        if (dump) for (int c = 0; c < nk; c++) {
          a.dump_s[(size_t)i * Skv + k0 + c] = NEG_INF;
          a.dump_p_codes[(size_t)i * Skv + k0 + c] = 0;
          if (c % 32 == 0) a.dump_p_scales[(size_t)i * ((Skv + 31) / 32) + (k0 + c) / 32] = 0;
        }
        continue;
      }
      float bmax = NEG_INF;
      for (int c = 0; c < nk; c++) {
        // faithful mode: the mesh returns S in bf16 (mx_gemm, flash_attention_model.py:76-86), then q_bf16(S * scale) (:226)
        float sv = rb(rb(dot_f32(&Q[(size_t)i * d], &K[(size_t)(k0 + c) * d], d)) * a.softmax_scale);
        if (a.softcap > 0.0f) sv = rb(a.softcap * std::tanh(sv / a.softcap));   // cap before mask/max
        const int kpos = k0 + c;
        bool msk = a.causal && kpos > q_pos;
        if (a.window > 0) msk = msk || (kpos + a.window <= q_pos);
        s[c] = msk ? NEG_INF : sv;
        bmax = std::max(bmax, s[c]);
        if (dump) a.dump_s[(size_t)i * Skv + kpos] = s[c];
      }
      const float m_new = std::max(m_run, bmax);
      // corr = exp(m_old - m_new); 1 while nothing has been accumulated yet.
      const float corr = (m_run == NEG_INF) ? 1.0f : rb(std::exp(m_run - m_new));
      float lsum = 0.0f;
      for (int c = 0; c < nk; c++) {
        p[c] = (s[c] == NEG_INF) ? 0.0f : rb(std::exp(s[c] - m_new));   // masked -> exactly 0
        lsum += p[c];
      }
      l_run = rb(l_run * corr + rb(lsum));
      std::vector<float> pv;
      if (bf) { pv.assign(d, 0.0f); } else { for (int c = 0; c < d; c++) o[c] *= corr; }
      for (int g0 = 0; g0 < nk; g0 += 32) {
        const int ng = std::min(32, nk - g0);
        float pmax = 0.0f;
        for (int c = 0; c < ng; c++) pmax = std::max(pmax, p[g0 + c]);
        const uint8_t sc = p_block_scale_code(pmax);
        const float sf = e8m0_decode(sc);
        if (dump) a.dump_p_scales[(size_t)i * ((Skv + 31) / 32) + (k0 + g0) / 32] = sc;
        for (int c = 0; c < ng; c++) {
          const uint8_t code = p_code(p[g0 + c], sc);
          if (dump) a.dump_p_codes[(size_t)i * Skv + k0 + g0 + c] = code;
          pq[g0 + c] = decode_elem(code, kFmt[0]) * sf;
        }
      }
      float* acc = bf ? pv.data() : o.data();
      for (int c = 0; c < nk; c++) {
        const float w = pq[c];
        if (w == 0.0f) continue;
        const float* vr = &V[(size_t)(k0 + c) * d];
        for (int e = 0; e < d; e++) acc[e] += w * vr[e];
      }
      // faithful mode: P.V comes back from the mesh in bf16 and the accumulator is re-rounded after every block (:241)
      if (bf) for (int e = 0; e < d; e++) o[e] = rb(o[e] * corr + rb(pv[e]));
      m_run = m_new;
    }
    const float safe_l = l_run > 0.0f ? l_run : 1.0f;
    const float inv = 1.0f / safe_l;
    for (int c = 0; c < d; c++) {
      const float val = bf ? rb(o[c] / safe_l) : o[c] * inv;   // q_bf16(O / safe_l), flash_attention_model.py:246
      if (a.o_f32) a.o_f32[(qoff + i) * d + c] = val;
      if (a.o_bf16) { uint16_t bb; bf16_round_to_f32(val, &bb); a.o_bf16[(qoff + i) * d + c] = bb; }
    }
    if (a.lse) a.lse[qoff + i] = (l_run > 0.0f) ? m_run + std::log(l_run) : NEG_INF;
    if (dump) { a.dump_m[i] = m_run; a.dump_l[i] = l_run; }
  }
}

int rko_attn_prefill(const rko_prefill_args* a) {
  if (a->d % 32 || a->H % a->Hkv || a->block_n % 32 || a->block_n <= 0) return -1;
  int64_t s0 = 0, s1 = (int64_t)a->B * a->H;
  if (a->slice_end > 0) { s0 = a->slice_begin; s1 = a->slice_end; }
  parallel_for(s1 - s0, a->nthreads, [&](int64_t i) { prefill_slice(*a, s0 + i); });
  return 0;
}

// Unquantised fp32 softmax attention, the reference's attention_reference*
// (kernels/flash_attention_mx_gqa/flash_attention_model.py:189-202,
//  kernels/flash_attention_mx_gemma/flash_attention_model.py:299-314).
void rko_attn_fp32_ref(const float* Q, const float* K, const float* V, int B, int H, int Hkv,
                       int Sq, int Skv, int d, int q_pos0, int causal, int window, float softcap,
                       float scale, float* O, int nthreads) {
  parallel_for((int64_t)B * H, nthreads, [&](int64_t sl) {
    const int b = (int)(sl / H), h = (int)(sl % H), kv = h / (H / Hkv);
    const float* q = Q + sl * Sq * d;
    const float* k = K + ((int64_t)b * Hkv + kv) * Skv * d;
    const float* v = V + ((int64_t)b * Hkv + kv) * Skv * d;
    std::vector<float> s(Skv);
    for (int i = 0; i < Sq; i++) {
      float m = -std::numeric_limits<float>::infinity();
      for (int c = 0; c < Skv; c++) {
        float x = dot_f32(q + (size_t)i * d, k + (size_t)c * d, d) * scale;
        if (softcap > 0) x = softcap * std::tanh(x / softcap);
        bool msk = causal && c > q_pos0 + i;
        if (window > 0) msk = msk || (c + window <= q_pos0 + i);
        s[c] = msk ? -std::numeric_limits<float>::infinity() : x;
        m = std::max(m, s[c]);
      }
      float l = 0;
      float* o = O + (sl * Sq + i) * d;
      for (int e = 0; e < d; e++) o[e] = 0;
      for (int c = 0; c < Skv; c++) {
        if (s[c] == -std::numeric_limits<float>::infinity()) continue;
        const float p = std::exp(s[c] - m);
        l += p;
        for (int e = 0; e < d; e++) o[e] += p * v[(size_t)c * d + e];
      }
      const float inv = l > 0 ? 1.0f / l : 1.0f;
      for (int e = 0; e < d; e++) o[e] *= inv;
    }
  });
}

// ------------------------------ decode attention ---------------------------
// Single-token attention over an MX KV cache.  The reference has no decode
// attention kernel; this is its prefill semantics at Sq = 1 with the query at
// position kv_len-1 (so every cached key is visible), GQA head map h -> h/grp
// (kernels/flash_attention_mx_gqa/flash_attention_model.py:213-215), K and V
// decoded exactly, fp32 softmax, no P requant, one pass over the keys.
struct rko_decode_args {
  const uint16_t* q;       // bf16 [B][H][d]
  const uint8_t* k;        // [B][Hkv][L][d]
  const uint8_t* v;        // [B][Hkv][L][d]
  const uint8_t* k_scale;  // [B][Hkv][L][d/32]
  const uint8_t* v_scale;  // [B][Hkv][L][d/32]
  const int32_t* kv_len;   // [B] or null (= L)
  int32_t B, H, Hkv, L, d;
  float softmax_scale;
  int32_t kv_fmt;
  int32_t nthreads;
  int64_t unit_begin, unit_end;  // flattened (b*Hkv+kv) range, end<=0 = all
  float* o_f32;            // [B][H][d] or null
  uint16_t* o_bf16;        // [B][H][d] or null
  float* lse;              // [B][H] or null
};

static void decode_unit(const rko_decode_args& a, int64_t unit) {
  const int b = (int)(unit / a.Hkv), kv = (int)(unit % a.Hkv);
  const int grp = a.H / a.Hkv, d = a.d, nbd = d / 32;
  const int len = a.kv_len ? a.kv_len[b] : a.L;
  const Fmt& f = kFmt[a.kv_fmt];
  const int64_t base = ((int64_t)b * a.Hkv + kv) * a.L;
  std::vector<float> q((size_t)grp * d), o((size_t)grp * d, 0.0f), m(grp, -std::numeric_limits<float>::infinity()), l(grp, 0.0f);
  for (int g = 0; g < grp; g++)
    for (int c = 0; c < d; c++)
      q[(size_t)g * d + c] = bits_f32((uint32_t)a.q[((int64_t)b * a.H + kv * grp + g) * d + c] << 16);
  std::vector<float> kr(d), vr(d);
  for (int t = 0; t < len; t++) {
    for (int c = 0; c < d; c++) {
      kr[c] = decode_elem(a.k[(base + t) * d + c], f) * e8m0_decode(a.k_scale[(base + t) * nbd + c / 32]);
      vr[c] = decode_elem(a.v[(base + t) * d + c], f) * e8m0_decode(a.v_scale[(base + t) * nbd + c / 32]);
    }
    for (int g = 0; g < grp; g++) {
      const float s = dot_f32(&q[(size_t)g * d], kr.data(), d) * a.softmax_scale;
      const float m_new = std::max(m[g], s);
      const float corr = (m[g] == -std::numeric_limits<float>::infinity()) ? 1.0f : std::exp(m[g] - m_new);
      const float p = std::exp(s - m_new);
      l[g] = l[g] * corr + p;
      float* og = &o[(size_t)g * d];
      for (int c = 0; c < d; c++) og[c] = og[c] * corr + p * vr[c];
      m[g] = m_new;
    }
  }
  for (int g = 0; g < grp; g++) {
    const int64_t oh = ((int64_t)b * a.H + kv * grp + g);
    const float inv = l[g] > 0 ? 1.0f / l[g] : 1.0f;
    for (int c = 0; c < d; c++) {
      const float val = o[(size_t)g * d + c] * inv;
      if (a.o_f32) a.o_f32[oh * d + c] = val;
      if (a.o_bf16) { uint16_t bb; bf16_round_to_f32(val, &bb); a.o_bf16[oh * d + c] = bb; }
    }
    if (a.lse) a.lse[oh] = l[g] > 0 ? m[g] + std::log(l[g]) : -std::numeric_limits<float>::infinity();
  }
}

int rko_attn_decode(const rko_decode_args* a) {
  if (a->d % 32 || a->H % a->Hkv) return -1;
  int64_t u0 = 0, u1 = (int64_t)a->B * a->Hkv;
  if (a->unit_end > 0) { u0 = a->unit_begin; u1 = a->unit_end; }
  parallel_for(u1 - u0, a->nthreads, [&](int64_t i) { decode_unit(*a, u0 + i); });
  return 0;
}

int rko_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
