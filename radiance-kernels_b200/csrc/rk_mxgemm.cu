// MX matmul in the hardware-accumulate semantics of the MX-Gemmini mesh: the golden of the reference's GEMM and
// batched-decode projection kernels (kernels/gemm_mxgemmini*, kernels/gemv_batched_fp8_m128; golden program
// lib/golden/mx_golden.cpp:114-144).  The mesh does not accumulate in fp32: per 16-deep K step the partial sum
// passes through 16 accumulator stages of growing width (exponent bits 4 ... 8, fraction bits 4 ... 7), every
// product is truncated to 3 fraction bits and saturated at 448, both addends are re-rounded to the stage's
// format, and after the 16th stage the sum is scaled by the two E8M0 codes of its 32-element K group and added
// into a bf16 accumulator.  A tensor core cannot reproduce that rounding sequence, so this is integer / fp32
// work on the CUDA cores: one thread per output element walks K in order (the order is the definition).
// A [M][K] and B [K][N] are E4M3 codes, SA [K/32][M], SB [K/32][N] E8M0 codes, C [M][N] bf16 bits.
// Bound: ALU (about 30 integer operations per multiply-accumulate); bytes are negligible.
#include <cuda_runtime.h>

#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

namespace {

constexpr uint32_t kQuietNaN = 0x7FC00000u;

RK_DEVINL bool is_nan_bits(uint32_t b) { return (b & 0x7FFFFFFFu) > 0x7F800000u; }
RK_DEVINL bool is_inf_bits(uint32_t b) { return (b & 0x7FFFFFFFu) == 0x7F800000u; }

// x (fp32 bit pattern) rounded to the nearest value of a float format with `ebits` exponent and `mbits` fraction
// bits, ties to even, gradual underflow, overflow to infinity; a zero result is +0
// (fp_quantize_rne_scalar, lib/golden/mx_fp_math.h:120-172).
RK_DEVINL uint32_t quantize_rne_fmt(uint32_t b, int ebits, int mbits) {
  if (is_nan_bits(b)) return kQuietNaN;
  if (is_inf_bits(b)) return b;
  const uint32_t mag = b & 0x7FFFFFFFu;
  if (mag == 0u) return 0u;
  const uint32_t sign = b & 0x80000000u;
  const int e_raw = (int)(mag >> 23);
  const uint32_t sig = e_raw ? ((mag & 0x7FFFFFu) | 0x800000u) : (mag & 0x7FFFFFu);   // |x| = sig * 2^ex
  const int ex = (e_raw ? e_raw : 1) - 150;
  const int top = 31 - __clz(sig);
  const int bias = (1 << (ebits - 1)) - 1, emin = 1 - bias, emax = bias;
  const int E = ex + top;
  const int qexp = max(E, emin) - mbits;                      // exponent of the format's quantum at this magnitude
  const int sh = qexp - ex;
  const uint32_t q = sh <= 0 ? (sig << (-sh)) : round_shift(sig, sh);
  if (q == 0u) return 0u;
  const int qtop = 31 - __clz(q);
  if (qtop + qexp > emax) return sign | 0x7F800000u;
  // q * 2^qexp is a normal or subnormal fp32: the conversion and the scaling below are exact
  return sign | __float_as_uint(ldexpf((float)q, qexp));
}

// fp_add_exact, lib/golden/mx_fp_math.h:179-189
RK_DEVINL uint32_t add_then_round(uint32_t x, uint32_t y, int ebits, int mbits) {
  if (is_nan_bits(x) || is_nan_bits(y)) return kQuietNaN;
  if (is_inf_bits(x) || is_inf_bits(y)) {
    if (is_inf_bits(x) && is_inf_bits(y) && ((x ^ y) >> 31)) return kQuietNaN;
    return is_inf_bits(x) ? x : y;
  }
  if ((x & 0x7FFFFFFFu) == 0u) return y;
  if ((y & 0x7FFFFFFFu) == 0u) return x;
  return quantize_rne_fmt(__float_as_uint(__fadd_rn(__uint_as_float(x), __uint_as_float(y))), ebits, mbits);
}

// fp32 -> bf16 -> fp32 as the reference rounds (f32_to_bf16_rne, lib/golden/mx_fp_math.h:11-28): nearest even on the
// bit pattern, zero magnitudes canonicalised to +0, a NaN keeps a quiet payload
RK_DEVINL uint32_t bf16_round_bits(uint32_t b) {
  if ((b & 0x7FFFFFFFu) == 0u) return 0u;
  if (((b >> 23) & 0xFFu) == 0xFFu) {
    uint32_t hi = b >> 16;
    if ((b & 0x7FFFFFu) && !(hi & 0x40u)) hi |= 0x40u;
    return hi << 16;
  }
  const uint32_t hi = (b + 0x7FFFu + ((b >> 16) & 1u)) >> 16;
  return (hi & 0x7FFFu) ? (hi << 16) : 0u;
}

__constant__ int8_t kAccFrac[16] = {4, 4, 4, 4, 4, 4, 4, 4, 5, 5, 6, 6, 6, 6, 6, 7};   // ACC_M, mx_golden.cpp:47; ACC_E is 4 except 8 at the last stage

}  // namespace

__global__ void __launch_bounds__(256)
mx_gemm_hw_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B, const uint8_t* __restrict__ SA,
                  const uint8_t* __restrict__ SB, int M, int N, int K, uint16_t* __restrict__ C) {
  const int64_t total = (int64_t)M * N;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(idx / N), n = (int)(idx % N);         // consecutive threads: consecutive n (B, SB, C coalesced; A broadcast)
    uint32_t acc = 0u;                                        // the bf16 accumulator, as an fp32 bit pattern
    for (int k0 = 0; k0 < K; k0 += 16) {
      uint32_t ct = 0u;
      const uint4 a16 = *reinterpret_cast<const uint4*>(A + (size_t)m * K + k0);
      const uint32_t aw[4] = {a16.x, a16.y, a16.z, a16.w};
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const float a = decode_elem<0>((aw[kk >> 2] >> (8 * (kk & 3))) & 0xFFu);
        const float b = decode_elem<0>(B[(size_t)(k0 + kk) * N + n]);
        uint32_t pb = __float_as_uint(__fmul_rn(a, b));       // exact: two 4-bit significands
        if ((pb & 0x7FFFFFFFu) == 0u) pb = 0u;
        else {
          pb &= 0xFFF00000u;                                  // product truncated to 3 fraction bits ...
          if ((pb & 0x7FFFFFFFu) > 0x43E00000u) pb = (pb & 0x80000000u) | 0x43E00000u;   // ... and saturated at 448
        }
        const bool last = (kk == 15);
        const int ae = last ? 8 : 4, am = kAccFrac[kk];
        const uint32_t cq = last ? bf16_round_bits(ct) : quantize_rne_fmt(ct, ae, am);
        const uint32_t pq = last ? bf16_round_bits(pb) : quantize_rne_fmt(pb, ae, am);
        ct = add_then_round(cq, pq, ae, am);
      }
      const int g = k0 >> 5;
      int e = (int)SA[(size_t)g * M + m] + (int)SB[(size_t)g * N + n] - 127;
      e = e < 0 ? 0 : (e > 254 ? 254 : e);
      const uint32_t scaled = bf16_round_bits(__float_as_uint(__fmul_rn(__uint_as_float(ct), e8m0_to_f32((uint32_t)e))));
      acc = bf16_round_bits(add_then_round(bf16_round_bits(acc), bf16_round_bits(scaled), 8, 7));
    }
    const uint32_t out = bf16_round_bits(acc);
    C[idx] = is_nan_bits(out) ? (uint16_t)0x7FC0u : (uint16_t)(out >> 16);
  }
}

int launch_mx_gemm_hw(const uint8_t* A, const uint8_t* B, const uint8_t* SA, const uint8_t* SB, int M, int N, int K,
                      uint16_t* C, cudaStream_t st) {
  const int64_t total = (int64_t)M * N;
  if (total == 0) return RK_OK;
  const int64_t blocks = (total + 255) / 256;
  const int grid = (int)(blocks < (int64_t)num_sms() * 16 ? blocks : (int64_t)num_sms() * 16);
  mx_gemm_hw_kernel<<<grid, 256, 0, st>>>(A, B, SA, SB, M, N, K, C);
  return (int)cudaGetLastError();
}

}  // namespace rk
