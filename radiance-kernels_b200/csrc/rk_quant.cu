// MX block quantizer kernels (HBM-bound streaming kernels, no tensor cores).
//
//  quantize_rows   fp32 [rows][cols] -> codes + one E8M0 scale per 32 contiguous
//                  elements.  Same results as quantize_one_block,
//                  kernels/simt_quant/kernel.cpp:95-129 (golden:
//                  lib/golden/golden.py:118-170), bit for bit.  4 lanes share a
//                  block, each lane loads 2 x float4 and stores 8 packed codes.
//                  Algorithmic traffic 4 B in + 1 B + 1/32 B out per element.
//  quantize_keys   same rule with the blocks running down the rows (the key
//                  axis) of each matrix in a batch -- the reference's V layout
//                  (kernels/flash_attention_mx/gen_data.py:77).
//  rebase_v        codes+scales blocked along d -> decode exactly -> re-block
//                  along the keys.  Writes the scales either row-major
//                  [ceil(S/32)][d] or directly in the 512-byte scale-factor
//                  atoms the attention kernel copies into TMEM.
//  retile_*scales  row-major scales -> scale-factor atoms.
//
// Element encoding: the reference's integer round-shift encoder (rk::encode_rne)
// defines the result.  The hot loops use the hardware converter
// cvt.rn.satfinite.<fmt>x2.f32 instead, which verify_encoder_kernel proves equal
// to it on every finite fp32 input (all 2^32 bit patterns are swept in the GPU
// tests); blocks that hold a NaN or an infinity take the integer encoder.
#include <algorithm>

#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

// four floats -> four packed element codes (byte k = code of v[k]); finite inputs only
template <int FMT> RK_DEVINL uint32_t hw_encode4(float a, float b, float c, float d) {
  uint32_t r;
  if (FMT == 0)
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\tmov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  else if (FMT == 1)
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e5m2x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e5m2x2.f32 hi, %4, %3;\n\tmov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  else if (FMT == 4)      // 4-bit codes cross the interfaces one per byte: the integer encoder serves them
    r = encode_rne<4>(a) | (encode_rne<4>(b) << 8) | (encode_rne<4>(c) << 16) | (encode_rne<4>(d) << 24);
  else if (FMT == 2)
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e2m3x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e2m3x2.f32 hi, %4, %3;\n\tmov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  else
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e3m2x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e3m2x2.f32 hi, %4, %3;\n\tmov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}
template <int FMT> RK_DEVINL uint32_t ref_encode4(float a, float b, float c, float d) {
  return encode_rne<FMT>(a) | (encode_rne<FMT>(b) << 8) | (encode_rne<FMT>(c) << 16) | (encode_rne<FMT>(d) << 24);
}

// Sweeps fp32 bit patterns [first, first + count): counts inputs on which the hardware converter and the
// reference's integer encoder disagree (NaNs excluded: the kernels never hand one to the converter).
template <int FMT>
__global__ void verify_encoder_kernel(uint64_t first, uint64_t count, unsigned long long* mismatches, uint32_t* first_bad) {
  unsigned long long bad = 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t bits = (uint32_t)(first + i);
    if ((bits & 0x7FFFFFFFu) > 0x7F800000u) continue;
    const float x = __uint_as_float(bits);
    const uint32_t hw = hw_encode4<FMT>(x, 0.0f, 0.0f, 0.0f) & 0xFFu;
    const uint32_t rf = encode_rne<FMT>(x);
    if (hw != rf) { if (bad == 0) atomicMin(first_bad, bits); ++bad; }
  }
  if (bad) atomicAdd(mismatches, bad);
}

// BF16IN: the input is bf16 (one 16-byte load per chunk, widened exactly to fp32) instead of fp32.
// Offset of (row r of a 128-row tile, 32-element block kb of a 128-element
// chunk) inside a 512-byte scale-factor atom: 32 rows x 16 bytes, row r%32,
// byte (r/32)*4 + kb.  One tcgen05.cp 32x128b.warpx4 moves an atom to 4 TMEM
// columns (lane = r%32, column = r/32, byte = kb).
__host__ __device__ inline int sf_atom_offset(int r, int kb) { return (r & 31) * 16 + (r >> 5) * 4 + kb; }

// LAYOUT: where a block's scale byte goes -- 0 row-major [rows][d/32]; 1 group-major [batch][d/32][S]; 2 the
// 512-byte scale-factor atoms [batch][ceil(S/128)][ceil(d/128)][512] the attention kernel copies into TMEM
// (S = rows per matrix of the batch, nbd = d/32; both unused for layout 0).
template <int FMT, bool BF16IN = false, int LAYOUT = 0>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float4* __restrict__ x, int64_t nchunks,
                                                            uint2* __restrict__ codes, uint8_t* __restrict__ scales,
                                                            int64_t S = 0, int nbd = 0) {
  // chunk = 8 consecutive elements; 4 consecutive lanes = one 32-element block.
  // Warp-uniform loop bound: all 32 lanes run the shuffles even when the last
  // chunks of the array end inside this warp (nchunks is a multiple of 4, so a
  // 4-lane group is either wholly live or wholly idle).
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  // U chunks per trip, their loads issued together: the bf16 path loads half the bytes per chunk and gains 7 %
  // from two chunks in flight (measured); the fp32 path does not.
  constexpr int U = BF16IN ? 2 : 1;
  for (int64_t c0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c0 - lane < nchunks; c0 += U * stride) {
    float4 a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t c = c0 + u * stride;
      a[u] = make_float4(0.f, 0.f, 0.f, 0.f); b[u] = a[u];
      if (c < nchunks) {
        if (BF16IN) {
          const float4 raw = __ldcs(x + c);                      // 8 bf16
          const uint32_t w[4] = {__float_as_uint(raw.x), __float_as_uint(raw.y), __float_as_uint(raw.z), __float_as_uint(raw.w)};
          a[u] = make_float4(__uint_as_float(w[0] << 16), __uint_as_float(w[0] & 0xFFFF0000u), __uint_as_float(w[1] << 16), __uint_as_float(w[1] & 0xFFFF0000u));
          b[u] = make_float4(__uint_as_float(w[2] << 16), __uint_as_float(w[2] & 0xFFFF0000u), __uint_as_float(w[3] << 16), __uint_as_float(w[3] & 0xFFFF0000u));
        } else {
          a[u] = __ldcs(x + 2 * c); b[u] = __ldcs(x + 2 * c + 1);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t c = c0 + u * stride;
      if (c - lane >= nchunks) break;                            // warp-uniform: the shuffles below need whole warps
      const bool live = c < nchunks;
      const float v[8] = {a[u].x, a[u].y, a[u].z, a[u].w, b[u].x, b[u].y, b[u].z, b[u].w};
      float amax = 0.0f, nonfinite = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        amax = fmaxf(amax, fabsf(v[j]));          // a NaN never wins, as in the reference's compare loop
        nonfinite = fmaf(v[j], 0.0f, nonfinite);  // stays 0 unless an element is NaN or +-inf
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      if (!live) continue;
      uint32_t scode = 0; float p2 = 1.0f;
      if (amax > 0.0f) block_scale<FMT>(amax, scode, p2);
      uint32_t w0, w1;
      if (nonfinite == 0.0f) {
        w0 = hw_encode4<FMT>(v[0] * p2, v[1] * p2, v[2] * p2, v[3] * p2);
        w1 = hw_encode4<FMT>(v[4] * p2, v[5] * p2, v[6] * p2, v[7] * p2);
      } else {
        w0 = ref_encode4<FMT>(v[0] * p2, v[1] * p2, v[2] * p2, v[3] * p2);
        w1 = ref_encode4<FMT>(v[4] * p2, v[5] * p2, v[6] * p2, v[7] * p2);
      }
      __stcs(codes + c, make_uint2(w0, w1));
      if ((c & 3) == 0) {
        if (LAYOUT == 0) {
          scales[c >> 2] = (uint8_t)scode;
        } else {
          const int64_t bi = c >> 2, row = bi / nbd, mat = row / S;
          const int blk = (int)(bi % nbd), r = (int)(row % S);
          if (LAYOUT == 1) {
            scales[(mat * nbd + blk) * S + r] = (uint8_t)scode;
          } else {
            const int64_t ntile = (S + 127) / 128, dch = (nbd + 3) / 4;
            scales[((mat * ntile + r / 128) * dch + blk / 4) * 512 + sf_atom_offset(r & 127, blk & 3)] = (uint8_t)scode;
          }
        }
      }
    }
  }
}

// RoPE fused with the block quantizer, so that rotated Q / K never exist in HBM as fp32: rotate-half form with
// half-width caches (lib/golden/golden.py:229-236): out[:half] = c0 cos - c1 sin, out[half:] = c1 cos + c0 sin,
// every product and sum rounded on its own (no fused multiply-add, as numpy float32 does), then the lib/golden block
// rule along d.  chunk = 8 consecutive elements of the first half and their 8 partners of the second half; 4 lanes
// = one 32-element block in each half.  Row r uses cache row pos[r], or pos0 + r % seq_len when pos is null.
template <int FMT>
__global__ void __launch_bounds__(256) rope_quantize_rows_kernel(const float* __restrict__ x, int64_t rows, int d,
                                                                 const int32_t* __restrict__ pos, int seq_len, int pos0,
                                                                 const float* __restrict__ cos_h, const float* __restrict__ sin_h,
                                                                 uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const int half = d / 2, cpr = half / 8;                     // chunks per row (a multiple of 4)
  const int64_t nchunks = rows * cpr;
  const int lane = threadIdx.x & 31;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c - lane < nchunks; c += (int64_t)gridDim.x * blockDim.x) {
    const bool live = c < nchunks;
    const int64_t cc = live ? c : 0;
    const int64_t r = cc / cpr;
    const int i0 = (int)(cc % cpr) * 8;
    float o0[8], o1[8];
#pragma unroll
    for (int j = 0; j < 8; j++) { o0[j] = 0.0f; o1[j] = 0.0f; }
    if (live) {
      const int64_t at = pos ? (int64_t)pos[r] : (int64_t)pos0 + (r % seq_len);
      const float* xr = x + r * d;
      const float4 a0 = __ldcs(reinterpret_cast<const float4*>(xr + i0)), a1 = __ldcs(reinterpret_cast<const float4*>(xr + i0 + 4));
      const float4 b0 = __ldcs(reinterpret_cast<const float4*>(xr + half + i0)), b1 = __ldcs(reinterpret_cast<const float4*>(xr + half + i0 + 4));
      const float4 c0 = *reinterpret_cast<const float4*>(cos_h + at * half + i0), c1 = *reinterpret_cast<const float4*>(cos_h + at * half + i0 + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sin_h + at * half + i0), s1 = *reinterpret_cast<const float4*>(sin_h + at * half + i0 + 4);
      const float lo[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float hi[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int j = 0; j < 8; j++) {
        o0[j] = __fsub_rn(__fmul_rn(lo[j], cs[j]), __fmul_rn(hi[j], sn[j]));
        o1[j] = __fadd_rn(__fmul_rn(hi[j], cs[j]), __fmul_rn(lo[j], sn[j]));
      }
    }
    float am0 = 0.0f, am1 = 0.0f, nf = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      am0 = fmaxf(am0, fabsf(o0[j])); am1 = fmaxf(am1, fabsf(o1[j]));
      nf = fmaf(o0[j], 0.0f, nf); nf = fmaf(o1[j], 0.0f, nf);
    }
    am0 = fmaxf(am0, __shfl_xor_sync(0xffffffffu, am0, 1)); am1 = fmaxf(am1, __shfl_xor_sync(0xffffffffu, am1, 1));
    am0 = fmaxf(am0, __shfl_xor_sync(0xffffffffu, am0, 2)); am1 = fmaxf(am1, __shfl_xor_sync(0xffffffffu, am1, 2));
    if (!live) continue;
    uint32_t sc0 = 0, sc1 = 0; float p0 = 1.0f, p1 = 1.0f;
    if (am0 > 0.0f) block_scale<FMT>(am0, sc0, p0);
    if (am1 > 0.0f) block_scale<FMT>(am1, sc1, p1);
    uint32_t w[4];
    if (nf == 0.0f) {
      w[0] = hw_encode4<FMT>(o0[0] * p0, o0[1] * p0, o0[2] * p0, o0[3] * p0);
      w[1] = hw_encode4<FMT>(o0[4] * p0, o0[5] * p0, o0[6] * p0, o0[7] * p0);
      w[2] = hw_encode4<FMT>(o1[0] * p1, o1[1] * p1, o1[2] * p1, o1[3] * p1);
      w[3] = hw_encode4<FMT>(o1[4] * p1, o1[5] * p1, o1[6] * p1, o1[7] * p1);
    } else {
      w[0] = ref_encode4<FMT>(o0[0] * p0, o0[1] * p0, o0[2] * p0, o0[3] * p0);
      w[1] = ref_encode4<FMT>(o0[4] * p0, o0[5] * p0, o0[6] * p0, o0[7] * p0);
      w[2] = ref_encode4<FMT>(o1[0] * p1, o1[1] * p1, o1[2] * p1, o1[3] * p1);
      w[3] = ref_encode4<FMT>(o1[4] * p1, o1[5] * p1, o1[6] * p1, o1[7] * p1);
    }
    __stcs(reinterpret_cast<uint2*>(codes + r * d + i0), make_uint2(w[0], w[1]));
    __stcs(reinterpret_cast<uint2*>(codes + r * d + half + i0), make_uint2(w[2], w[3]));
    if ((i0 & 31) == 0) {
      scales[r * (d / 32) + i0 / 32] = (uint8_t)sc0;
      scales[r * (d / 32) + (half + i0) / 32] = (uint8_t)sc1;
    }
  }
}

// RMSNorm fused with the block quantizer: the prologue of the QKV projection (kernels/rmsnorm_qkv_fused), so that the
// normalized activation never exists in HBM as fp32.  Bit-exact with the reference's fp32 path
// (lib/golden/golden.py:203-216): the sum of squares runs in index order with every product and sum rounded on its
// own, mean = ss / K, rms = 1 / sqrt(mean + eps) (correctly rounded square root and division), y = (x * rms) * gamma.
// A warp owns 32 rows.  Per 32-column chunk it loads a 32 x 32 tile with coalesced row reads into shared memory;
// lane L then walks row L of the tile: in the first pass it extends its row's sequential sum, in the second pass
// the chunk is exactly one MX block of its row (amax, scale, codes: 32 bytes stored at once).
// UNIT: no block scale (code = E4M3(y) under 2^0, every scale byte 0x7F), the reference kernel's own choice
// (kernels/rmsnorm_qkv_fused/gen_data.py:33-41: the prologue owns the row scaling).
template <int FMT, bool BF16IN, bool UNIT>
__global__ void __launch_bounds__(256) rmsnorm_quantize_kernel(const void* __restrict__ xin, int64_t rows, int K,
                                                               const float* __restrict__ gamma, float eps,
                                                               uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  __shared__ float tile_all[8][32][33];
  __shared__ float gam_all[8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float (*tile)[33] = tile_all[warp];
  float* gam = gam_all[warp];
  const int64_t n_groups = (rows + 31) / 32;
  for (int64_t grp = (int64_t)blockIdx.x * 8 + warp; grp < n_groups; grp += (int64_t)gridDim.x * 8) {
    const int64_t row0 = grp * 32;
    auto load_tile = [&](int c0) {
#pragma unroll 8
      for (int i = 0; i < 32; ++i) {
        const int64_t r = row0 + i;
        float v = 0.0f;
        if (r < rows) {
          if (BF16IN) v = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(xin)[r * K + c0 + lane] << 16);
          else v = reinterpret_cast<const float*>(xin)[r * K + c0 + lane];
        }
        tile[i][lane] = v;
      }
    };
    float ss = 0.0f;
    for (int c0 = 0; c0 < K; c0 += 32) {
      load_tile(c0);
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 32; ++j) { const float v = tile[lane][j]; ss = __fadd_rn(ss, __fmul_rn(v, v)); }
      __syncwarp();
    }
    const float rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
    const int64_t r = row0 + lane;
    for (int c0 = 0; c0 < K; c0 += 32) {
      load_tile(c0);
      gam[lane] = gamma[c0 + lane];
      __syncwarp();
      float y[32];
      float amax = 0.0f, nonfinite = 0.0f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        y[j] = __fmul_rn(__fmul_rn(tile[lane][j], rms), gam[j]);
        amax = fmaxf(amax, fabsf(y[j]));
        nonfinite = fmaf(y[j], 0.0f, nonfinite);
      }
      __syncwarp();
      uint32_t scode = UNIT ? 127u : 0u; float p2 = 1.0f;
      if (!UNIT && amax > 0.0f) block_scale<FMT>(amax, scode, p2);
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        w[q] = (nonfinite == 0.0f) ? hw_encode4<FMT>(y[4 * q] * p2, y[4 * q + 1] * p2, y[4 * q + 2] * p2, y[4 * q + 3] * p2)
                                   : ref_encode4<FMT>(y[4 * q] * p2, y[4 * q + 1] * p2, y[4 * q + 2] * p2, y[4 * q + 3] * p2);
      if (r < rows) {
        uint4* dst = reinterpret_cast<uint4*>(codes + r * K + c0);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        scales[r * (K / 32) + c0 / 32] = (uint8_t)scode;
      }
    }
  }
}

// Append one token to a KV cache: row pos[b] of every (batch, KV head) of K and of V is quantized (blocks of 32
// along d, same rule and same code path as quantize_rows_kernel) and written in place.  chunk = 8 consecutive
// elements of one new row; 4 consecutive lanes = one block.  A position outside [0, L) is skipped.
template <int FMT>
__global__ void __launch_bounds__(128) kv_append_kernel(const float* __restrict__ k_new, const float* __restrict__ v_new,
                                                        int B, int H_kv, int L, int d, const int32_t* __restrict__ pos,
                                                        uint8_t* __restrict__ k_codes, uint8_t* __restrict__ k_scales,
                                                        uint8_t* __restrict__ v_codes, uint8_t* __restrict__ v_scales) {
  const int cpr = d / 8;                                     // chunks per row (a multiple of 4)
  const int64_t rows = (int64_t)B * H_kv, nchunks = 2 * rows * cpr;
  const int lane = threadIdx.x & 31;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c - lane < nchunks; c += (int64_t)gridDim.x * blockDim.x) {
    const bool live = c < nchunks;
    const int64_t cc = live ? c : 0;
    const int which = (int)(cc / (rows * cpr));              // 0 = K, 1 = V
    const int64_t row = (cc / cpr) % rows;
    const int col = (int)(cc % cpr) * 8;
    const float* src = (which ? v_new : k_new) + row * d + col;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b4 = a;
    if (live) { a = *reinterpret_cast<const float4*>(src); b4 = *reinterpret_cast<const float4*>(src + 4); }
    const float v[8] = {a.x, a.y, a.z, a.w, b4.x, b4.y, b4.z, b4.w};
    float amax = 0.0f, nonfinite = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) { amax = fmaxf(amax, fabsf(v[j])); nonfinite = fmaf(v[j], 0.0f, nonfinite); }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!live) continue;
    const int bidx = (int)(row / H_kv);
    const int at = pos[bidx];
    if (at < 0 || at >= L) continue;
    uint32_t scode = 0; float p2 = 1.0f;
    if (amax > 0.0f) block_scale<FMT>(amax, scode, p2);
    uint32_t w0, w1;
    if (nonfinite == 0.0f) {
      w0 = hw_encode4<FMT>(v[0] * p2, v[1] * p2, v[2] * p2, v[3] * p2);
      w1 = hw_encode4<FMT>(v[4] * p2, v[5] * p2, v[6] * p2, v[7] * p2);
    } else {
      w0 = ref_encode4<FMT>(v[0] * p2, v[1] * p2, v[2] * p2, v[3] * p2);
      w1 = ref_encode4<FMT>(v[4] * p2, v[5] * p2, v[6] * p2, v[7] * p2);
    }
    const int64_t crow = row * L + at;                        // row of the cache
    *reinterpret_cast<uint2*>((which ? v_codes : k_codes) + crow * d + col) = make_uint2(w0, w1);
    if ((col & 31) == 0) (which ? v_scales : k_scales)[crow * (d / 32) + col / 32] = (uint8_t)scode;
  }
}

// One thread = 4 adjacent columns x one 32-row block.
// ATOMS: scales go to the scale-factor atoms [batch][ceil(rows/128)][ceil(cols/128)][512] (byte = column n of the
// chunk, 32-key block kbi of the tile) instead of row-major [batch][ceil(rows/32)][cols].
template <int FMT, bool ATOMS = false>
__global__ void __launch_bounds__(128) quantize_keys_kernel(const float* __restrict__ x, int64_t batch, int64_t rows,
                                                            int64_t cols, uint8_t* __restrict__ codes,
                                                            uint8_t* __restrict__ scales) {
  const int64_t c4n = cols / 4, nkb = (rows + 31) / 32;
  const int64_t total = batch * nkb * c4n;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c4 = t % c4n, kb = (t / c4n) % nkb, bt = t / (c4n * nkb);
    const int64_t r0 = kb * 32;
    const int n = (int)min((int64_t)32, rows - r0);
    const float* xb = x + (bt * rows + r0) * cols + c4 * 4;
    float amax[4] = {0.f, 0.f, 0.f, 0.f};
    float nonfinite = 0.0f;
    for (int j = 0; j < n; j++) {
      const float4 v = *reinterpret_cast<const float4*>(xb + (int64_t)j * cols);
      amax[0] = fmaxf(amax[0], fabsf(v.x)); amax[1] = fmaxf(amax[1], fabsf(v.y));
      amax[2] = fmaxf(amax[2], fabsf(v.z)); amax[3] = fmaxf(amax[3], fabsf(v.w));
      nonfinite = fmaf(v.x, 0.0f, fmaf(v.y, 0.0f, fmaf(v.z, 0.0f, fmaf(v.w, 0.0f, nonfinite))));
    }
    uint32_t sc[4]; float p2[4];
#pragma unroll
    for (int q = 0; q < 4; q++) { sc[q] = 0; p2[q] = 1.0f; if (amax[q] > 0.0f) block_scale<FMT>(amax[q], sc[q], p2[q]); }
    uint8_t* cb = codes + (bt * rows + r0) * cols + c4 * 4;
    for (int j = 0; j < n; j++) {
      const float4 v = *reinterpret_cast<const float4*>(xb + (int64_t)j * cols);
      const uint32_t w = (nonfinite == 0.0f) ? hw_encode4<FMT>(v.x * p2[0], v.y * p2[1], v.z * p2[2], v.w * p2[3])
                                             : ref_encode4<FMT>(v.x * p2[0], v.y * p2[1], v.z * p2[2], v.w * p2[3]);
      *reinterpret_cast<uint32_t*>(cb + (int64_t)j * cols) = w;
    }
    if (!ATOMS) {
      *reinterpret_cast<uint32_t*>(scales + (bt * nkb + kb) * cols + c4 * 4) = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24);
    } else {
      const int64_t ntile = (rows + 127) / 128, dch = (cols + 127) / 128;
      uint8_t* atom = scales + ((bt * ntile + kb / 4) * dch + (c4 * 4) / 128) * 512;
#pragma unroll
      for (int q = 0; q < 4; q++) atom[((int)((c4 * 4 + q) & 31)) * 16 + ((int)(((c4 * 4 + q) & 127) >> 5)) * 4 + (int)(kb & 3)] = (uint8_t)sc[q];
    }
  }
}

// Exact value of element code `c` times 2^(s-127) as an fp32.  Normal codes under ordinary scales are
// placed by integer arithmetic (E4M3: bits = (mag + 8 s - 56) << 20); everything else (subnormal codes,
// scale codes near the ends of the range, the other formats) takes the generic multiply.
template <int FMT> RK_DEVINL float decode_scaled(uint32_t c, uint32_t s) {
  if (FMT == 0) {
    const uint32_t mag = c & 0x7Fu;
    if (mag >= 8u && s >= 16u && s <= 240u) return __uint_as_float(((c & 0x80u) << 24) | ((mag + 8u * s - 56u) << 20));
  }
  return decode_elem<FMT>(c) * e8m0_to_f32(s);
}

// Generic re-blocking of one (4 columns x up to 32 keys) block through fp32: decode every element exactly,
// block rule down each column, encode.  Used for formats other than E4M3 and for E4M3 blocks that hold
// subnormal codes or extreme scale codes.
template <int FMT>
__device__ __noinline__ void rebase_block_generic(const uint8_t* cb, const uint8_t* sb, int n, int64_t d, int64_t nbd,
                                                  uint8_t* ob, uint32_t (&sc)[4]) {
  float amax[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < n; j++) {
    const uint32_t cw = *reinterpret_cast<const uint32_t*>(cb + (int64_t)j * d);
    const uint32_t sj = sb[(int64_t)j * nbd];
#pragma unroll
    for (int q = 0; q < 4; q++) amax[q] = fmaxf(amax[q], fabsf(decode_scaled<FMT>((cw >> (8 * q)) & 0xFFu, sj)));
  }
  float p2[4];
#pragma unroll
  for (int q = 0; q < 4; q++) { sc[q] = 0; p2[q] = 1.0f; if (amax[q] > 0.0f) block_scale<FMT>(amax[q], sc[q], p2[q]); }
  for (int j = 0; j < n; j++) {
    const uint32_t cw = *reinterpret_cast<const uint32_t*>(cb + (int64_t)j * d);
    const uint32_t sj = sb[(int64_t)j * nbd];
    *reinterpret_cast<uint32_t*>(ob + (int64_t)j * d) =
        ref_encode4<FMT>(decode_scaled<FMT>(cw & 0xFFu, sj) * p2[0], decode_scaled<FMT>((cw >> 8) & 0xFFu, sj) * p2[1],
                         decode_scaled<FMT>((cw >> 16) & 0xFFu, sj) * p2[2], decode_scaled<FMT>(cw >> 24, sj) * p2[3]);
  }
}

// ---- re-blocking in integer arithmetic ------------------------------------------------------------------------
// Written out for E4M3 (the other formats differ in the constants of RebaseT): a normal code c (magnitude bits
// mag = c & 0x7F >= 8) under scale code s has the value (1 + m/8) * 2^(L/8 - 134) with L = mag + 8 s (m = L & 7),
// so the largest |value| of a block is the largest L, the block rule gives the new scale code
// s' = L_max/8 - 15 (+1 when the mantissa of the maximum is 7, i.e. above 1.75 = 448/256; only E4M3 has a top
// mantissa that its largest normal lacks), and an element's new code is sign | (L - 8 s') whenever that is a
// normal code; smaller ones are rounded to nearest-even into the subnormal grid.  A subnormal input is first
// normalised to the same (1 + m/8) * 2^x form, which gives it a (possibly negative) pseudo-magnitude.
// Identical to decoding to fp32 and re-quantizing (which the generic path does).
// Two elements ride in one register as 16-bit lanes (L < 4096), maxima by max.u16x2.
template <int FMT> struct RebaseT {
  static constexpr int MB = FmtT<FMT>::mbits;                                        // mantissa bits
  static constexpr uint32_t MAG = (1u << (FmtT<FMT>::ebits + FmtT<FMT>::mbits)) - 1u;   // magnitude bits of a code
  static constexpr uint32_t SIGN = MAG + 1u;
  static constexpr int ONE = 1 << MB;                                                // smallest normal magnitude
  static constexpr int OFF = FmtT<FMT>::bias + FmtT<FMT>::emax;                      // s' = L_max / ONE - OFF
  static constexpr bool PLUS1 = (FmtT<FMT>::max_mant != ONE - 1);                    // the block rule's "+1" can fire
  static constexpr uint32_t S_LO = OFF + MB + 1;                                     // scale codes the integer path takes
  static constexpr uint32_t MAG2 = MAG | (MAG << 16), SIGN4 = SIGN * 0x01010101u;
  static constexpr uint32_t EXP4 = (MAG & ~(uint32_t)(ONE - 1)) * 0x01010101u, LOW4 = (uint32_t)ONE * 0x01010101u;
};
RK_DEVINL uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// pseudo-magnitude of a subnormal code, mag in 1 .. ONE-1: value = mag * 2^x = (1 + m'/ONE) * 2^(x')
template <int FMT> RK_DEVINL int rb_subnormal_mag(int mag) {
  using R = RebaseT<FMT>;
  const int p = 31 - __clz(mag);                       // 0 .. MB-1
  return ((mag << (R::MB - p)) & (R::ONE - 1)) + R::ONE * (p - R::MB + 1);
}
// new code (without sign) of an element with L - ONE s' = tt
template <int FMT> RK_DEVINL uint32_t rb_code_from_tt(int tt) {
  using R = RebaseT<FMT>;
  if (tt >= R::ONE) return (uint32_t)tt;
  const int sh = 1 - (tt >> R::MB);                    // >= 1: below the smallest normal
  return sh > R::MB + 2 ? 0u : round_shift((uint32_t)R::ONE | (uint32_t)(tt & (R::ONE - 1)), sh);
}
// non-zero when some byte of w has a zero exponent field (zero or subnormal code)
template <int FMT> RK_DEVINL uint32_t rb_exp0_bits(uint32_t w) {
  using R = RebaseT<FMT>;
  const uint32_t e = w & R::EXP4;
  return (e - R::LOW4) & ~e & 0x80808080u;
}
RK_DEVINL uint32_t addmax_u16x2(uint32_t a, uint32_t b, uint32_t c) {   // max(a + b, c) in both 16-bit lanes
  uint32_t r;
  asm("{ .reg .b32 t; add.u16x2 t, %1, %2; max.u16x2 %0, t, %3; }" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

// Rare rows (a zero or subnormal code among the four): per-byte L, packed as lanes (0, 2) and (1, 3).
template <int FMT> __device__ __noinline__ uint2 rb_rare_l(uint32_t cw, int sj) {
  using R = RebaseT<FMT>;
  uint32_t l[4];
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int mag = (int)((cw >> (8 * q)) & R::MAG);
    l[q] = mag == 0 ? 0u : (uint32_t)((mag >= R::ONE ? mag : rb_subnormal_mag<FMT>(mag)) + R::ONE * sj) & 0xFFFFu;
  }
  return make_uint2(l[0] | (l[2] << 16), l[1] | (l[3] << 16));
}
// Rare rows of the second pass: some lane leaves the normal range, or an input was zero / subnormal.
// sub02 / sub13 carry ONE * s' of columns (0, 2) and (1, 3) as 16-bit lanes.
template <int FMT> __device__ __noinline__ uint32_t rb_rare_recode(uint32_t cw, int sj, uint32_t sub02, uint32_t sub13) {
  using R = RebaseT<FMT>;
  uint32_t out = cw & R::SIGN4;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int mag = (int)((cw >> (8 * q)) & R::MAG);
    const int sub = (int)((((q & 1) ? sub13 : sub02) >> (16 * (q >> 1))) & 0xFFFFu);
    if (mag != 0) out |= rb_code_from_tt<FMT>((mag >= R::ONE ? mag : rb_subnormal_mag<FMT>(mag)) + R::ONE * sj - sub) << (8 * q);
  }
  return out;
}

// scales along d, row-major [batch][S][d/32]  ->  atoms [batch][ntile][dch][512]
// (rows beyond S and blocks beyond d/32 get code 0x7F = 2^0); one thread per (atom, row) writes 4 bytes.
RK_DEVINL void retile_rowscales_body(const uint8_t* __restrict__ in, int64_t batch, int64_t S, int64_t d,
                                     uint8_t* __restrict__ out, int64_t tid, int64_t nthreads) {
  const int64_t nbd = d / 32, ntile = (S + 127) / 128, dch = (d + 127) / 128;
  const int64_t total = batch * ntile * dch * 128;
  for (int64_t t = tid; t < total; t += nthreads) {
    const int r = (int)(t % 128);
    const int64_t atom = t / 128;
    int64_t ch, tile, bt;
    if (total < (int64_t)1 << 31) {           // 32-bit divisions whenever the index fits
      const uint32_t a32 = (uint32_t)atom, q = a32 / (uint32_t)dch;
      ch = a32 - q * (uint32_t)dch;
      const uint32_t b32 = q / (uint32_t)ntile;
      tile = q - b32 * (uint32_t)ntile;
      bt = b32;
    } else {
      ch = atom % dch; tile = (atom / dch) % ntile; bt = atom / (dch * ntile);
    }
    const int64_t row = tile * 128 + r;
    uint32_t w = 0;
#pragma unroll
    for (int kb = 0; kb < 4; kb++) {
      const int64_t blk = ch * 4 + kb;
      const uint32_t sc = (row < S && blk < nbd) ? in[(bt * S + row) * nbd + blk] : 0x7Fu;
      w |= sc << (8 * kb);
    }
    *reinterpret_cast<uint32_t*>(out + atom * 512 + sf_atom_offset(r, 0)) = w;
  }
}
// Two row-major scale tensors (Q's and K's) that the re-blocking launch re-tiles on the side, so that the usual
// prefill call is two launches (this one and the attention kernel) instead of four; in == nullptr: nothing to do.
struct RetileJobs { const uint8_t* in[2]; uint8_t* out[2]; int64_t batch[2], S[2], d[2]; };

// Four lanes share one unit = 16 adjacent columns x one 32-key block: lane "rg" holds rows 8 rg .. 8 rg + 7 as
// eight 16-byte words in registers between the two passes (all loads of a thread in flight together), the
// column maxima meet by two shuffles.  A warp covers 8 adjacent units, so each 16-byte access of a warp touches
// four full 128-byte lines.  Blocks with scale codes outside [S_LO, 240] go through the generic fp32 path, each
// lane taking 4 of the unit's 16 columns over all 32 keys.
template <int FMT, bool TILED>
__global__ void __launch_bounds__(128, 4) rebase_v_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                                          int64_t batch, int64_t S, int64_t d,
                                                          uint8_t* __restrict__ out_codes, uint8_t* __restrict__ out_scales,
                                                          const RetileJobs jobs) {
#pragma unroll
  for (int jb = 0; jb < 2; ++jb)
    if (jobs.in[jb])
      retile_rowscales_body(jobs.in[jb], jobs.batch[jb], jobs.S[jb], jobs.d[jb], jobs.out[jb],
                            (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x);
  const int64_t c16n = d / 16, nkb = (S + 31) / 32, nbd = d / 32;
  const int64_t units = batch * nkb * c16n;
  const int64_t ntile = (S + 127) / 128, dch = (d + 127) / 128;   // atom grid of the TILED layout
  const int64_t warps_total = (units + 7) / 8;
  const int lane = threadIdx.x & 31, rg = lane >> 3;
  for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < warps_total;
       w += ((int64_t)gridDim.x * blockDim.x) >> 5) {
    const int64_t u = w * 8 + (lane & 7);
    const bool valid = u < units;
    const int64_t uu = valid ? u : 0;
    // unit index -> (batch, key block, column group): in 32 bits whenever it fits (a 64-bit division by a run-time
    // value is about a hundred instructions, and there are three of them per unit)
    int64_t c16, kb, bt;
    if (units < (int64_t)1 << 31) {
      const uint32_t u32 = (uint32_t)uu, q = u32 / (uint32_t)c16n;
      c16 = u32 - q * (uint32_t)c16n;
      const uint32_t b32 = q / (uint32_t)nkb;
      kb = q - b32 * (uint32_t)nkb;
      bt = b32;
    } else {
      c16 = uu % c16n; kb = (uu / c16n) % nkb; bt = uu / (c16n * nkb);
    }
    const int64_t r0 = kb * 32;
    const int n = valid ? (int)min((int64_t)32, S - r0) : 0;      // keys of this block that exist
    const uint8_t* cb = codes + (bt * S + r0) * d + c16 * 16;
    const uint8_t* sb = scales + (bt * S + r0) * nbd + c16 / 2;
    uint8_t* ob = out_codes + (bt * S + r0) * d + c16 * 16;
    uint32_t sc[4];                                               // new scale codes of columns 4 rg .. 4 rg + 3
    using R = RebaseT<FMT>;
    uint32_t bad = 0u;
    {
      // rows past a ragged end read as zero codes under a mid-range scale: they change nothing
      uint4 cw[8];
      uint32_t s8[8];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int j = rg * 8 + i;
        const bool in = j < n;
        cw[i] = in ? __ldg(reinterpret_cast<const uint4*>(cb + (int64_t)j * d)) : make_uint4(0u, 0u, 0u, 0u);
        s8[i] = in ? (uint32_t)__ldg(sb + (int64_t)j * nbd) : 127u;
      }
      // pass 1: largest L per column; word x of a row holds columns 4x .. 4x+3, lanes (0, 2) in lo[x], (1, 3) in hi[x]
      uint32_t lo[4] = {0u, 0u, 0u, 0u}, hi[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        bad |= (s8[i] - R::S_LO > 240u - R::S_LO) ? 1u : 0u;
        s8[i] *= (uint32_t)R::ONE * 0x00010001u;
        const uint32_t wv[4] = {cw[i].x, cw[i].y, cw[i].z, cw[i].w};
        // one test per row: does any of its 16 codes have a zero exponent field (zero or subnormal)?
        if ((rb_exp0_bits<FMT>(wv[0]) | rb_exp0_bits<FMT>(wv[1]) | rb_exp0_bits<FMT>(wv[2]) | rb_exp0_bits<FMT>(wv[3])) == 0u) {
#pragma unroll
          for (int x = 0; x < 4; x++) {
            lo[x] = addmax_u16x2(wv[x] & R::MAG2, s8[i], lo[x]);
            hi[x] = addmax_u16x2((wv[x] >> 8) & R::MAG2, s8[i], hi[x]);
          }
        } else {
#pragma unroll
          for (int x = 0; x < 4; x++) {
            uint2 l = make_uint2((wv[x] & R::MAG2) + s8[i], ((wv[x] >> 8) & R::MAG2) + s8[i]);
            if (rb_exp0_bits<FMT>(wv[x]) != 0u) l = rb_rare_l<FMT>(wv[x], (int)((s8[i] & 0xFFFFu) >> R::MB));
            lo[x] = max_u16x2(lo[x], l.x);
            hi[x] = max_u16x2(hi[x], l.y);
          }
        }
      }
#pragma unroll
      for (int x = 0; x < 4; x++) {
        lo[x] = max_u16x2(lo[x], __shfl_xor_sync(0xFFFFFFFFu, lo[x], 8));
        hi[x] = max_u16x2(hi[x], __shfl_xor_sync(0xFFFFFFFFu, hi[x], 8));
        lo[x] = max_u16x2(lo[x], __shfl_xor_sync(0xFFFFFFFFu, lo[x], 16));
        hi[x] = max_u16x2(hi[x], __shfl_xor_sync(0xFFFFFFFFu, hi[x], 16));
      }
      bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, 8);
      bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, 16);
      if (bad == 0u) {
        // s' = L_max / 8 - 15 (+1 when the mantissa bits are 7) in both 16-bit lanes at once; all-zero columns
        // (L_max = 0) get scale code 0
        uint32_t sub_lo[4], sub_hi[4];
#pragma unroll
        for (int x = 0; x < 4; x++) {
          uint32_t v[2] = {lo[x], hi[x]};
#pragma unroll
          for (int h = 0; h < 2; h++) {
            constexpr uint32_t M2 = (uint32_t)(R::ONE - 1) * 0x00010001u, Q2 = (0xFFFFu >> R::MB) * 0x00010001u;
            uint32_t sn = (v[h] >> R::MB) & Q2;
            if (R::PLUS1) sn += (((v[h] & M2) + 0x00010001u) >> R::MB) & 0x00010001u;
            if ((v[h] & 0xFFFFu) == 0u) sn = (sn & 0xFFFF0000u) | (uint32_t)R::OFF;          // an all-zero column: scale code 0
            if ((v[h] >> 16) == 0u) sn = (sn & 0x0000FFFFu) | ((uint32_t)R::OFF << 16);
            v[h] = sn - (uint32_t)R::OFF * 0x00010001u;
          }
          sub_lo[x] = v[0] << R::MB;
          sub_hi[x] = v[1] << R::MB;
          if (x == rg) {
            sc[0] = v[0] & 0xFFFFu; sc[1] = v[1] & 0xFFFFu; sc[2] = v[0] >> 16; sc[3] = v[1] >> 16;
          }
        }
        // pass 2: lanes carry tt + 0x4000 (tt = L - 8 s') so that they stay non-negative
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint32_t wv[4] = {cw[i].x, cw[i].y, cw[i].z, cw[i].w};
          uint32_t ov[4];
          // lanes that leave the normal range (tt < 8) set bit 15 of their half; zero / subnormal inputs set bit 7
          uint32_t rare[4];
#pragma unroll
          for (int x = 0; x < 4; x++) {
            const uint32_t t_lo = (wv[x] & R::MAG2) + s8[i] + (0x40004000u - sub_lo[x]);
            const uint32_t t_hi = ((wv[x] >> 8) & R::MAG2) + s8[i] + (0x40004000u - sub_hi[x]);
            ov[x] = (wv[x] & R::SIGN4) | (t_lo & R::MAG2) | ((t_hi & R::MAG2) << 8);
            rare[x] = (((t_lo - (0x40004000u + (uint32_t)R::ONE * 0x00010001u)) | (t_hi - (0x40004000u + (uint32_t)R::ONE * 0x00010001u))) & 0x80008000u) | rb_exp0_bits<FMT>(wv[x]);
          }
          if ((rare[0] | rare[1] | rare[2] | rare[3]) != 0u) {      // one branch per row in the common case
#pragma unroll
            for (int x = 0; x < 4; x++)
              if (rare[x] != 0u) ov[x] = rb_rare_recode<FMT>(wv[x], (int)((s8[i] & 0xFFFFu) >> R::MB), sub_lo[x], sub_hi[x]);
          }
          const int j = rg * 8 + i;
          if (j < n) *reinterpret_cast<uint4*>(ob + (int64_t)j * d) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
        }
      }
    }
    if (!valid) continue;
    if (bad != 0u) rebase_block_generic<FMT>(cb + rg * 4, sb, n, d, nbd, ob + rg * 4, sc);
    const int64_t col0 = c16 * 16 + rg * 4;
    if (TILED) {
      const int64_t kt = kb / 4;
      const int kbi = (int)(kb % 4);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int64_t col = col0 + q;
        const int64_t atom = (bt * ntile + kt) * dch + col / 128;
        out_scales[atom * 512 + sf_atom_offset((int)(col % 128), kbi)] = (uint8_t)sc[q];
      }
    } else {
      *reinterpret_cast<uint32_t*>(out_scales + (bt * nkb + kb) * d + col0) = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24);
    }
  }
}

// scales along keys, row-major [batch][ceil(S/32)][d]  ->  atoms [batch][ntile][dch][512]
__global__ void retile_keyscales_kernel(const uint8_t* __restrict__ in, int64_t batch, int64_t S, int64_t d,
                                        uint8_t* __restrict__ out) {
  const int64_t nkb = (S + 31) / 32, ntile = (S + 127) / 128, dch = (d + 127) / 128;
  const int64_t total = batch * ntile * dch * 128;   // one thread per (atom, column n): writes 4 bytes
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int n = (int)(t % 128);
    const int64_t atom = t / 128, nc = atom % dch, kt = (atom / dch) % ntile, bt = atom / (dch * ntile);
    const int64_t col = nc * 128 + n;
    uint32_t w = 0;
#pragma unroll
    for (int kbi = 0; kbi < 4; kbi++) {
      const int64_t kb = kt * 4 + kbi;
      const uint32_t s = (kb < nkb && col < d) ? in[(bt * nkb + kb) * d + col] : 0x7Fu;
      w |= s << (8 * kbi);
    }
    *reinterpret_cast<uint32_t*>(out + atom * 512 + sf_atom_offset(n, 0)) = w;
  }
}

__global__ void retile_rowscales_kernel(const uint8_t* __restrict__ in, int64_t batch, int64_t S, int64_t d,
                                        uint8_t* __restrict__ out) {
  retile_rowscales_body(in, batch, S, d, out, (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x);
}

// scales along d, group-major [batch][d/32][S] (the reference's QK_A_scales_row[FA_GK][FA_SQ] per head,
// kernels/flash_attention_mx/gen_data.py:82-83)  ->  atoms [batch][ntile][dch][512]
__global__ void retile_groupscales_kernel(const uint8_t* __restrict__ in, int64_t batch, int64_t S, int64_t d,
                                          uint8_t* __restrict__ out) {
  const int64_t nbd = d / 32, ntile = (S + 127) / 128, dch = (d + 127) / 128;
  const int64_t total = batch * ntile * dch * 128;   // one thread per (atom, row): writes 4 bytes; a warp reads 32 adjacent rows
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(t % 128);
    const int64_t atom = t / 128, ch = atom % dch, tile = (atom / dch) % ntile, bt = atom / (dch * ntile);
    const int64_t row = tile * 128 + r;
    uint32_t w = 0;
#pragma unroll
    for (int kb = 0; kb < 4; kb++) {
      const int64_t blk = ch * 4 + kb;
      const uint32_t sc = (row < S && blk < nbd) ? in[(bt * nbd + blk) * S + row] : 0x7Fu;
      w |= sc << (8 * kb);
    }
    *reinterpret_cast<uint32_t*>(out + atom * 512 + sf_atom_offset(r, 0)) = w;
  }
}

// The reference's streaming K operand (kernels/flash_attention_mx_gqa/fa_gen_data.py:110-117): per KV head and key
// block j a transposed tile K^T [d][Bk] (QK_B_blocks) with group-major scales [d/32][Bk] (QK_B_scales_blocks)
// -> natural K codes [heads][nblk*Bk][d] and row-major scales [heads][nblk*Bk][d/32].
// One CTA transposes a 32 x 32 byte tile through shared memory; scales by one thread per output byte.
__global__ void __launch_bounds__(256) import_kt_blocks_kernel(const uint8_t* __restrict__ kt, const uint8_t* __restrict__ kts,
                                                               int64_t heads, int nblk, int Bk, int d,
                                                               uint8_t* __restrict__ k, uint8_t* __restrict__ ks) {
  __shared__ uint8_t tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;           // 32 x 8
  const int64_t tiles_k = Bk / 32, tiles_d = d / 32;
  const int64_t ntiles = heads * nblk * tiles_d * tiles_k;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t tk = t % tiles_k, td = (t / tiles_k) % tiles_d, blk = t / (tiles_k * tiles_d);   // blk = head * nblk + j
    const uint8_t* src = kt + (blk * d + td * 32) * Bk + tk * 32;    // rows = d index, cols = key inside the block
#pragma unroll
    for (int i = 0; i < 4; ++i) tile[ty + 8 * i][tx] = src[(int64_t)(ty + 8 * i) * Bk + tx];
    __syncthreads();
    uint8_t* dst = k + (blk * Bk + tk * 32) * d + td * 32;            // rows = key, cols = d index
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[(int64_t)(ty + 8 * i) * d + tx] = tile[tx][ty + 8 * i];
    __syncthreads();
  }
  const int nbd = d / 32;
  const int64_t nsc = heads * nblk * (int64_t)Bk * nbd;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < nsc; t += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(t % nbd);
    const int64_t key = (t / nbd) % Bk, blk = t / ((int64_t)nbd * Bk);
    ks[t] = kts[(blk * nbd + g) * Bk + key];
  }
}

// 16 codes of BITS bits each -> BITS/2 32-bit words, code i in bits [BITS*i, BITS*i + BITS) (the order TMA's
// 16U6_ALIGN16B / 16U4_ALIGN16B types expand from)
template <int BITS> RK_DEVINL void pack16(const uint32_t* c, uint32_t* w) {
  if (BITS == 4) {
    uint32_t a = 0, b = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { a |= (c[i] & 0xFu) << (4 * i); b |= (c[8 + i] & 0xFu) << (4 * i); }
    w[0] = a; w[1] = b;
    return;
  }
  uint64_t lo = 0, hi = 0;     // 96 bits
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint64_t v = c[i] & 0x3Fu;
    const int bit = 6 * i;
    if (bit < 64) { lo |= v << bit; if (bit + 6 > 64) hi |= v >> (64 - bit); }
    else hi |= v << (bit - 64);
  }
  w[0] = (uint32_t)lo; w[1] = (uint32_t)(lo >> 32); w[2] = (uint32_t)hi;
}

// byte codes [rows][d] -> packed [rows][dp * BITS/8 bytes], dp = d rounded up to 128, padding codes 0
template <int BITS>
__global__ void pack_rows_kernel(const uint8_t* __restrict__ in, int64_t rows, int64_t d, int64_t dp, uint8_t* __restrict__ out) {
  const int64_t groups = dp / 16, total = rows * groups;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / groups, gidx = t % groups;
    uint32_t c[16], w[3];
    if (gidx * 16 < d) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + r * d + gidx * 16);
      const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 16; ++i) c[i] = (ww[i >> 2] >> (8 * (i & 3))) & 0xFFu;
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) c[i] = 0;
    }
    pack16<BITS>(c, w);
    uint32_t* o = reinterpret_cast<uint32_t*>(out + r * (dp * BITS / 8) + gidx * (2 * BITS));
    o[0] = w[0]; o[1] = w[1];
    if (BITS == 6) o[2] = w[2];
  }
}

// byte codes [batch][S][d] -> packed transposed [batch][d][Sp * BITS/8 bytes], Sp = S rounded up to 128.
// One CTA = one tile of 128 keys x 128 columns through shared memory: coalesced 16-byte reads along d, then each
// thread packs 16 keys of one column and the 8 threads of a column write 96 (64) contiguous bytes.
template <int BITS>
__global__ void __launch_bounds__(256) pack_transpose_kernel(const uint8_t* __restrict__ in, int64_t batch, int64_t S, int64_t d,
                                                              int64_t Sp, uint8_t* __restrict__ out) {
  __shared__ uint8_t tile[128][128 + 4];                       // [key][col], rows padded by one word against bank conflicts
  const int64_t ktiles = Sp / 128, ctiles = (d + 127) / 128;
  const int64_t ntiles = batch * ktiles * ctiles;
  for (int64_t tix = blockIdx.x; tix < ntiles; tix += gridDim.x) {
    const int64_t ct = tix % ctiles, kt = (tix / ctiles) % ktiles, bt = tix / (ctiles * ktiles);
    const int64_t key0 = kt * 128, col0 = ct * 128;
    __syncthreads();                                           // the previous tile has been read out
    for (int i = threadIdx.x; i < 128 * 8; i += 256) {         // 128 rows x 8 chunks of 16 columns
      const int r = i >> 3, ch = i & 7;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (key0 + r < S && col0 + ch * 16 < d) v = *reinterpret_cast<const uint4*>(in + (bt * S + key0 + r) * d + col0 + ch * 16);
      uint32_t* dst = reinterpret_cast<uint32_t*>(&tile[r][ch * 16]);
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 128 * 8; i += 256) {         // 128 columns x 8 groups of 16 keys
      const int col = i >> 3, gi = i & 7;
      if (col0 + col >= d) continue;
      uint32_t c[16], w[3];
#pragma unroll
      for (int k = 0; k < 16; ++k) c[k] = tile[gi * 16 + k][col];
      pack16<BITS>(c, w);
      uint32_t* o = reinterpret_cast<uint32_t*>(out + (bt * d + col0 + col) * (Sp * BITS / 8) + (kt * 8 + gi) * (2 * BITS));
      o[0] = w[0]; o[1] = w[1];
      if (BITS == 6) o[2] = w[2];
    }
  }
}

static int grid_for(int64_t work_items, int threads, int per_sm) {
  const int64_t want = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)num_sms() * per_sm;
  return (int)max((int64_t)1, min(want, cap));
}

#define RK_DISPATCH_FMT(fmt, ...)                  \
  switch (fmt) {                                   \
    case 0: { constexpr int F = 0; __VA_ARGS__; } break; \
    case 1: { constexpr int F = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int F = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int F = 3; __VA_ARGS__; } break; \
    case 4: { constexpr int F = 4; __VA_ARGS__; } break; \
    default: return RK_ERR_BAD_FORMAT;             \
  }

int launch_quantize_rows_bf16(const void* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales,
                              cudaStream_t st) {
  const int64_t nchunks = rows * cols / 8;
  if (nchunks == 0) return RK_OK;
  const int grid = grid_for(nchunks, 256, 8);
  RK_DISPATCH_FMT(fmt, (quantize_rows_kernel<F, true><<<grid, 256, 0, st>>>(reinterpret_cast<const float4*>(x), nchunks,
                                                                            reinterpret_cast<uint2*>(codes), scales)));
  return (int)cudaGetLastError();
}

// Blocks along d with a chosen scale layout (see quantize_rows_kernel); x is fp32 or bf16 [batch][S][d].
int launch_quantize_rows_ex(const void* x, bool bf16, int64_t batch, int64_t S, int64_t d, int fmt, uint8_t* codes,
                            uint8_t* scales, int layout, cudaStream_t st) {
  const int64_t nchunks = batch * S * d / 8;
  if (nchunks == 0) return RK_OK;
  const int grid = grid_for(nchunks, 256, 8);
  const float4* xp = reinterpret_cast<const float4*>(x);
  uint2* cp = reinterpret_cast<uint2*>(codes);
  const int nbd = (int)(d / 32);
#define RK_QX(BF, LAY) RK_DISPATCH_FMT(fmt, (quantize_rows_kernel<F, BF, LAY><<<grid, 256, 0, st>>>(xp, nchunks, cp, scales, S, nbd)))
  if (layout == RK_SCALES_ROWMAJOR) { if (bf16) { RK_QX(true, 0); } else { RK_QX(false, 0); } }
  else if (layout == RK_SCALES_GROUPMAJOR) { if (bf16) { RK_QX(true, 1); } else { RK_QX(false, 1); } }
  else if (layout == RK_SCALES_SF_ATOMS) { if (bf16) { RK_QX(true, 2); } else { RK_QX(false, 2); } }
  else return RK_ERR_BAD_FORMAT;
#undef RK_QX
  return (int)cudaGetLastError();
}

int launch_quantize_keys_atoms(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt, uint8_t* codes,
                               uint8_t* scales, cudaStream_t st) {
  const int64_t total = batch * ((rows + 31) / 32) * (cols / 4);
  if (total == 0) return RK_OK;
  const int grid = grid_for(total, 128, 16);
  RK_DISPATCH_FMT(fmt, (quantize_keys_kernel<F, true><<<grid, 128, 0, st>>>(x, batch, rows, cols, codes, scales)));
  return (int)cudaGetLastError();
}

int launch_retile_groupscales(const uint8_t* in, int64_t batch, int64_t S, int64_t d, uint8_t* out, cudaStream_t st) {
  const int64_t total = batch * ((S + 127) / 128) * ((d + 127) / 128) * 128;
  if (total == 0) return RK_OK;
  retile_groupscales_kernel<<<grid_for(total, 256, 8), 256, 0, st>>>(in, batch, S, d, out);
  return (int)cudaGetLastError();
}

int launch_import_kt_blocks(const uint8_t* kt, const uint8_t* kts, int64_t heads, int nblk, int Bk, int d, uint8_t* k,
                            uint8_t* ks, cudaStream_t st) {
  const int64_t ntiles = heads * nblk * (d / 32) * (Bk / 32);
  if (ntiles == 0) return RK_OK;
  import_kt_blocks_kernel<<<(int)min(ntiles, (int64_t)num_sms() * 16), 256, 0, st>>>(kt, kts, heads, nblk, Bk, d, k, ks);
  return (int)cudaGetLastError();
}

int launch_rmsnorm_quantize(const void* x, bool bf16, int64_t rows, int K, const float* gamma, float eps, int fmt,
                            bool unit_scale, uint8_t* codes, uint8_t* scales, cudaStream_t st) {
  if (rows == 0 || K == 0) return RK_OK;
  const int64_t groups = (rows + 31) / 32;
  const int grid = (int)std::min<int64_t>((groups + 7) / 8, (int64_t)num_sms() * 8);
#define RK_RN(BF, UN) RK_DISPATCH_FMT(fmt, (rmsnorm_quantize_kernel<F, BF, UN><<<grid, 256, 0, st>>>(x, rows, K, gamma, eps, codes, scales)))
  if (bf16) { if (unit_scale) { RK_RN(true, true); } else { RK_RN(true, false); } }
  else      { if (unit_scale) { RK_RN(false, true); } else { RK_RN(false, false); } }
#undef RK_RN
  return (int)cudaGetLastError();
}

int launch_quantize_rows(const float* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales,
                         cudaStream_t st) {
  const int64_t nchunks = rows * cols / 8;
  if (nchunks == 0) return RK_OK;
  const int grid = grid_for(nchunks, 256, 8);
  RK_DISPATCH_FMT(fmt, (quantize_rows_kernel<F><<<grid, 256, 0, st>>>(reinterpret_cast<const float4*>(x), nchunks,
                                                                      reinterpret_cast<uint2*>(codes), scales)));
  return (int)cudaGetLastError();
}

int launch_quantize_keys(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt, uint8_t* codes,
                         uint8_t* scales, cudaStream_t st) {
  const int64_t total = batch * ((rows + 31) / 32) * (cols / 4);
  if (total == 0) return RK_OK;
  const int grid = grid_for(total, 128, 16);
  RK_DISPATCH_FMT(fmt, (quantize_keys_kernel<F><<<grid, 128, 0, st>>>(x, batch, rows, cols, codes, scales)));
  return (int)cudaGetLastError();
}

int launch_rope_quantize_rows(const float* x, int64_t rows, int d, const int32_t* pos, int seq_len, int pos0, const float* cos_h,
                              const float* sin_h, int fmt, uint8_t* codes, uint8_t* scales, cudaStream_t st) {
  const int64_t nchunks = rows * (d / 16);
  if (nchunks == 0) return RK_OK;
  const int grid = grid_for(nchunks, 256, 8);
  RK_DISPATCH_FMT(fmt, (rope_quantize_rows_kernel<F><<<grid, 256, 0, st>>>(x, rows, d, pos, seq_len, pos0, cos_h, sin_h, codes, scales)));
  return (int)cudaGetLastError();
}

int launch_kv_append(const float* k_new, const float* v_new, int B, int H_kv, int L, int d, const int32_t* pos, int fmt,
                     uint8_t* k_codes, uint8_t* k_scales, uint8_t* v_codes, uint8_t* v_scales, cudaStream_t st) {
  const int64_t total = 2LL * B * H_kv * (d / 8);
  if (total == 0) return RK_OK;
  const int grid = grid_for(total, 128, 8);
  RK_DISPATCH_FMT(fmt, (kv_append_kernel<F><<<grid, 128, 0, st>>>(k_new, v_new, B, H_kv, L, d, pos, k_codes, k_scales, v_codes, v_scales)));
  return (int)cudaGetLastError();
}

// q_scales / k_scales (optional, both or neither): row-major E8M0 scales of Q [bhq][S_q][d/32] and K [batch][S][d/32]
// re-tiled into atoms by the same launch.
int launch_rebase_v(const uint8_t* codes, const uint8_t* scales, int64_t batch, int64_t S, int64_t d, int fmt,
                    uint8_t* out_codes, uint8_t* out_scales, bool tiled, cudaStream_t st, const uint8_t* q_scales,
                    int64_t bhq, int64_t S_q, uint8_t* q_atoms, const uint8_t* k_scales, uint8_t* k_atoms) {
  const int64_t total = ((batch * ((S + 31) / 32) * (d / 16) + 7) / 8) * 32;     // 4 lanes per 16-column unit, whole warps
  if (total == 0) return RK_OK;
  const int grid = grid_for(total, 128, 16);      // four CTAs are resident per SM; four waves of them end more evenly than two (-6 %)
  RetileJobs jobs = {};
  if (q_scales && k_scales) {
    jobs.in[0] = q_scales; jobs.out[0] = q_atoms; jobs.batch[0] = bhq; jobs.S[0] = S_q; jobs.d[0] = d;
    jobs.in[1] = k_scales; jobs.out[1] = k_atoms; jobs.batch[1] = batch; jobs.S[1] = S; jobs.d[1] = d;
  }
  if (tiled) { RK_DISPATCH_FMT(fmt, (rebase_v_kernel<F, true><<<grid, 128, 0, st>>>(codes, scales, batch, S, d, out_codes, out_scales, jobs))); }
  else       { RK_DISPATCH_FMT(fmt, (rebase_v_kernel<F, false><<<grid, 128, 0, st>>>(codes, scales, batch, S, d, out_codes, out_scales, jobs))); }
  return (int)cudaGetLastError();
}

int launch_retile_rowscales(const uint8_t* in, int64_t batch, int64_t S, int64_t d, uint8_t* out, cudaStream_t st) {
  const int64_t total = batch * ((S + 127) / 128) * ((d + 127) / 128) * 128;
  if (total == 0) return RK_OK;
  retile_rowscales_kernel<<<grid_for(total, 256, 8), 256, 0, st>>>(in, batch, S, d, out);
  return (int)cudaGetLastError();
}

int launch_retile_keyscales(const uint8_t* in, int64_t batch, int64_t S, int64_t d, uint8_t* out, cudaStream_t st) {
  const int64_t total = batch * ((S + 127) / 128) * ((d + 127) / 128) * 128;
  if (total == 0) return RK_OK;
  retile_keyscales_kernel<<<grid_for(total, 256, 8), 256, 0, st>>>(in, batch, S, d, out);
  return (int)cudaGetLastError();
}

// bits = 6 (E2M3, E3M2) or 4 (E2M1)
int launch_pack_rows(const uint8_t* in, int64_t rows, int64_t d, int bits, uint8_t* out, cudaStream_t st) {
  const int64_t dp = (d + 127) / 128 * 128, total = rows * (dp / 16);
  if (total == 0) return RK_OK;
  if (bits == 4) pack_rows_kernel<4><<<grid_for(total, 256, 8), 256, 0, st>>>(in, rows, d, dp, out);
  else pack_rows_kernel<6><<<grid_for(total, 256, 8), 256, 0, st>>>(in, rows, d, dp, out);
  return (int)cudaGetLastError();
}

int launch_pack_transpose(const uint8_t* in, int64_t batch, int64_t S, int64_t d, int bits, uint8_t* out, cudaStream_t st) {
  const int64_t Sp = (S + 127) / 128 * 128, tiles = batch * (Sp / 128) * ((d + 127) / 128);
  if (tiles == 0) return RK_OK;
  const int grid = (int)min(tiles, (int64_t)num_sms() * 8);
  if (bits == 4) pack_transpose_kernel<4><<<grid, 256, 0, st>>>(in, batch, S, d, Sp, out);
  else pack_transpose_kernel<6><<<grid, 256, 0, st>>>(in, batch, S, d, Sp, out);
  return (int)cudaGetLastError();
}

// Runs the exhaustive encoder check for one format over all 2^32 fp32 bit patterns.
int launch_verify_encoder(int fmt, unsigned long long* mismatches, uint32_t* first_bad, cudaStream_t st) {
  const int grid = num_sms() * 8;
  RK_DISPATCH_FMT(fmt, (verify_encoder_kernel<F><<<grid, 256, 0, st>>>(0ull, 1ull << 32, mismatches, first_bad)));
  return (int)cudaGetLastError();
}

}  // namespace rk
