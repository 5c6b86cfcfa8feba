// MX block quantizer kernels (HBM-bound streaming kernels, no tensor cores).
//
//  quantize_rows   fp32 [rows][cols] -> codes + one E8M0 scale per 32 contiguous
//                  elements.  Bit-exact restatement of quantize_one_block,
//                  kernels/simt_quant/kernel.cpp:95-129 (golden:
//                  lib/golden/golden.py:118-170), vectorised: 4 lanes share a
//                  block, each lane loads 2 x float4 and stores 8 packed codes.
//                  Algorithmic traffic 4 B in + 1 B + 1/32 B out per element.
//  quantize_keys   same rule with the blocks running down the rows (the key
//                  axis) of each matrix in a batch -- the reference's V layout
//                  (kernels/flash_attention_mx/gen_data.py:77).
//  rebase_v        codes+scales blocked along d -> decode exactly -> re-block
//                  along the keys.  Writes the scales either row-major
//                  [ceil(S/32)][d] or directly in the 512-byte scale-factor
//                  atoms the attention kernel copies into TMEM.
//  retile_scales   row-major [rows][d/32] scales -> scale-factor atoms.
#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

template <int FMT>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float4* __restrict__ x, int64_t nchunks,
                                                            uint2* __restrict__ codes, uint8_t* __restrict__ scales) {
  // chunk = 8 consecutive elements; 4 consecutive lanes = one 32-element block
  // Warp-uniform loop bound: all 32 lanes run the shuffles even when the last
  // chunks of the array end inside this warp (nchunks is a multiple of 4, so a
  // 4-lane group is either wholly live or wholly idle).
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c - lane < nchunks; c += stride) {
    const bool live = c < nchunks;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (live) { a = __ldcs(x + 2 * c); b = __ldcs(x + 2 * c + 1); }
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float av = fabsf(v[j]);
      if (av > amax) amax = av;    // NaN never wins, as in the reference loop
    }
    float o = __shfl_xor_sync(0xffffffffu, amax, 1); if (o > amax) amax = o;
    o = __shfl_xor_sync(0xffffffffu, amax, 2); if (o > amax) amax = o;
    if (!live) continue;
    uint32_t scode = 0; float p2 = 1.0f;
    if (amax > 0.0f) block_scale<FMT>(amax, scode, p2);
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      w0 |= encode_rne<FMT>(v[j] * p2) << (8 * j);
      w1 |= encode_rne<FMT>(v[4 + j] * p2) << (8 * j);
    }
    __stcs(codes + c, make_uint2(w0, w1));
    if ((c & 3) == 0) scales[c >> 2] = (uint8_t)scode;
  }
}

// One thread = 4 adjacent columns x one 32-row block.
template <int FMT>
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
    for (int j = 0; j < n; j++) {
      const float4 v = *reinterpret_cast<const float4*>(xb + (int64_t)j * cols);
      const float av[4] = {fabsf(v.x), fabsf(v.y), fabsf(v.z), fabsf(v.w)};
#pragma unroll
      for (int q = 0; q < 4; q++) if (av[q] > amax[q]) amax[q] = av[q];
    }
    uint32_t sc[4]; float p2[4];
#pragma unroll
    for (int q = 0; q < 4; q++) { sc[q] = 0; p2[q] = 1.0f; if (amax[q] > 0.0f) block_scale<FMT>(amax[q], sc[q], p2[q]); }
    uint8_t* cb = codes + (bt * rows + r0) * cols + c4 * 4;
    for (int j = 0; j < n; j++) {
      const float4 v = *reinterpret_cast<const float4*>(xb + (int64_t)j * cols);
      const uint32_t w = encode_rne<FMT>(v.x * p2[0]) | (encode_rne<FMT>(v.y * p2[1]) << 8) |
                         (encode_rne<FMT>(v.z * p2[2]) << 16) | (encode_rne<FMT>(v.w * p2[3]) << 24);
      *reinterpret_cast<uint32_t*>(cb + (int64_t)j * cols) = w;
    }
    *reinterpret_cast<uint32_t*>(scales + (bt * nkb + kb) * cols + c4 * 4) = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24);
  }
}

// Offset of (row r of a 128-row tile, 32-element block kb of a 128-element
// chunk) inside a 512-byte scale-factor atom: 32 rows x 16 bytes, row r%32,
// byte (r/32)*4 + kb.  One tcgen05.cp 32x128b.warpx4 moves an atom to 4 TMEM
// columns (lane = r%32, column = r/32, byte = kb).
__host__ __device__ inline int sf_atom_offset(int r, int kb) { return (r & 31) * 16 + (r >> 5) * 4 + kb; }

template <int FMT, bool TILED>
__global__ void __launch_bounds__(128) rebase_v_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                                       int64_t batch, int64_t S, int64_t d,
                                                       uint8_t* __restrict__ out_codes, uint8_t* __restrict__ out_scales) {
  const int64_t c4n = d / 4, nkb = (S + 31) / 32, nbd = d / 32;
  const int64_t total = batch * nkb * c4n;
  const int64_t ntile = (S + 127) / 128, dch = (d + 127) / 128;   // atom grid of the TILED layout
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c4 = t % c4n, kb = (t / c4n) % nkb, bt = t / (c4n * nkb);
    const int64_t r0 = kb * 32;
    const int n = (int)min((int64_t)32, S - r0);
    const uint8_t* cb = codes + (bt * S + r0) * d + c4 * 4;
    const uint8_t* sb = scales + (bt * S + r0) * nbd + (c4 * 4) / 32;
    float val[32][4];
    float amax[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 32; j++) {
      if (j < n) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(cb + (int64_t)j * d);
        const float sf = e8m0_to_f32(sb[(int64_t)j * nbd]);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          val[j][q] = decode_elem<FMT>((w >> (8 * q)) & 0xFFu) * sf;
          const float av = fabsf(val[j][q]);
          if (av > amax[q]) amax[q] = av;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; q++) val[j][q] = 0.0f;
      }
    }
    uint32_t sc[4]; float p2[4];
#pragma unroll
    for (int q = 0; q < 4; q++) { sc[q] = 0; p2[q] = 1.0f; if (amax[q] > 0.0f) block_scale<FMT>(amax[q], sc[q], p2[q]); }
    uint8_t* ob = out_codes + (bt * S + r0) * d + c4 * 4;
#pragma unroll
    for (int j = 0; j < 32; j++) {
      if (j < n) {
        const uint32_t w = encode_rne<FMT>(val[j][0] * p2[0]) | (encode_rne<FMT>(val[j][1] * p2[1]) << 8) |
                           (encode_rne<FMT>(val[j][2] * p2[2]) << 16) | (encode_rne<FMT>(val[j][3] * p2[3]) << 24);
        *reinterpret_cast<uint32_t*>(ob + (int64_t)j * d) = w;
      }
    }
    if (TILED) {
      const int64_t kt = kb / 4;
      const int kbi = (int)(kb % 4);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int64_t col = c4 * 4 + q;
        const int64_t atom = (bt * ntile + kt) * dch + col / 128;
        out_scales[atom * 512 + sf_atom_offset((int)(col % 128), kbi)] = (uint8_t)sc[q];
      }
    } else {
      *reinterpret_cast<uint32_t*>(out_scales + (bt * nkb + kb) * d + c4 * 4) = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24);
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

// scales along d, row-major [batch][S][d/32]  ->  atoms [batch][ntile][dch][512]
// (rows beyond S and blocks beyond d/32 get code 0x7F = 2^0).
__global__ void retile_rowscales_kernel(const uint8_t* __restrict__ in, int64_t batch, int64_t S, int64_t d,
                                        uint8_t* __restrict__ out) {
  const int64_t nbd = d / 32, ntile = (S + 127) / 128, dch = (d + 127) / 128;
  const int64_t total = batch * ntile * dch * 128;   // one thread per (atom, row): writes 4 bytes
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(t % 128);
    const int64_t atom = t / 128, ch = atom % dch, tile = (atom / dch) % ntile, bt = atom / (dch * ntile);
    const int64_t row = tile * 128 + r;
    uint32_t w = 0;
#pragma unroll
    for (int kb = 0; kb < 4; kb++) {
      const int64_t blk = ch * 4 + kb;
      const uint32_t s = (row < S && blk < nbd) ? in[(bt * S + row) * nbd + blk] : 0x7Fu;
      w |= s << (8 * kb);
    }
    *reinterpret_cast<uint32_t*>(out + atom * 512 + sf_atom_offset(r, 0)) = w;
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
    default: return RK_ERR_BAD_FORMAT;             \
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

int launch_rebase_v(const uint8_t* codes, const uint8_t* scales, int64_t batch, int64_t S, int64_t d, int fmt,
                    uint8_t* out_codes, uint8_t* out_scales, bool tiled, cudaStream_t st) {
  const int64_t total = batch * ((S + 31) / 32) * (d / 4);
  if (total == 0) return RK_OK;
  const int grid = grid_for(total, 128, 8);
  if (tiled) { RK_DISPATCH_FMT(fmt, (rebase_v_kernel<F, true><<<grid, 128, 0, st>>>(codes, scales, batch, S, d, out_codes, out_scales))); }
  else       { RK_DISPATCH_FMT(fmt, (rebase_v_kernel<F, false><<<grid, 128, 0, st>>>(codes, scales, batch, S, d, out_codes, out_scales))); }
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

}  // namespace rk
