// Measurement aid: the throughput of the block-scaled tensor-core instruction the attention kernels are built
// from, with nothing else in the way.  One CTA per SM holds one A tile and one B tile ([128 rows][128 bytes],
// K-major, 128-byte swizzle: the shape of a Q tile and a K tile) in shared memory and issues
// tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale M=128 N=128 K=32 back to back: four per 128-deep product,
// `iters` products, alternating between two TMEM accumulators.  No softmax, no TMA in the loop, operands and
// scales resident: the number it gives is the ceiling the attention kernel's 128 x 128 x 32 MMAs could reach on
// this part at the clocks it ran at.  The reference has no counterpart (its mesh-busy figure,
// kernels/flash_attention_mx/README.md:28-29, plays the same role there).
#include <cuda.h>

#include "rk_common.cuh"
#include "rk_internal.h"

namespace rk {

namespace peak {
constexpr int kTile = 128 * 128;
constexpr int a_off = 0, b_off = kTile, sf_off = 2 * kTile, bar_off = sf_off + 1024, misc_off = bar_off + 32;
constexpr int total = misc_off + 32;
constexpr uint32_t kCols = 512;
}  // namespace peak

__global__ void __launch_bounds__(128, 1)
mxfp8_mma_loop_kernel(const uint8_t* __restrict__ a_tile, const uint8_t* __restrict__ b_tile, int iters, int* status,
                      uint32_t idesc) {
  using namespace peak;
  extern __shared__ __align__(1024) uint8_t peak_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(peak_smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + bar_off);       // [0] loads, [1] drain, [2], [3] pacing
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + misc_off + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (*reinterpret_cast<volatile int*>(status) != 0) return;

  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[2], 1); mbar_init(&bars[3], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // scale atoms: every block scale 2^0
  for (int i = threadIdx.x; i < 256; i += blockDim.x) reinterpret_cast<uint32_t*>(smem + sf_off)[i] = 0x7F7F7F7Fu;
  if (warp == 1) { tmem_alloc(tmem_ptr, kCols); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0 && lane == 0) {
    mbar_arrive_expect_tx(&bars[0], 2 * kTile);
    bulk_load_1d(smem + a_off, a_tile, kTile, &bars[0]);
    bulk_load_1d(smem + b_off, b_tile, kTile, &bars[0]);
    bool ok = mbar_wait(&bars[0], 0, abort_flag, status, 801);
    if (ok) {
      const uint32_t a_addr = smem_u32(smem + a_off), b_addr = smem_u32(smem + b_off);
      const uint32_t sfa = tmem_base + 256, sfb = tmem_base + 260;
      tc_cp_32x128b_warpx4(sfa, make_smem_desc(smem_u32(smem + sf_off), 0, 128, kLayoutNone));
      tc_cp_32x128b_warpx4(sfb, make_smem_desc(smem_u32(smem + sf_off + 512), 0, 128, kLayoutNone));
      uint32_t batch = 0;            // batches of 64 products committed so far
      for (int i = 0; i < iters && ok; ++i) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t adesc = make_smem_desc(a_addr + kk * 32, 16, 1024, kLayoutSw128);
          const uint64_t bdesc = make_smem_desc(b_addr + kk * 32, 16, 1024, kLayoutSw128);
          mma_mxf8f6f4_ss(tmem_base + (i & 1) * 128, adesc, bdesc, idesc_with_sf(idesc, kk, kk), sfa, sfb, kk > 0 ? 1u : 0u);
        }
        // Every 64 products: wait for the batch issued before this one, so the queue of outstanding work stays
        // bounded.  Batch k commits to pacing barrier k & 1 and is waited for before batch k + 2 commits to the
        // same barrier: a barrier never completes two phases unobserved.  (With both batches on one barrier a
        // parity wait saw the phase it asked for AND the next one completed once in ~10 000 launches, read that as
        // "not yet" and ran into its limit.)
        if ((i & 63) == 63) {
          tc_commit(&bars[2 + (batch & 1)]);
          if (batch >= 1) ok = mbar_wait(&bars[2 + ((batch - 1) & 1)], ((batch - 1) >> 1) & 1, abort_flag, status, 802);
          ++batch;
        }
      }
      tc_commit(&bars[1]);
      mbar_wait(&bars[1], 0, abort_flag, status, 803);
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kCols); }
}

// Launches the loop on every SM; FLOP of the launch = SMs * iters * 2 * 128 * 128 * 128.
int launch_mxfp8_mma_loop(const uint8_t* a_tile, const uint8_t* b_tile, int iters, cudaStream_t st) {
  int* status = device_status_word();
  if (!status) return RK_ERR_NO_DEVICE;
  const int smem_bytes = peak::total + 1024;
  cudaError_t e = cudaFuncSetAttribute(mxfp8_mma_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  const uint32_t idesc = make_idesc(RK_FMT_E4M3, RK_FMT_E4M3, false, false, 128, 128);
  mxfp8_mma_loop_kernel<<<num_sms(), 128, smem_bytes, st>>>(a_tile, b_tile, iters, status, idesc);
  return (int)cudaGetLastError();
}

}  // namespace rk
