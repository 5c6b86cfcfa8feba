// Declarations shared by the .cu files of the library (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rk_mx_attn.h"

namespace rk {

extern cudaEvent_t g_ev_before, g_ev_after;   // optional profiling events around the main kernels
int num_sms();                 // SM count of the current device (cached per device)
int* device_status_word();     // per-device int inside the library image, zero at load; kernels CAS error codes into it.
                               // NULL when the device could not be queried: callers return RK_ERR_NO_DEVICE

int launch_quantize_rows_bf16(const void* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales, cudaStream_t st);
int launch_quantize_rows(const float* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales, cudaStream_t st);
int launch_quantize_keys(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales, cudaStream_t st);
int launch_rebase_v(const uint8_t* codes, const uint8_t* scales, int64_t batch, int64_t S, int64_t d, int fmt,
                    uint8_t* out_codes, uint8_t* out_scales, bool tiled, cudaStream_t st, const uint8_t* q_scales = nullptr,
                    int64_t bhq = 0, int64_t S_q = 0, uint8_t* q_atoms = nullptr, const uint8_t* k_scales = nullptr,
                    uint8_t* k_atoms = nullptr);
int launch_retile_rowscales(const uint8_t* in, int64_t batch, int64_t S, int64_t d, uint8_t* out, cudaStream_t st);
int launch_pack_rows(const uint8_t* in, int64_t rows, int64_t d, int bits, uint8_t* out, cudaStream_t st);
int launch_pack_transpose(const uint8_t* in, int64_t batch, int64_t S, int64_t d, int bits, uint8_t* out, cudaStream_t st);
int launch_verify_encoder(int fmt, unsigned long long* mismatches, uint32_t* first_bad, cudaStream_t st);
int launch_quantize_rows_ex(const void* x, bool bf16, int64_t batch, int64_t S, int64_t d, int fmt, uint8_t* codes,
                            uint8_t* scales, int layout, cudaStream_t st);
int launch_quantize_keys_atoms(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt, uint8_t* codes,
                               uint8_t* scales, cudaStream_t st);
int launch_rmsnorm_quantize(const void* x, bool bf16, int64_t rows, int K, const float* gamma, float eps, int fmt,
                            bool unit_scale, uint8_t* codes, uint8_t* scales, cudaStream_t st);
int launch_mx_gemm_hw(const uint8_t* A, const uint8_t* B, const uint8_t* SA, const uint8_t* SB, int M, int N, int K,
                      uint16_t* C, cudaStream_t st);
int launch_retile_groupscales(const uint8_t* in, int64_t batch, int64_t S, int64_t d, uint8_t* out, cudaStream_t st);
int launch_import_kt_blocks(const uint8_t* kt, const uint8_t* kts, int64_t heads, int nblk, int Bk, int d, uint8_t* k,
                            uint8_t* ks, cudaStream_t st);
int launch_retile_keyscales(const uint8_t* in, int64_t batch, int64_t S, int64_t d, uint8_t* out, cudaStream_t st);

// q/k/v_codes: byte codes as the caller gave them, or -- for 6-bit formats -- the packed copies made by
// launch_pack_rows (Q, K) and launch_pack_transpose (V, stored [d][keys]).
int launch_prefill(const rk_prefill_args& a, const uint8_t* q_codes, const uint8_t* k_codes, const uint8_t* v_codes,
                   const uint8_t* q_sf, const uint8_t* k_sf, const uint8_t* v_sf, cudaStream_t st);

int launch_rope_quantize_rows(const float* x, int64_t rows, int d, const int32_t* pos, int seq_len, int pos0, const float* cos_h,
                              const float* sin_h, int fmt, uint8_t* codes, uint8_t* scales, cudaStream_t st);
int launch_kv_append(const float* k_new, const float* v_new, int B, int H_kv, int L, int d, const int32_t* pos, int fmt,
                     uint8_t* k_codes, uint8_t* k_scales, uint8_t* v_codes, uint8_t* v_scales, cudaStream_t st);
int launch_decode(const rk_decode_args& a, int num_splits, cudaStream_t st);
int launch_decode_noalloc(const rk_decode_args& a, cudaStream_t st);
int noalloc_status_read_clear();                            // status word of the no-allocation decode path: read, then clear
int launch_mxfp8_mma_loop(const uint8_t* a_tile, const uint8_t* b_tile, int iters, cudaStream_t st);   // tensor-pipe ceiling probe
int launch_wait_runs_out(int limit_us, bool noalloc, cudaStream_t st);   // test hook: a bounded wait that must give up
extern int g_decode_path;                                   // test hook: 0 = by shape, 1 = mma.sync kernel only
bool decode_uses_tc(const rk_decode_args& a);                // true when the tcgen05 decode kernel serves this call
int decode_ctas_per_sm(const rk_decode_args& a);             // resident CTAs per SM of the kernel that serves it

}  // namespace rk
