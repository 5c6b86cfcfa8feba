/* A plain C host that feeds the library the arrays of a generated fa_data.h exactly as they lie.
 *
 * The reference's attention kernels read their operands from link-time arrays of a generated header
 * (kernels/flash_attention_mx_gqa/fa_gen_data.py:122-158: QK_A_in, QK_A_scales_row, QK_B_blocks,
 * QK_B_scales_blocks, V_in, V_scales, O_gold and the FA_* macros) and report pass / fail through a tohost
 * code (lib/include/kernel_verify.h:29-44).  This program is the same protocol on the C ABI: it includes such a
 * header (written by the test that compiles it), copies the arrays to the device without touching their
 * layout, and calls
 *   rk_import_kt_blocks  for the per-block K^T tiles and their group-major scales,
 *   rk_attn_prefill      with q_scale_layout = RK_SCALES_GROUPMAJOR and V scaled along the keys,
 * then compares O with O_gold.  Exit code 0 = pass, (errors << 1) | 1 = fail, 2 = a call failed.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime_api.h>

#include "fa_data.h"
#include "rk_mx_attn.h"

static float bf16_to_float(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

#define CK(call)                                                              \
  do {                                                                        \
    int rc_ = (int)(call);                                                    \
    if (rc_ != 0) {                                                           \
      fprintf(stderr, "%s failed with code %d\n", #call, rc_);                \
      return 2;                                                               \
    }                                                                         \
  } while (0)

static void* to_device(const void* src, size_t bytes) {
  void* p = NULL;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return NULL;
  if (cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
  return p;
}

int main(void) {
  const int skv = FA_NBLK_USED * FA_BK;                 /* only the used key blocks are emitted */
  void* q = to_device(QK_A_in, sizeof QK_A_in);
  void* qs = to_device(QK_A_scales_row, sizeof QK_A_scales_row);
  void* kt = to_device(QK_B_blocks, sizeof QK_B_blocks);
  void* kts = to_device(QK_B_scales_blocks, sizeof QK_B_scales_blocks);
  void* v = to_device(V_in, sizeof V_in);
  void* vs = to_device(V_scales, sizeof V_scales);
  void *k = NULL, *ks = NULL, *o = NULL, *ws = NULL;
  if (!q || !qs || !kt || !kts || !v || !vs) return 2;
  CK(cudaMalloc(&k, (size_t)FA_NKV * skv * FA_D));
  CK(cudaMalloc(&ks, (size_t)FA_NKV * skv * FA_GK));
  CK(cudaMalloc(&o, sizeof O_gold));

  CK(rk_import_kt_blocks((const uint8_t*)kt, (const uint8_t*)kts, FA_NKV, FA_NBLK_USED, FA_BK, FA_D, (uint8_t*)k,
                         (uint8_t*)ks, NULL));

  rk_prefill_args a;
  memset(&a, 0, sizeof a);
  a.q = (const uint8_t*)q; a.k = (const uint8_t*)k; a.v = (const uint8_t*)v;
  a.q_scale = (const uint8_t*)qs; a.k_scale = (const uint8_t*)ks; a.v_scale = (const uint8_t*)vs;
  a.o = o;
  a.B = 1; a.H = FA_NQ; a.H_kv = FA_NKV; a.S_q = FA_SQ; a.S_kv = skv; a.d = FA_D;
  a.q_pos0 = FA_QPOS0; a.causal = 1;
  a.softmax_scale = bf16_to_float(FA_SOFTMAX_SCALE_BF16);
#ifdef FA_ATTN_SOFTCAP_BF16
  a.softcap = bf16_to_float(FA_ATTN_SOFTCAP_BF16);
#endif
#ifdef FA_WINDOW
  a.window = FA_WINDOW;
#endif
  a.q_fmt = RK_FMT_E4M3; a.kv_fmt = RK_FMT_E4M3;
  a.v_scale_axis = RK_V_SCALES_ALONG_KEYS;              /* V_scales[Bk/32][d] per block = [S_kv/32][d] per head */
  a.q_scale_layout = RK_SCALES_GROUPMAJOR;              /* QK_A_scales_row[FA_GK][FA_SQ] per head */
  a.k_scale_layout = RK_SCALES_ROWMAJOR;                /* as rk_import_kt_blocks wrote them */
  a.workspace_bytes = rk_attn_prefill_workspace_bytes(&a);
  if (a.workspace_bytes == 0) return 2;
  CK(cudaMalloc(&ws, a.workspace_bytes));
  a.workspace = ws;
  CK(rk_attn_prefill(&a, NULL));
  CK(cudaDeviceSynchronize());
  CK(rk_last_device_status());

  static uint16_t got[FA_NQ * FA_SQ][FA_D];
  CK(cudaMemcpy(got, o, sizeof got, cudaMemcpyDeviceToHost));
  double num = 0.0, den = 0.0, max_abs = 0.0;
  long errors = 0;
  for (int r = 0; r < FA_NQ * FA_SQ; ++r)
    for (int c = 0; c < FA_D; ++c) {
      const double g = bf16_to_float(got[r][c]), w = bf16_to_float(O_gold[r][c]);
      const double e = fabs(g - w);
      if (!(e <= 2e-2)) ++errors;                       /* also counts NaN */
      if (e > max_abs) max_abs = e;
      num += (g - w) * (g - w); den += w * w;
    }
  const double rel = sqrt(num / (den > 0.0 ? den : 1.0));
  printf("block_n %d  max_abs %.4g  rel_l2 %.4g  errors %ld\n", rk_attn_prefill_block_n(&a), max_abs, rel, errors);
  if (!(rel <= 1e-2)) ++errors;
  cudaFree(q); cudaFree(qs); cudaFree(kt); cudaFree(kts); cudaFree(v); cudaFree(vs); cudaFree(k); cudaFree(ks); cudaFree(o); cudaFree(ws);
  return errors ? (int)(((errors << 1) | 1) & 0x7F) : 0;
}
