// extern "C" entry points of librk_mx_attn.so: argument validation, workspace
// carving, the preparation passes and the kernel launches.  See
// include/rk_mx_attn.h for the contract of every function.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <mutex>

#include "rk_internal.h"

namespace rk {
extern int g_prefill_perturb;

// The status word kernels record a given-up wait in: part of the library image (zero at load) on every device,
// so it can never fail to allocate; its device address is looked up once per device.
static __device__ int g_status_word;

namespace {
struct DeviceState { int sms = 0; int* status = nullptr; };
std::mutex g_mu;
DeviceState g_dev[64];

DeviceState dev_state() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return DeviceState();
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& s = g_dev[dev & 63];
  if (s.sms == 0 || !s.status) {                 // a failed lookup is not cached: the next call tries again
    int sms = 0;
    void* ptr = nullptr;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return DeviceState();
    if (cudaGetSymbolAddress(&ptr, g_status_word) != cudaSuccess || !ptr) { cudaGetLastError(); return DeviceState(); }
    s.sms = sms;
    s.status = static_cast<int*>(ptr);
  }
  return s;
}
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
}  // namespace

int num_sms() { const int n = dev_state().sms; return n > 0 ? n : 1; }
int* device_status_word() { return dev_state().status; }

extern float* g_prefill_dbg;
cudaEvent_t g_ev_before = nullptr, g_ev_after = nullptr;

// bits of an element code in the packed form the tensor core reads: 8, 6 (E2M3, E3M2) or 4 (E2M1)
static int fmt_bits(int fmt) { return fmt == RK_FMT_E2M1 ? 4 : fmt >= RK_FMT_E2M3 ? 6 : 8; }

struct PrefillWs { size_t q_sf, k_sf, v_sf, v_codes, q6, k6, v6t, total; };

static PrefillWs prefill_ws(const rk_prefill_args& a) {
  const size_t dch = (a.d + 127) / 128, nqt = (a.S_q + 127) / 128, nkt = (a.S_kv + 127) / 128;
  PrefillWs w;
  size_t off = 0;
  w.q_sf = off; off = align_up(off + (size_t)a.B * a.H * nqt * dch * 512, 1024);
  w.k_sf = off; off = align_up(off + (size_t)a.B * a.H_kv * nkt * dch * 512, 1024);
  w.v_sf = off; off = align_up(off + (size_t)a.B * a.H_kv * nkt * dch * 512, 1024);
  w.v_codes = off;
  if (a.v_scale_axis == RK_V_SCALES_ALONG_D) off = align_up(off + (size_t)a.B * a.H_kv * a.S_kv * a.d, 1024);
  // 6-bit and 4-bit operands: densely packed copies (Q, K along d; V transposed, along the keys), rows padded to
  // 128 codes; sized for 6 bits, which also holds 4
  const size_t dp = dch * 128, skp = nkt * 128;
  w.q6 = off;
  if (a.q_fmt >= RK_FMT_E2M3 && !a.q_packed) off = align_up(off + (size_t)a.B * a.H * a.S_q * dp * 3 / 4, 1024);
  w.k6 = off;
  if (a.kv_fmt >= RK_FMT_E2M3 && !a.kv_packed) off = align_up(off + (size_t)a.B * a.H_kv * a.S_kv * dp * 3 / 4, 1024);
  w.v6t = off;
  if (a.kv_fmt >= RK_FMT_E2M3 && !a.kv_packed) off = align_up(off + (size_t)a.B * a.H_kv * a.d * skp * 3 / 4, 1024);
  w.total = off;
  return w;
}

static int check_prefill_shape(const rk_prefill_args* a) {
  if (!a) return RK_ERR_NULL_POINTER;
  if (a->B <= 0 || a->H <= 0 || a->H_kv <= 0 || a->S_q <= 0 || a->S_kv <= 0) return RK_ERR_BAD_SHAPE;
  if (a->d != 64 && a->d != 128 && a->d != 256) return RK_ERR_BAD_SHAPE;
  if (a->H % a->H_kv != 0) return RK_ERR_BAD_SHAPE;
  if (a->window < 0 || a->softcap < 0.0f || a->softmax_scale < 0.0f) return RK_ERR_BAD_SHAPE;
  if (a->v_scale_axis != RK_V_SCALES_ALONG_KEYS && a->v_scale_axis != RK_V_SCALES_ALONG_D) return RK_ERR_BAD_FORMAT;
  if (a->q_fmt < 0 || a->q_fmt > RK_FMT_E2M1 || a->kv_fmt < 0 || a->kv_fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (a->block_n != 0 && a->block_n != 128) return RK_ERR_UNSUPPORTED;
  if (a->q_scale_layout < 0 || a->q_scale_layout > RK_SCALES_SF_ATOMS || a->k_scale_layout < 0 ||
      a->k_scale_layout > RK_SCALES_SF_ATOMS)
    return RK_ERR_BAD_FORMAT;
  if (a->v_scale_layout != RK_SCALES_ROWMAJOR &&
      !(a->v_scale_layout == RK_SCALES_SF_ATOMS && a->v_scale_axis == RK_V_SCALES_ALONG_KEYS))
    return RK_ERR_BAD_FORMAT;
  // dense sub-byte operands: only formats that have a dense form; V then has to be blocked along the keys already
  if (a->q_packed && a->q_fmt < RK_FMT_E2M3) return RK_ERR_BAD_FORMAT;
  if (a->kv_packed && (a->kv_fmt < RK_FMT_E2M3 || a->v_scale_axis != RK_V_SCALES_ALONG_KEYS)) return RK_ERR_BAD_FORMAT;
  return RK_OK;
}

}  // namespace rk

using namespace rk;

extern "C" {

const char* rk_error_string(int code) {
  switch (code) {
    case RK_OK: return "ok";
    case RK_ERR_NULL_POINTER: return "null pointer";
    case RK_ERR_BAD_SHAPE: return "bad shape";
    case RK_ERR_BAD_FORMAT: return "bad element format or layout";
    case RK_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
    case RK_ERR_MISALIGNED: return "tensor pointer not 16-byte aligned";
    case RK_ERR_UNSUPPORTED: return "not implemented in this build";
    case RK_ERR_NO_DEVICE: return "no usable device or driver entry point";
    case RK_ERR_KERNEL_TIMEOUT: return "a bounded device-side wait gave up";
    case RK_ERR_TOO_LARGE: return "request exceeds a fixed capacity";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}

int rk_version(void) { return 200; }

int rk_mx_quantize(const float* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales, void* stream) {
  if (!x || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (rows < 0 || cols < 0 || cols % 32 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 16) || !aligned(codes, 8)) return RK_ERR_MISALIGNED;
  return launch_quantize_rows(x, rows, cols, fmt, codes, scales, (cudaStream_t)stream);
}

int rk_mx_quantize_bf16(const void* x, int64_t rows, int64_t cols, int fmt, uint8_t* codes, uint8_t* scales, void* stream) {
  if (!x || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (rows < 0 || cols < 0 || cols % 32 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 16) || !aligned(codes, 8)) return RK_ERR_MISALIGNED;
  return launch_quantize_rows_bf16(x, rows, cols, fmt, codes, scales, (cudaStream_t)stream);
}

int rk_mx_quantize_keys(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt, uint8_t* codes,
                        uint8_t* scales, void* stream) {
  if (!x || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (batch < 0 || rows < 0 || cols < 0 || cols % 4 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 16) || !aligned(codes, 4) || !aligned(scales, 4)) return RK_ERR_MISALIGNED;
  return launch_quantize_keys(x, batch, rows, cols, fmt, codes, scales, (cudaStream_t)stream);
}

int rk_mx_quantize_ex(const void* x, int x_is_bf16, int64_t batch, int64_t S, int64_t d, int fmt, uint8_t* codes,
                      uint8_t* scales, int scale_layout, void* stream) {
  if (!x || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (batch < 0 || S < 0 || d < 0 || d % 32 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (scale_layout < 0 || scale_layout > RK_SCALES_SF_ATOMS) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 16) || !aligned(codes, 8)) return RK_ERR_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  if (scale_layout == RK_SCALES_SF_ATOMS) {
    if (!aligned(scales, 16)) return RK_ERR_MISALIGNED;
    if (S % 128 != 0 || d % 128 != 0) {   // bytes of rows / blocks past the edge are never written by the kernel
      const size_t bytes = (size_t)batch * ((S + 127) / 128) * ((d + 127) / 128) * 512;
      cudaError_t e = cudaMemsetAsync(scales, 0x7F, bytes, st);
      if (e != cudaSuccess) return (int)e;
    }
  }
  return launch_quantize_rows_ex(x, x_is_bf16 != 0, batch, S, d, fmt, codes, scales, scale_layout, st);
}

int rk_mx_quantize_keys_ex(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt, uint8_t* codes,
                           uint8_t* scales, int scale_layout, void* stream) {
  if (scale_layout == RK_SCALES_ROWMAJOR) return rk_mx_quantize_keys(x, batch, rows, cols, fmt, codes, scales, stream);
  if (scale_layout != RK_SCALES_SF_ATOMS) return RK_ERR_BAD_FORMAT;
  if (!x || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (batch < 0 || rows < 0 || cols < 0 || cols % 4 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 16) || !aligned(codes, 4) || !aligned(scales, 16)) return RK_ERR_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows % 128 != 0 || cols % 128 != 0) {
    const size_t bytes = (size_t)batch * ((rows + 127) / 128) * ((cols + 127) / 128) * 512;
    cudaError_t e = cudaMemsetAsync(scales, 0x7F, bytes, st);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_quantize_keys_atoms(x, batch, rows, cols, fmt, codes, scales, st);
}

int rk_import_kt_blocks(const uint8_t* kt_blocks, const uint8_t* kt_scale_blocks, int64_t heads, int32_t n_blocks,
                        int32_t Bk, int32_t d, uint8_t* k_codes, uint8_t* k_scales, void* stream) {
  if (!kt_blocks || !kt_scale_blocks || !k_codes || !k_scales) return RK_ERR_NULL_POINTER;
  if (heads < 0 || n_blocks < 0 || Bk <= 0 || d <= 0 || Bk % 32 != 0 || d % 32 != 0) return RK_ERR_BAD_SHAPE;
  return launch_import_kt_blocks(kt_blocks, kt_scale_blocks, heads, n_blocks, Bk, d, k_codes, k_scales, (cudaStream_t)stream);
}

int rk_mx_rebase_v(const uint8_t* codes, const uint8_t* scales, int64_t batch, int64_t S, int64_t d, int fmt,
                   uint8_t* out_codes, uint8_t* out_scales, void* stream) {
  if (!codes || !scales || !out_codes || !out_scales) return RK_ERR_NULL_POINTER;
  if (batch < 0 || S < 0 || d <= 0 || d % 32 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(codes, 4) || !aligned(out_codes, 4) || !aligned(out_scales, 4)) return RK_ERR_MISALIGNED;
  return launch_rebase_v(codes, scales, batch, S, d, fmt, out_codes, out_scales, false, (cudaStream_t)stream);
}

static size_t packed_len(int64_t n, int fmt) { return (size_t)((n + 127) / 128 * 128) * fmt_bits(fmt) / 8; }

size_t rk_mx_packed_rows_bytes(int64_t rows, int64_t d, int fmt) {
  if (rows < 0 || d <= 0 || fmt < RK_FMT_E2M3 || fmt > RK_FMT_E2M1) return 0;
  return (size_t)rows * packed_len(d, fmt);
}

int rk_mx_pack_rows(const uint8_t* codes, int64_t rows, int64_t d, int fmt, uint8_t* out, void* stream) {
  if (!codes || !out) return RK_ERR_NULL_POINTER;
  if (rows < 0 || d <= 0 || d % 16 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < RK_FMT_E2M3 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(codes, 16) || !aligned(out, 16)) return RK_ERR_MISALIGNED;
  return launch_pack_rows(codes, rows, d, fmt_bits(fmt), out, (cudaStream_t)stream);
}

size_t rk_mx_packed_vt_bytes(int64_t batch, int64_t S, int64_t d, int fmt) {
  if (batch < 0 || S <= 0 || d <= 0 || fmt < RK_FMT_E2M3 || fmt > RK_FMT_E2M1) return 0;
  return (size_t)batch * d * packed_len(S, fmt);
}

int rk_mx_pack_vt(const uint8_t* v_codes, int64_t batch, int64_t S, int64_t d, int fmt, uint8_t* out, void* stream) {
  if (!v_codes || !out) return RK_ERR_NULL_POINTER;
  if (batch < 0 || S <= 0 || d <= 0 || d % 16 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < RK_FMT_E2M3 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(v_codes, 16) || !aligned(out, 16)) return RK_ERR_MISALIGNED;
  return launch_pack_transpose(v_codes, batch, S, d, fmt_bits(fmt), out, (cudaStream_t)stream);
}

int rk_attn_prefill_block_n(const rk_prefill_args* a) { (void)a; return 128; }

size_t rk_attn_prefill_workspace_bytes(const rk_prefill_args* a) {
  if (check_prefill_shape(a) != RK_OK) return 0;
  return prefill_ws(*a).total;
}

int rk_attn_prefill(const rk_prefill_args* a, void* stream) {
  int rc = check_prefill_shape(a);
  if (rc != RK_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->q_scale || !a->k_scale || !a->v_scale || !a->o) return RK_ERR_NULL_POINTER;
  if (!aligned(a->q, 16) || !aligned(a->k, 16) || !aligned(a->v, 16) || !aligned(a->o, 16)) return RK_ERR_MISALIGNED;
  const PrefillWs w = prefill_ws(*a);
  if (!a->workspace || a->workspace_bytes < w.total || !aligned(a->workspace, 256)) return RK_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* ws = reinterpret_cast<uint8_t*>(a->workspace);
  const int64_t bhq = (int64_t)a->B * a->H, bhkv = (int64_t)a->B * a->H_kv;

  // Q / K scales -> scale-factor atoms (or the caller's atoms as they lie)
  const uint8_t* q_sf = ws + w.q_sf;
  const uint8_t* k_sf = ws + w.k_sf;
  const uint8_t* v_sf = ws + w.v_sf;
  // the usual call (row-major Q and K scales, V scaled along d): the V re-blocking launch re-tiles the Q and K scales
  // on the side, two launches in all instead of four
  const bool fused_retile = a->q_scale_layout == RK_SCALES_ROWMAJOR && a->k_scale_layout == RK_SCALES_ROWMAJOR &&
                            a->v_scale_axis == RK_V_SCALES_ALONG_D;
  if (!fused_retile) {
    if (a->q_scale_layout == RK_SCALES_SF_ATOMS) {
      if (!aligned(a->q_scale, 16)) return RK_ERR_MISALIGNED;
      q_sf = a->q_scale;
    } else if ((rc = (a->q_scale_layout == RK_SCALES_GROUPMAJOR ? launch_retile_groupscales : launch_retile_rowscales)(
                    a->q_scale, bhq, a->S_q, a->d, ws + w.q_sf, st)) != RK_OK) {
      return rc;
    }
    if (a->k_scale_layout == RK_SCALES_SF_ATOMS) {
      if (!aligned(a->k_scale, 16)) return RK_ERR_MISALIGNED;
      k_sf = a->k_scale;
    } else if ((rc = (a->k_scale_layout == RK_SCALES_GROUPMAJOR ? launch_retile_groupscales : launch_retile_rowscales)(
                    a->k_scale, bhkv, a->S_kv, a->d, ws + w.k_sf, st)) != RK_OK) {
      return rc;
    }
  }
  const uint8_t* v_codes = a->v;
  if (a->v_scale_axis == RK_V_SCALES_ALONG_D) {
    if (a->S_kv % 128 != 0 || a->d % 128 != 0) {
      // atoms of ragged tiles keep bytes the re-blocking pass never writes: make them 2^0
      cudaError_t e = cudaMemsetAsync(ws + w.v_sf, 0x7F, w.v_codes - w.v_sf, st);
      if (e != cudaSuccess) return (int)e;
    }
    if ((rc = launch_rebase_v(a->v, a->v_scale, bhkv, a->S_kv, a->d, a->kv_fmt, ws + w.v_codes, ws + w.v_sf, true, st,
                              fused_retile ? a->q_scale : nullptr, bhq, a->S_q, ws + w.q_sf, fused_retile ? a->k_scale : nullptr,
                              ws + w.k_sf)) != RK_OK)
      return rc;
    v_codes = ws + w.v_codes;
  } else if (a->v_scale_layout == RK_SCALES_SF_ATOMS) {
    if (!aligned(a->v_scale, 16)) return RK_ERR_MISALIGNED;
    v_sf = a->v_scale;
  } else {
    if ((rc = launch_retile_keyscales(a->v_scale, bhkv, a->S_kv, a->d, ws + w.v_sf, st)) != RK_OK) return rc;
  }
  const uint8_t* q_codes = a->q;
  const uint8_t* k_codes = a->k;
  if (a->q_fmt >= RK_FMT_E2M3 && !a->q_packed) {
    if ((rc = launch_pack_rows(a->q, bhq * a->S_q, a->d, fmt_bits(a->q_fmt), ws + w.q6, st)) != RK_OK) return rc;
    q_codes = ws + w.q6;
  }
  if (a->kv_fmt >= RK_FMT_E2M3 && !a->kv_packed) {
    if ((rc = launch_pack_rows(a->k, bhkv * a->S_kv, a->d, fmt_bits(a->kv_fmt), ws + w.k6, st)) != RK_OK) return rc;
    k_codes = ws + w.k6;
    if ((rc = launch_pack_transpose(v_codes, bhkv, a->S_kv, a->d, fmt_bits(a->kv_fmt), ws + w.v6t, st)) != RK_OK) return rc;
    v_codes = ws + w.v6t;
  }
  return launch_prefill(*a, q_codes, k_codes, v_codes, q_sf, k_sf, v_sf, st);
}

size_t rk_attn_prefill_host_arena_bytes(const rk_prefill_args* a) {
  if (check_prefill_shape(a) != RK_OK) return 0;
  const size_t nbd = a->d / 32;
  const size_t q = (size_t)a->B * a->H * a->S_q * a->d, kv = (size_t)a->B * a->H_kv * a->S_kv * a->d;
  const size_t vs = a->v_scale_axis == RK_V_SCALES_ALONG_D ? kv / 32 : (size_t)a->B * a->H_kv * ((a->S_kv + 31) / 32) * a->d;
  size_t off = 0;
  off = align_up(off + q, 1024); off = align_up(off + kv, 1024); off = align_up(off + kv, 1024);
  off = align_up(off + q / a->d * nbd, 1024); off = align_up(off + kv / a->d * nbd, 1024); off = align_up(off + vs, 1024);
  off = align_up(off + q * 2, 1024); off = align_up(off + q / a->d * 4, 1024);
  return off + prefill_ws(*a).total;
}

// Copy streams and events of the host-buffer entry point, one set per device, made on first use.
namespace {
constexpr int kHostMaxChunks = 16;
struct HostPipe {
  bool ready = false;
  cudaStream_t h2d = nullptr, d2h = nullptr;
  cudaEvent_t start = nullptr, end = nullptr, in[kHostMaxChunks] = {}, out[kHostMaxChunks] = {};
};
HostPipe g_host_pipe[64];
std::mutex g_host_pipe_mu;

int host_pipe_init(HostPipe& hp) {
  if (hp.ready) return RK_OK;
  cudaError_t e;
  if ((e = cudaStreamCreateWithFlags(&hp.h2d, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
  if ((e = cudaStreamCreateWithFlags(&hp.d2h, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
  if ((e = cudaEventCreateWithFlags(&hp.start, cudaEventDisableTiming)) != cudaSuccess) return (int)e;
  if ((e = cudaEventCreateWithFlags(&hp.end, cudaEventDisableTiming)) != cudaSuccess) return (int)e;
  for (int i = 0; i < kHostMaxChunks; ++i) {
    if ((e = cudaEventCreateWithFlags(&hp.in[i], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
    if ((e = cudaEventCreateWithFlags(&hp.out[i], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
  }
  hp.ready = true;
  return RK_OK;
}
}  // namespace

// Host buffers in, host buffer out.  The (batch, KV head) units are independent, so the call is cut into a few
// chunks of whole units and pipelined: chunk c+1 crosses PCIe on a copy stream while chunk c is computed on
// the caller's stream and the output of chunk c-1 goes back on a second copy stream.
int rk_attn_prefill_host(const rk_prefill_args* h, void* arena, size_t arena_bytes, void* stream) {
  int rc = check_prefill_shape(h);
  if (rc != RK_OK) return rc;
  if (!h->q || !h->k || !h->v || !h->q_scale || !h->k_scale || !h->v_scale || !h->o || !arena) return RK_ERR_NULL_POINTER;
  // the chunk offsets below are those of row-major scales and of codes one per byte
  if (h->q_scale_layout != RK_SCALES_ROWMAJOR || h->k_scale_layout != RK_SCALES_ROWMAJOR || h->v_scale_layout != RK_SCALES_ROWMAJOR ||
      h->q_packed || h->kv_packed)
    return RK_ERR_UNSUPPORTED;
  if (arena_bytes < rk_attn_prefill_host_arena_bytes(h) || !aligned(arena, 256)) return RK_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t nbd = h->d / 32;
  const size_t q = (size_t)h->B * h->H * h->S_q * h->d, kv = (size_t)h->B * h->H_kv * h->S_kv * h->d;
  const size_t qs = q / h->d * nbd, ks = kv / h->d * nbd;
  const bool v_along_d = h->v_scale_axis == RK_V_SCALES_ALONG_D;
  const size_t vs_head = v_along_d ? (size_t)h->S_kv * nbd : (size_t)((h->S_kv + 31) / 32) * h->d;   // V scale bytes per KV head
  const size_t vs = (size_t)h->B * h->H_kv * vs_head;
  uint8_t* base = reinterpret_cast<uint8_t*>(arena);
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* p = base + off; off = align_up(off + bytes, 1024); return p; };
  uint8_t* dq = take(q); uint8_t* dk = take(kv); uint8_t* dv = take(kv);
  uint8_t* dqs = take(qs); uint8_t* dks = take(ks); uint8_t* dvs = take(vs);
  uint8_t* dout = take(q * 2); uint8_t* dlse = take(q / h->d * 4);
  uint8_t* ws = base + off;
  const size_t ws_bytes = arena_bytes - off;

  int dev = 0;
  cudaError_t e;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
  std::lock_guard<std::mutex> lk(g_host_pipe_mu);      // one pipelined call per process at a time: the streams are shared
  HostPipe& hp = g_host_pipe[dev & 63];
  if ((rc = host_pipe_init(hp)) != RK_OK) return rc;

  // Chunks are contiguous ranges of (batch, KV head) units; a range of n units is a problem of its own with
  // B = n, H = heads per KV head, H_kv = 1.  Every copy costs some tens of microseconds on top of its bytes, so there
  // are few of them: all scales go over first (three copies), then five chunks of 1/2, 1/4, 1/8, 1/16 and 1/16 of
  // the units -- what cannot overlap with the inbound copies is the last chunk's compute and its copy back, so the
  // last chunks are the small ones (measured on C2: 2 chunks 5.67 ms, 3 5.55, 4 5.01-5.21, 5 4.99-5.13, 6 5.02, 8 5.14;
  // eight equal chunks with per-chunk scale copies 6.7).
  const int grp = h->H / h->H_kv;
  const int64_t units = (int64_t)h->B * h->H_kv;
#ifndef RK_HOST_CHUNKS
#define RK_HOST_CHUNKS 5
#endif
  constexpr int kTarget = RK_HOST_CHUNKS;
  static_assert(kTarget >= 1 && kTarget <= kHostMaxChunks, "event pool");
  int64_t chunk_units[kHostMaxChunks];
  int n_chunks = 0;
  {
    int64_t left = units;
    for (int i = 0; i < kTarget && left > 0; ++i) {
      int64_t n = (i == kTarget - 1) ? left : std::max<int64_t>(1, (units + (2ll << i) - 1) / (2ll << i));
      n = std::min(n, left);
      chunk_units[n_chunks++] = n;
      left -= n;
    }
    if (left > 0) chunk_units[n_chunks - 1] += left;
  }

  // an error in the middle leaves copies and kernels queued on three streams: wait for them before handing the
  // buffers back to the caller
  auto drain = [&](int code) {
    cudaStreamSynchronize(hp.h2d); cudaStreamSynchronize(st); cudaStreamSynchronize(hp.d2h);
    return code;
  };
  if ((e = cudaEventRecord(hp.start, st)) != cudaSuccess) return drain((int)e);
  if ((e = cudaStreamWaitEvent(hp.h2d, hp.start, 0)) != cudaSuccess) return drain((int)e);
  if ((e = cudaStreamWaitEvent(hp.d2h, hp.start, 0)) != cudaSuccess) return drain((int)e);
  const size_t q_row = (size_t)h->S_q * h->d, k_row = (size_t)h->S_kv * h->d;
#define RK_CP(dst, src, o, n) if ((e = cudaMemcpyAsync((dst) + (o), reinterpret_cast<const uint8_t*>(src) + (o), n, cudaMemcpyHostToDevice, hp.h2d)) != cudaSuccess) return drain((int)e)
  RK_CP(dqs, h->q_scale, 0, qs);
  RK_CP(dks, h->k_scale, 0, ks);
  RK_CP(dvs, h->v_scale, 0, vs);
  int64_t u0 = 0;
  for (int c = 0; c < n_chunks; ++c) {
    const int64_t nu = chunk_units[c];
    const size_t qh = (size_t)u0 * grp, kh = (size_t)u0;             // first query head / KV head of the chunk
    const size_t nqh = (size_t)nu * grp, nkh = (size_t)nu;
    RK_CP(dq, h->q, qh * q_row, nqh * q_row);
    RK_CP(dk, h->k, kh * k_row, nkh * k_row);
    RK_CP(dv, h->v, kh * k_row, nkh * k_row);
    if ((e = cudaEventRecord(hp.in[c], hp.h2d)) != cudaSuccess) return drain((int)e);
    if ((e = cudaStreamWaitEvent(st, hp.in[c], 0)) != cudaSuccess) return drain((int)e);
    rk_prefill_args d = *h;
    d.B = (int32_t)nu; d.H = grp; d.H_kv = 1;
    d.q = dq + qh * q_row; d.k = dk + kh * k_row; d.v = dv + kh * k_row;
    d.q_scale = dqs + qh * q_row / 32; d.k_scale = dks + kh * k_row / 32; d.v_scale = dvs + kh * vs_head;
    d.o = dout + qh * q_row * 2;
    d.lse = h->lse ? reinterpret_cast<float*>(dlse) + qh * h->S_q : nullptr;
    d.workspace = ws; d.workspace_bytes = ws_bytes;       // chunks run one after the other on `st`: one workspace serves all
    if ((rc = rk_attn_prefill(&d, stream)) != RK_OK) return drain(rc);
    if ((e = cudaEventRecord(hp.out[c], st)) != cudaSuccess) return drain((int)e);
    if ((e = cudaStreamWaitEvent(hp.d2h, hp.out[c], 0)) != cudaSuccess) return drain((int)e);
    if ((e = cudaMemcpyAsync(reinterpret_cast<uint8_t*>(h->o) + qh * q_row * 2, dout + qh * q_row * 2, nqh * q_row * 2,
                             cudaMemcpyDeviceToHost, hp.d2h)) != cudaSuccess) return drain((int)e);
    if (h->lse && (e = cudaMemcpyAsync(h->lse + qh * h->S_q, reinterpret_cast<float*>(dlse) + qh * h->S_q,
                                       nqh * h->S_q * 4, cudaMemcpyDeviceToHost, hp.d2h)) != cudaSuccess) return drain((int)e);
    u0 += nu;
  }
#undef RK_CP
  if ((e = cudaEventRecord(hp.end, hp.d2h)) != cudaSuccess) return drain((int)e);
  if ((e = cudaStreamWaitEvent(st, hp.end, 0)) != cudaSuccess) return drain((int)e);
  return (int)cudaStreamSynchronize(st);
}

// ------------------------------------------------------------------------------------------------
static int check_decode_shape(const rk_decode_args* a) {
  if (!a) return RK_ERR_NULL_POINTER;
  if (a->B <= 0 || a->H <= 0 || a->H_kv <= 0 || a->L <= 0) return RK_ERR_BAD_SHAPE;
  if (a->d != 128) return RK_ERR_BAD_SHAPE;
  if (a->H % a->H_kv != 0) return RK_ERR_BAD_SHAPE;
  const int grp = a->H / a->H_kv;
  if (grp != 1 && grp != 2 && grp != 4 && grp != 8) return RK_ERR_BAD_SHAPE;
  if (a->L % 4 != 0) return RK_ERR_BAD_SHAPE;   // keeps every scale-row copy a 16-byte multiple
  if (a->kv_fmt < 0 || a->kv_fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (a->num_splits < 0 || a->num_splits > 64 || a->softmax_scale < 0.0f) return RK_ERR_BAD_SHAPE;
  return RK_OK;
}

int rk_rope_mx_quantize(const float* x, int64_t rows, int32_t d, const int32_t* pos, int32_t seq_len, int32_t pos0,
                        const float* cos_half, const float* sin_half, int32_t n_pos, int32_t fmt, uint8_t* codes,
                        uint8_t* scales, void* stream) {
  if (!x || !cos_half || !sin_half || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (rows < 0 || d <= 0 || d % 64 != 0 || n_pos <= 0) return RK_ERR_BAD_SHAPE;      // both halves are whole blocks
  if (!pos && (seq_len <= 0 || pos0 < 0 || (int64_t)pos0 + seq_len > n_pos)) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 16) || !aligned(cos_half, 16) || !aligned(sin_half, 16) || !aligned(codes, 8)) return RK_ERR_MISALIGNED;
  return launch_rope_quantize_rows(x, rows, d, pos, seq_len, pos0, cos_half, sin_half, fmt, codes, scales, (cudaStream_t)stream);
}

int rk_rmsnorm_mx_quantize(const void* x, int x_is_bf16, int64_t rows, int32_t K, const float* gamma, float eps, int32_t fmt,
                           int32_t unit_scale, uint8_t* codes, uint8_t* scales, void* stream) {
  if (!x || !gamma || !codes || !scales) return RK_ERR_NULL_POINTER;
  if (rows < 0 || K <= 0 || K % 32 != 0 || !(eps >= 0.0f)) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(x, 4) || !aligned(gamma, 4) || !aligned(codes, 16)) return RK_ERR_MISALIGNED;
  return launch_rmsnorm_quantize(x, x_is_bf16 != 0, rows, K, gamma, eps, fmt, unit_scale != 0, codes, scales, (cudaStream_t)stream);
}

int rk_mx_gemm_hw(const uint8_t* a, const uint8_t* b, const uint8_t* a_scales, const uint8_t* b_scales, int32_t M, int32_t N,
                  int32_t K, void* c_bf16, void* stream) {
  if (!a || !b || !a_scales || !b_scales || !c_bf16) return RK_ERR_NULL_POINTER;
  if (M < 0 || N < 0 || K < 0 || M % 16 != 0 || N % 16 != 0 || K % 32 != 0) return RK_ERR_BAD_SHAPE;
  if (!aligned(a, 16) || !aligned(c_bf16, 2)) return RK_ERR_MISALIGNED;
  return launch_mx_gemm_hw(a, b, a_scales, b_scales, M, N, K, reinterpret_cast<uint16_t*>(c_bf16), (cudaStream_t)stream);
}

int rk_kv_cache_append(const float* k_new, const float* v_new, int32_t B, int32_t H_kv, int32_t L, int32_t d,
                       const int32_t* pos, int32_t fmt, uint8_t* k_codes, uint8_t* k_scales, uint8_t* v_codes,
                       uint8_t* v_scales, void* stream) {
  if (!k_new || !v_new || !pos || !k_codes || !k_scales || !v_codes || !v_scales) return RK_ERR_NULL_POINTER;
  if (B < 0 || H_kv < 0 || L <= 0 || d <= 0 || d % 32 != 0) return RK_ERR_BAD_SHAPE;
  if (fmt < 0 || fmt > RK_FMT_E2M1) return RK_ERR_BAD_FORMAT;
  if (!aligned(k_new, 16) || !aligned(v_new, 16) || !aligned(k_codes, 8) || !aligned(v_codes, 8)) return RK_ERR_MISALIGNED;
  return launch_kv_append(k_new, v_new, B, H_kv, L, d, pos, fmt, k_codes, k_scales, v_codes, v_scales, (cudaStream_t)stream);
}

int rk_attn_decode_num_splits(const rk_decode_args* a) {
  if (check_decode_shape(a) != RK_OK) return 0;
  const int tiles = (a->L + 127) / 128;
  if (a->num_splits > 0) return a->num_splits < tiles ? a->num_splits : tiles;
  // Pick the split count with the lowest modelled time (microseconds; fitted to B = 1 .. 64 at L = 4096 .. 32768 with
  // 32 and 64 heads on 8): streaming time = bytes / bandwidth, where the bandwidth grows with the number of CTAs in
  // flight as (CTAs / slots)^0.8 up to the 6.5 TB/s of a full machine (two CTAs fit on an SM; 128 CTAs reach 3.3
  // TB/s, 256 reach 5) and a last, partly filled wave costs half of what strict waves would; plus 10 us for the
  // first wave and 3 for each further one.  Fewer splits win unless more are 3 % faster.  (The wave-efficiency rule
  // used before took 23 splits at B = 8, L = 32768: 142 us against 118 with 4; and 4 at B = 64, L = 4096: 146 us
  // against 126 with 1.)
  const long slots = (long)decode_ctas_per_sm(*a) * num_sms(), units = (long)a->B * a->H_kv;
  const double stream_us = (double)units * tiles * (2.0 * 128 * 132 / 6.5e6);      // K + V tile with scales at 6.5 TB/s
  int best = 1; double best_t = 1e30;
  for (int s = 1; s <= 64 && (s == 1 || tiles / s >= 4); ++s) {
    const long ctas = units * s, waves = (ctas + slots - 1) / slots;
    double bw = 1.0;
    if (ctas < slots) bw = std::pow((double)ctas / (double)slots, 0.8);
    else bw = 0.5 * (1.0 + (double)ctas / (double)(waves * slots));
    const double t = 10.0 + 3.0 * (double)(waves - 1) + stream_us / bw;
    if (t < best_t * 0.97) { best_t = t; best = s; }
  }
  return best;
}

size_t rk_attn_decode_workspace_bytes(const rk_decode_args* a) {
  const int ns = rk_attn_decode_num_splits(a);
  if (ns <= 0) return 0;
  return (size_t)a->B * a->H * ns * (128 + 2) * sizeof(float);
}

int rk_attn_decode(const rk_decode_args* a, void* stream) {
  int rc = check_decode_shape(a);
  if (rc != RK_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->k_scale || !a->v_scale || !a->o) return RK_ERR_NULL_POINTER;
  if (!aligned(a->q, 16) || !aligned(a->k, 16) || !aligned(a->v, 16) || !aligned(a->k_scale, 16) ||
      !aligned(a->v_scale, 16) || !aligned(a->o, 16))
    return RK_ERR_MISALIGNED;
  const int ns = rk_attn_decode_num_splits(a);
  if (!a->workspace || a->workspace_bytes < rk_attn_decode_workspace_bytes(a) || !aligned(a->workspace, 16))
    return RK_ERR_WORKSPACE;
  return launch_decode(*a, ns, (cudaStream_t)stream);
}

int rk_attn_decode_noalloc(const rk_decode_args* a, void* stream) {
  int rc = check_decode_shape(a);
  if (rc != RK_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->k_scale || !a->v_scale || !a->o) return RK_ERR_NULL_POINTER;
  if (!aligned(a->q, 16) || !aligned(a->k, 16) || !aligned(a->v, 16) || !aligned(a->k_scale, 16) ||
      !aligned(a->v_scale, 16) || !aligned(a->o, 16))
    return RK_ERR_MISALIGNED;
  if (a->kv_fmt != RK_FMT_E4M3) return RK_ERR_UNSUPPORTED;      // this entry always takes the mma.sync kernel
  return launch_decode_noalloc(*a, (cudaStream_t)stream);
}

int rk_shard_units(int64_t n_units, int32_t rank, int32_t world, int64_t* begin, int64_t* end) {
  if (!begin || !end) return RK_ERR_NULL_POINTER;
  if (n_units < 0 || world <= 0 || rank < 0 || rank >= world) return RK_ERR_BAD_SHAPE;
  const int64_t base = n_units / world, rem = n_units % world;
  *begin = rank * base + (rank < rem ? rank : rem);
  *end = *begin + base + (rank < rem ? 1 : 0);
  return RK_OK;
}

int rk_last_device_status(void) {
  int* w = device_status_word();
  if (!w) return RK_ERR_NO_DEVICE;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  int v = 0;
  if ((e = cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost)) != cudaSuccess) return (int)e;
  if (v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

int rk_attn_decode_noalloc_status(void) { return noalloc_status_read_clear(); }

void rk_profile_set_events(void* before, void* after) { g_ev_before = (cudaEvent_t)before; g_ev_after = (cudaEvent_t)after; }

/* The rk_debug_* hooks below and rk_profile_set_events above set plain process-wide variables that the launch
 * functions read: they are for tests and measurements run from one host thread, with no library call in flight on
 * another thread while a hook is changed.  The entry points of the public header keep no such state. */

/* Test hook (not in the public header): sweeps all 2^32 fp32 bit patterns and counts the inputs on which the
 * hardware element converter and the reference's integer encoder disagree (device outputs: a 64-bit count and
 * the smallest offending bit pattern, which the caller initialises to 0 and 0xFFFFFFFF). */
RK_API int rk_debug_verify_encoder(int fmt, unsigned long long* mismatches, uint32_t* first_bad, void* stream) {
  if (!mismatches || !first_bad) return RK_ERR_NULL_POINTER;
  return launch_verify_encoder(fmt, mismatches, first_bad, (cudaStream_t)stream);
}

/* Test hook (not in the public header): stage dump of the first query tile / first key tile of
 * the next prefill launches into `buf` (>= 32768 floats), or NULL to switch it off. */
RK_API void rk_debug_set_prefill_dump(float* buf) { g_prefill_dbg = buf; }

/* Test hook (not in the public header): 0 = choose the decode kernel by shape, 1 = always the mma.sync kernel. */
RK_API void rk_debug_set_decode_path(int path) { g_decode_path = path; }

/* Test hook (not in the public header): a one-CTA kernel that waits, with the library's bounded wait and a
 * limit of `limit_us` microseconds, on an mbarrier nobody ever arrives at.  The wait must run out, record
 * code 901 in the status word of the current device and let the kernel return normally.  `noalloc` != 0 uses
 * the status word of the no-allocation decode entry point instead. */
RK_API int rk_debug_wait_runs_out(int limit_us, int noalloc, void* stream) {
  return launch_wait_runs_out(limit_us, noalloc != 0, (cudaStream_t)stream);
}

/* Measurement hook (not in the public header): on every SM, `iters` back-to-back 128 x 128 x 128 block-scaled
 * MXFP8 products (four tcgen05.mma kind::mxf8f6f4 M=128 N=128 K=32 each) on one resident A tile and one resident
 * B tile of 16 KiB each (device pointers, 16-byte aligned, any valid E4M3 codes): the tensor-pipe ceiling for the
 * instruction shape the attention kernels use.  FLOP = SMs * iters * 2 * 128^3. */
RK_API int rk_debug_mxfp8_mma_loop(const uint8_t* a_tile, const uint8_t* b_tile, int iters, void* stream) {
  if (!a_tile || !b_tile) return RK_ERR_NULL_POINTER;
  if (iters <= 0 || iters > (1 << 22)) return RK_ERR_BAD_SHAPE;
  if (!aligned(a_tile, 16) || !aligned(b_tile, 16)) return RK_ERR_MISALIGNED;
  return launch_mxfp8_mma_loop(a_tile, b_tile, iters, (cudaStream_t)stream);
}

/* Test hook (not in the public header): which warp role of the d <= 128 prefill kernel sleeps a little at every key
 * tile (0 = none; 1, 2 = softmax of query tile A, B; 3 = correction; 4 = TMA producer; 5 = Q K^T issuer; 6 = P V issuer). */
RK_API void rk_debug_set_prefill_perturb(int role) { g_prefill_perturb = role; }

}  // extern "C"
