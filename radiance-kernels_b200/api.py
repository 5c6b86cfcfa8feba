"""Torch-tensor front end of the C ABI (include/rk_mx_attn.h).

Argument names and meaning follow the reference kernels' data headers
(kernels/flash_attention_mx_gemma/fa_gen_data.py:148-192): Q/K/V element codes
with E8M0 block scales, B/H/H_kv/S/d, q_pos0, causal, window, softcap,
softmax_scale.  torch is used for device memory and streams only; all math runs
in the library's CUDA kernels.
"""
import ctypes as C

import torch

from ._lib import DecodeArgs, PrefillArgs, check, lib

E4M3, E5M2, E2M3, E3M2, E2M1 = 0, 1, 2, 3, 4
V_SCALES_ALONG_KEYS, V_SCALES_ALONG_D = 0, 1
SCALES_ROWMAJOR, SCALES_GROUPMAJOR, SCALES_SF_ATOMS = 0, 1, 2


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _need_cuda(*ts):
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("expected contiguous CUDA tensors")


def _expect(t, name, dtype, shape):
    """A wrong dtype or shape must become a ValueError here: past this point the tensor is a raw pointer that TMA
    and bulk copies read with the sizes of the argument struct."""
    if t is None:
        return
    if t.dtype != dtype:
        raise ValueError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


def _scale_shape(lead, S, d, layout):
    if layout == SCALES_ROWMAJOR:
        return tuple(lead) + (S, d // 32)
    if layout == SCALES_GROUPMAJOR:
        return tuple(lead) + (d // 32, S)
    if layout == SCALES_SF_ATOMS:
        return _atoms_shape(lead, S, d)
    raise ValueError("scale layout must be SCALES_ROWMAJOR, SCALES_GROUPMAJOR or SCALES_SF_ATOMS")


def _check_prefill_tensors(q, k, v, q_scale, k_scale, v_scale, o, lse, v_scale_axis, q_scale_layout=SCALES_ROWMAJOR,
                           k_scale_layout=SCALES_ROWMAJOR, v_scale_layout=SCALES_ROWMAJOR):
    if q.dim() != 4 or k.dim() != 4:
        raise ValueError("q must be [B,H,S_q,d] and k/v [B,H_kv,S_kv,d]")
    B, H, S_q, d = q.shape
    H_kv, S_kv = k.shape[1], k.shape[2]
    if d % 32 != 0:
        raise ValueError("d must be a multiple of 32")
    _expect(q, "q", torch.uint8, (B, H, S_q, d))
    _expect(k, "k", torch.uint8, (B, H_kv, S_kv, d))
    _expect(v, "v", torch.uint8, (B, H_kv, S_kv, d))
    _expect(q_scale, "q_scale", torch.uint8, _scale_shape((B, H), S_q, d, q_scale_layout))
    _expect(k_scale, "k_scale", torch.uint8, _scale_shape((B, H_kv), S_kv, d, k_scale_layout))
    if v_scale_axis == V_SCALES_ALONG_D:
        if v_scale_layout != SCALES_ROWMAJOR:
            raise ValueError("V scales along d are row-major")
        _expect(v_scale, "v_scale", torch.uint8, (B, H_kv, S_kv, d // 32))
    elif v_scale_axis == V_SCALES_ALONG_KEYS:
        if v_scale_layout == SCALES_ROWMAJOR:
            _expect(v_scale, "v_scale", torch.uint8, (B, H_kv, (S_kv + 31) // 32, d))
        elif v_scale_layout == SCALES_SF_ATOMS:
            _expect(v_scale, "v_scale", torch.uint8, _atoms_shape((B, H_kv), S_kv, d))
        else:
            raise ValueError("V scales along the keys are row-major or scale-factor atoms")
    else:
        raise ValueError("v_scale_axis must be V_SCALES_ALONG_KEYS or V_SCALES_ALONG_D")
    _expect(o, "out", torch.bfloat16, (B, H, S_q, d))
    _expect(lse, "lse", torch.float32, (B, H, S_q))


def mx_quantize(x, fmt=E4M3):
    """fp32 or bf16 [..., cols] -> (codes uint8 [..., cols], scales uint8 [..., cols/32]); blocks along the last axis."""
    _need_cuda(x)
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("mx_quantize takes float32 or bfloat16")
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(x.shape[:-1] + (cols // 32,), dtype=torch.uint8, device=x.device)
    fn = lib().rk_mx_quantize if x.dtype == torch.float32 else lib().rk_mx_quantize_bf16
    check(fn(_ptr(x), rows, cols, fmt, _ptr(codes), _ptr(scales), _stream()), "rk_mx_quantize")
    return codes, scales


def _atoms_shape(lead, S, d):
    return tuple(lead) + ((S + 127) // 128, (d + 127) // 128, 512)


def mx_quantize_ex(x, fmt=E4M3, scale_layout=SCALES_ROWMAJOR):
    """fp32 or bf16 [..., S, d] -> (codes [..., S, d], scales in `scale_layout` per [S, d] matrix): row-major
    [..., S, d/32], group-major [..., d/32, S] or scale-factor atoms [..., ceil(S/128), ceil(d/128), 512]."""
    _need_cuda(x)
    if x.dtype not in (torch.float32, torch.bfloat16) or x.dim() < 2:
        raise ValueError("mx_quantize_ex takes float32 or bfloat16 [..., S, d]")
    S, d = x.shape[-2], x.shape[-1]
    batch = x.numel() // max(S * d, 1)
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    shape = {SCALES_ROWMAJOR: x.shape[:-1] + (d // 32,), SCALES_GROUPMAJOR: x.shape[:-2] + (d // 32, S),
             SCALES_SF_ATOMS: _atoms_shape(x.shape[:-2], S, d)}[scale_layout]
    scales = torch.empty(shape, dtype=torch.uint8, device=x.device)
    check(lib().rk_mx_quantize_ex(_ptr(x), int(x.dtype == torch.bfloat16), batch, S, d, fmt, _ptr(codes), _ptr(scales),
                                  scale_layout, _stream()), "rk_mx_quantize_ex")
    return codes, scales


def mx_quantize_keys_ex(x, fmt=E4M3, scale_layout=SCALES_ROWMAJOR):
    """fp32 [..., rows, cols], blocks down the rows -> codes and scales row-major [..., ceil(rows/32), cols] or
    scale-factor atoms [..., ceil(rows/128), ceil(cols/128), 512]."""
    _need_cuda(x)
    if x.dtype != torch.float32 or x.dim() < 2:
        raise ValueError("mx_quantize_keys_ex takes float32 [..., rows, cols]")
    rows, cols = x.shape[-2], x.shape[-1]
    batch = x.numel() // max(rows * cols, 1)
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    shape = x.shape[:-2] + ((rows + 31) // 32, cols) if scale_layout == SCALES_ROWMAJOR else _atoms_shape(x.shape[:-2], rows, cols)
    scales = torch.empty(shape, dtype=torch.uint8, device=x.device)
    check(lib().rk_mx_quantize_keys_ex(_ptr(x), batch, rows, cols, fmt, _ptr(codes), _ptr(scales), scale_layout, _stream()),
          "rk_mx_quantize_keys_ex")
    return codes, scales


def import_kt_blocks(kt_blocks, kt_scale_blocks, heads, n_blocks, Bk, d):
    """The reference's per-block K^T tiles [heads*n_blocks*d, Bk] and group-major scales [heads*n_blocks*d/32, Bk]
    -> natural K codes [heads, n_blocks*Bk, d] and row-major scales [heads, n_blocks*Bk, d/32]."""
    _need_cuda(kt_blocks, kt_scale_blocks)
    _expect(kt_blocks, "kt_blocks", torch.uint8, (heads * n_blocks * d, Bk))
    _expect(kt_scale_blocks, "kt_scale_blocks", torch.uint8, (heads * n_blocks * (d // 32), Bk))
    k = torch.empty((heads, n_blocks * Bk, d), dtype=torch.uint8, device=kt_blocks.device)
    ks = torch.empty((heads, n_blocks * Bk, d // 32), dtype=torch.uint8, device=kt_blocks.device)
    check(lib().rk_import_kt_blocks(_ptr(kt_blocks), _ptr(kt_scale_blocks), heads, n_blocks, Bk, d, _ptr(k), _ptr(ks), _stream()),
          "rk_import_kt_blocks")
    return k, ks


def rope_mx_quantize(x, cos_half, sin_half, *, pos=None, pos0=0, fmt=E4M3):
    """RoPE (rotate-half) then MX quantization along d.  x fp32 [..., S, d]; caches fp32 [n_pos, d/2]; rows use cache
    row pos0 + s, or pos[row] (int32 tensor with one entry per row) when given.  Returns (codes, scales)."""
    _need_cuda(x, cos_half, sin_half, pos)
    if x.dtype != torch.float32 or cos_half.dtype != torch.float32 or sin_half.dtype != torch.float32:
        raise ValueError("rope_mx_quantize takes float32")
    S, d = x.shape[-2], x.shape[-1]
    rows = x.numel() // max(d, 1)
    if cos_half.dim() != 2 or cos_half.shape[1] != d // 2 or sin_half.shape != cos_half.shape:
        raise ValueError("cos_half / sin_half must be [n_pos, d/2]")
    if pos is not None:
        _expect(pos, "pos", torch.int32, (rows,))
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(x.shape[:-1] + (d // 32,), dtype=torch.uint8, device=x.device)
    check(lib().rk_rope_mx_quantize(_ptr(x), rows, d, _ptr(pos), S, pos0, _ptr(cos_half), _ptr(sin_half),
                                    cos_half.shape[0], fmt, _ptr(codes), _ptr(scales), _stream()), "rk_rope_mx_quantize")
    return codes, scales


def rmsnorm_mx_quantize(x, gamma, eps, fmt=E4M3, unit_scale=False):
    """Row RMSNorm (the reference's fp32 order) then quantization along the last axis.  x fp32 or bf16 [..., K];
    gamma fp32 [K].  Returns (codes [..., K], scales [..., K/32]); unit_scale: E4M3 under 2^0, scales all 0x7F."""
    _need_cuda(x, gamma)
    if x.dtype not in (torch.float32, torch.bfloat16) or gamma.dtype != torch.float32:
        raise ValueError("rmsnorm_mx_quantize takes float32 or bfloat16 rows and a float32 gamma")
    K = x.shape[-1]
    _expect(gamma, "gamma", torch.float32, (K,))
    rows = x.numel() // max(K, 1)
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(x.shape[:-1] + (K // 32,), dtype=torch.uint8, device=x.device)
    check(lib().rk_rmsnorm_mx_quantize(_ptr(x), int(x.dtype == torch.bfloat16), rows, K, _ptr(gamma), float(eps), fmt,
                                       int(bool(unit_scale)), _ptr(codes), _ptr(scales), _stream()), "rk_rmsnorm_mx_quantize")
    return codes, scales


def mx_gemm_hw(a, b, a_scales, b_scales):
    """MX matmul in the mesh's accumulate semantics (bit-exact with the reference's mx_golden program).  a [M,K], b [K,N]
    E4M3 codes; a_scales [K/32,M], b_scales [K/32,N] E8M0 codes.  Returns C as bf16 [M,N]."""
    _need_cuda(a, b, a_scales, b_scales)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("a must be [M,K] and b [K,N]")
    M, K = a.shape
    N = b.shape[1]
    _expect(a, "a", torch.uint8, (M, K)); _expect(b, "b", torch.uint8, (K, N))
    _expect(a_scales, "a_scales", torch.uint8, (K // 32, M)); _expect(b_scales, "b_scales", torch.uint8, (K // 32, N))
    c = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    check(lib().rk_mx_gemm_hw(_ptr(a), _ptr(b), _ptr(a_scales), _ptr(b_scales), M, N, K, _ptr(c), _stream()), "rk_mx_gemm_hw")
    return c


def mx_quantize_keys(x, fmt=E4M3):
    """fp32 [..., rows, cols] -> codes same shape, scales [..., ceil(rows/32), cols]; blocks run down the rows."""
    _need_cuda(x)
    if x.dtype != torch.float32:
        raise ValueError("mx_quantize_keys takes float32")
    rows, cols = x.shape[-2], x.shape[-1]
    batch = x.numel() // max(rows * cols, 1)
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(x.shape[:-2] + ((rows + 31) // 32, cols), dtype=torch.uint8, device=x.device)
    check(lib().rk_mx_quantize_keys(_ptr(x), batch, rows, cols, fmt, _ptr(codes), _ptr(scales), _stream()),
          "rk_mx_quantize_keys")
    return codes, scales


def mx_rebase_v(codes, scales, fmt=E4M3):
    """[..., S, d] codes + [..., S, d/32] scales -> codes [..., S, d] + scales [..., ceil(S/32), d] (blocks along keys)."""
    _need_cuda(codes, scales)
    S, d = codes.shape[-2], codes.shape[-1]
    batch = codes.numel() // max(S * d, 1)
    oc = torch.empty_like(codes)
    osc = torch.empty(codes.shape[:-2] + ((S + 31) // 32, d), dtype=torch.uint8, device=codes.device)
    check(lib().rk_mx_rebase_v(_ptr(codes), _ptr(scales), batch, S, d, fmt, _ptr(oc), _ptr(osc), _stream()), "rk_mx_rebase_v")
    return oc, osc


def _prefill_args(q, k, v, q_scale, k_scale, v_scale, o, lse, causal, softmax_scale, q_pos0, window, softcap,
                  q_fmt, kv_fmt, v_scale_axis, q_scale_layout=SCALES_ROWMAJOR, k_scale_layout=SCALES_ROWMAJOR,
                  v_scale_layout=SCALES_ROWMAJOR):
    B, H, S_q, d = q.shape
    H_kv, S_kv = k.shape[1], k.shape[2]
    a = PrefillArgs()
    a.q, a.k, a.v = _ptr(q), _ptr(k), _ptr(v)
    a.q_scale, a.k_scale, a.v_scale = _ptr(q_scale), _ptr(k_scale), _ptr(v_scale)
    a.o, a.lse = _ptr(o), _ptr(lse)
    a.B, a.H, a.H_kv, a.S_q, a.S_kv, a.d = B, H, H_kv, S_q, S_kv, d
    a.q_pos0, a.causal, a.window = q_pos0, int(bool(causal)), window
    a.softcap, a.softmax_scale = float(softcap), float(softmax_scale)
    a.q_fmt, a.kv_fmt, a.v_scale_axis, a.block_n = q_fmt, kv_fmt, v_scale_axis, 0
    a.q_scale_layout, a.k_scale_layout, a.v_scale_layout = q_scale_layout, k_scale_layout, v_scale_layout
    return a


def attn_prefill_workspace_bytes(B, H, H_kv, S_q, S_kv, d, v_scale_axis=V_SCALES_ALONG_D, q_fmt=E4M3, kv_fmt=E4M3):
    a = PrefillArgs()
    a.B, a.H, a.H_kv, a.S_q, a.S_kv, a.d = B, H, H_kv, S_q, S_kv, d
    a.v_scale_axis, a.q_fmt, a.kv_fmt = v_scale_axis, q_fmt, kv_fmt
    return lib().rk_attn_prefill_workspace_bytes(C.byref(a))


def attn_prefill(q, k, v, q_scale, k_scale, v_scale, *, causal, softmax_scale=0.0, q_pos0=0, window=0, softcap=0.0,
                 q_fmt=E4M3, kv_fmt=E4M3, v_scale_axis=V_SCALES_ALONG_D, q_scale_layout=SCALES_ROWMAJOR,
                 k_scale_layout=SCALES_ROWMAJOR, v_scale_layout=SCALES_ROWMAJOR, out=None, lse=None, workspace=None):
    """MX flash-attention prefill.  q [B,H,S_q,d], k/v [B,H_kv,S_kv,d] uint8 codes; scales as the C header says.
    Returns O bf16 [B,H,S_q,d]."""
    _need_cuda(q, k, v, q_scale, k_scale, v_scale, out, lse, workspace)
    _check_prefill_tensors(q, k, v, q_scale, k_scale, v_scale, out, lse, v_scale_axis, q_scale_layout, k_scale_layout,
                           v_scale_layout)
    B, H, S_q, d = q.shape
    o = out if out is not None else torch.empty((B, H, S_q, d), dtype=torch.bfloat16, device=q.device)
    a = _prefill_args(q, k, v, q_scale, k_scale, v_scale, o, lse, causal, softmax_scale, q_pos0, window, softcap,
                      q_fmt, kv_fmt, v_scale_axis, q_scale_layout, k_scale_layout, v_scale_layout)
    need = lib().rk_attn_prefill_workspace_bytes(C.byref(a))
    if workspace is None:
        workspace = torch.empty(max(need, 1024), dtype=torch.uint8, device=q.device)
    elif workspace.dtype != torch.uint8:
        raise ValueError("workspace must be a uint8 tensor")
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    check(lib().rk_attn_prefill(C.byref(a), _stream()), "rk_attn_prefill")
    return o


def mx_pack_rows(codes, fmt):
    """6- or 4-bit codes one per byte [..., d] -> the dense rows form [..., dp * bits / 8] (dp = d rounded up to 128)."""
    _need_cuda(codes)
    if codes.dtype != torch.uint8 or codes.dim() < 2:
        raise ValueError("mx_pack_rows takes uint8 codes [..., d]")
    d = codes.shape[-1]
    rows = codes.numel() // max(d, 1)
    nbytes = lib().rk_mx_packed_rows_bytes(rows, d, fmt)
    if nbytes == 0 and rows > 0:
        raise ValueError("mx_pack_rows: format has no dense form (E2M3, E3M2, E2M1 only)")
    out = torch.empty(codes.shape[:-1] + (nbytes // max(rows, 1),), dtype=torch.uint8, device=codes.device)
    check(lib().rk_mx_pack_rows(_ptr(codes), rows, d, fmt, _ptr(out), _stream()), "rk_mx_pack_rows")
    return out


def mx_pack_vt(v_codes, fmt):
    """V codes blocked along the keys, one per byte [..., S, d] -> the dense transposed form [..., d, Sp * bits / 8]."""
    _need_cuda(v_codes)
    if v_codes.dtype != torch.uint8 or v_codes.dim() < 2:
        raise ValueError("mx_pack_vt takes uint8 codes [..., S, d]")
    S, d = v_codes.shape[-2], v_codes.shape[-1]
    batch = v_codes.numel() // max(S * d, 1)
    nbytes = lib().rk_mx_packed_vt_bytes(batch, S, d, fmt)
    if nbytes == 0 and batch > 0:
        raise ValueError("mx_pack_vt: format has no dense form (E2M3, E3M2, E2M1 only)")
    out = torch.empty(v_codes.shape[:-2] + (d, nbytes // max(batch * d, 1)), dtype=torch.uint8, device=v_codes.device)
    check(lib().rk_mx_pack_vt(_ptr(v_codes), batch, S, d, fmt, _ptr(out), _stream()), "rk_mx_pack_vt")
    return out


def attn_prefill_packed(q, k, vt, q_scale, k_scale, v_scale, *, S_q, S_kv, d, q_fmt, kv_fmt, causal, softmax_scale=0.0,
                        q_pos0=0, window=0, softcap=0.0, q_scale_layout=SCALES_ROWMAJOR, k_scale_layout=SCALES_ROWMAJOR,
                        v_scale_layout=SCALES_ROWMAJOR, out=None, lse=None, workspace=None):
    """Prefill over dense 6- / 4-bit operands: q [B,H,S_q,*] and k [B,H_kv,S_kv,*] from mx_pack_rows, vt
    [B,H_kv,d,*] from mx_pack_vt (V blocked along the keys, v_scale along the keys).  Returns O bf16 [B,H,S_q,d]."""
    _need_cuda(q, k, vt, q_scale, k_scale, v_scale, out, lse, workspace)
    if q.dim() != 4 or k.dim() != 4 or vt.dim() != 4:
        raise ValueError("q, k and vt are 4-d packed tensors")
    B, H = q.shape[0], q.shape[1]
    H_kv = k.shape[1]
    L = lib()
    _expect(q, "q", torch.uint8, (B, H, S_q, L.rk_mx_packed_rows_bytes(1, d, q_fmt)))
    _expect(k, "k", torch.uint8, (B, H_kv, S_kv, L.rk_mx_packed_rows_bytes(1, d, kv_fmt)))
    _expect(vt, "vt", torch.uint8, (B, H_kv, d, L.rk_mx_packed_vt_bytes(1, S_kv, 1, kv_fmt)))
    _expect(q_scale, "q_scale", torch.uint8, _scale_shape((B, H), S_q, d, q_scale_layout))
    _expect(k_scale, "k_scale", torch.uint8, _scale_shape((B, H_kv), S_kv, d, k_scale_layout))
    if v_scale_layout == SCALES_ROWMAJOR:
        _expect(v_scale, "v_scale", torch.uint8, (B, H_kv, (S_kv + 31) // 32, d))
    elif v_scale_layout == SCALES_SF_ATOMS:
        _expect(v_scale, "v_scale", torch.uint8, _atoms_shape((B, H_kv), S_kv, d))
    else:
        raise ValueError("V scales along the keys are row-major or scale-factor atoms")
    _expect(out, "out", torch.bfloat16, (B, H, S_q, d))
    _expect(lse, "lse", torch.float32, (B, H, S_q))
    o = out if out is not None else torch.empty((B, H, S_q, d), dtype=torch.bfloat16, device=q.device)
    a = PrefillArgs()
    a.q, a.k, a.v = _ptr(q), _ptr(k), _ptr(vt)
    a.q_scale, a.k_scale, a.v_scale = _ptr(q_scale), _ptr(k_scale), _ptr(v_scale)
    a.o, a.lse = _ptr(o), _ptr(lse)
    a.B, a.H, a.H_kv, a.S_q, a.S_kv, a.d = B, H, H_kv, S_q, S_kv, d
    a.q_pos0, a.causal, a.window = q_pos0, int(bool(causal)), window
    a.softcap, a.softmax_scale = float(softcap), float(softmax_scale)
    a.q_fmt, a.kv_fmt, a.v_scale_axis, a.block_n = q_fmt, kv_fmt, V_SCALES_ALONG_KEYS, 0
    a.q_scale_layout, a.k_scale_layout, a.v_scale_layout = q_scale_layout, k_scale_layout, v_scale_layout
    a.q_packed, a.kv_packed = 1, 1
    need = L.rk_attn_prefill_workspace_bytes(C.byref(a))
    if workspace is None:
        workspace = torch.empty(max(need, 1024), dtype=torch.uint8, device=q.device)
    elif workspace.dtype != torch.uint8:
        raise ValueError("workspace must be a uint8 tensor")
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    check(L.rk_attn_prefill(C.byref(a), _stream()), "rk_attn_prefill")
    return o


class PrefillHostRunner:
    """Prefill through the host-buffer entry point (rk_attn_prefill_host): inputs and output live in
    pinned host memory, the device arena is allocated once and reused."""

    def __init__(self, q, k, v, q_scale, k_scale, v_scale, *, causal, softmax_scale=0.0, q_pos0=0, window=0,
                 softcap=0.0, q_fmt=E4M3, kv_fmt=E4M3, v_scale_axis=V_SCALES_ALONG_D, want_lse=False, device="cuda"):
        for t in (q, k, v, q_scale, k_scale, v_scale):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("host runner takes contiguous CPU tensors (pinned for full copy speed)")
        _check_prefill_tensors(q, k, v, q_scale, k_scale, v_scale, None, None, v_scale_axis)
        self.keep = (q, k, v, q_scale, k_scale, v_scale)
        B, H, S_q, d = q.shape
        self.o = torch.empty((B, H, S_q, d), dtype=torch.bfloat16).pin_memory()
        self.lse = torch.empty((B, H, S_q), dtype=torch.float32).pin_memory() if want_lse else None
        self.args = _prefill_args(q, k, v, q_scale, k_scale, v_scale, self.o, self.lse, causal, softmax_scale, q_pos0,
                                  window, softcap, q_fmt, kv_fmt, v_scale_axis)
        need = lib().rk_attn_prefill_host_arena_bytes(C.byref(self.args))
        self.arena = torch.empty(need + 1024, dtype=torch.uint8, device=device)
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.keep)
        self.d2h_bytes = self.o.numel() * 2

    def run(self):
        check(lib().rk_attn_prefill_host(C.byref(self.args), _ptr(self.arena), self.arena.numel(), _stream()),
              "rk_attn_prefill_host")
        return self.o


def attn_prefill_host(q, k, v, q_scale, k_scale, v_scale, **kw):
    return PrefillHostRunner(q, k, v, q_scale, k_scale, v_scale, **kw).run()


def _decode_args(q, k, v, k_scale, v_scale, kv_len, o, lse, softmax_scale, kv_fmt, num_splits):
    B, H, d = q.shape
    H_kv, L = k.shape[1], k.shape[2]
    a = DecodeArgs()
    a.q, a.k, a.v, a.k_scale, a.v_scale = _ptr(q), _ptr(k), _ptr(v), _ptr(k_scale), _ptr(v_scale)
    a.kv_len, a.o, a.lse = _ptr(kv_len), _ptr(o), _ptr(lse)
    a.B, a.H, a.H_kv, a.L, a.d = B, H, H_kv, L, d
    a.softmax_scale, a.kv_fmt, a.num_splits = float(softmax_scale), kv_fmt, num_splits
    return a


def kv_cache_append(k_new, v_new, pos, k_codes, k_scales, v_codes, v_scales, fmt=E4M3):
    """Quantize one new K row and V row per (batch, KV head) (fp32 [B,H_kv,d]) into row pos[b] of the cache
    (codes [B,H_kv,L,d], scales [B,H_kv,L,d/32]); pos is an int32 CUDA tensor [B]."""
    _need_cuda(k_new, v_new, pos, k_codes, k_scales, v_codes, v_scales)
    if k_new.dtype != torch.float32 or v_new.dtype != torch.float32 or pos.dtype != torch.int32:
        raise ValueError("kv_cache_append takes float32 rows and int32 positions")
    if k_codes.dim() != 4:
        raise ValueError("k_codes must be [B,H_kv,L,d]")
    B, H_kv, L, d = k_codes.shape
    _expect(k_new, "k_new", torch.float32, (B, H_kv, d))
    _expect(v_new, "v_new", torch.float32, (B, H_kv, d))
    _expect(pos, "pos", torch.int32, (B,))
    _expect(k_codes, "k_codes", torch.uint8, (B, H_kv, L, d))
    _expect(v_codes, "v_codes", torch.uint8, (B, H_kv, L, d))
    _expect(k_scales, "k_scales", torch.uint8, (B, H_kv, L, d // 32))
    _expect(v_scales, "v_scales", torch.uint8, (B, H_kv, L, d // 32))
    check(lib().rk_kv_cache_append(_ptr(k_new), _ptr(v_new), B, H_kv, L, d, _ptr(pos), fmt, _ptr(k_codes), _ptr(k_scales),
                                   _ptr(v_codes), _ptr(v_scales), _stream()), "rk_kv_cache_append")


def attn_decode_num_splits(B, H, H_kv, L, d=128, num_splits=0):
    a = DecodeArgs()
    a.B, a.H, a.H_kv, a.L, a.d, a.num_splits = B, H, H_kv, L, d, num_splits
    return lib().rk_attn_decode_num_splits(C.byref(a))


def attn_decode_workspace_bytes(B, H, H_kv, L, d=128, num_splits=0):
    a = DecodeArgs()
    a.B, a.H, a.H_kv, a.L, a.d, a.num_splits = B, H, H_kv, L, d, num_splits
    return lib().rk_attn_decode_workspace_bytes(C.byref(a))


def _check_decode_tensors(q, k, v, k_scale, v_scale, kv_len, out, lse):
    if q.dim() != 3 or k.dim() != 4:
        raise ValueError("q must be [B,H,d] and k/v [B,H_kv,L,d]")
    B, H, d = q.shape
    H_kv, L = k.shape[1], k.shape[2]
    _expect(k, "k", torch.uint8, (B, H_kv, L, d))
    _expect(v, "v", torch.uint8, (B, H_kv, L, d))
    _expect(k_scale, "k_scale", torch.uint8, (B, H_kv, L, d // 32))
    _expect(v_scale, "v_scale", torch.uint8, (B, H_kv, L, d // 32))
    _expect(kv_len, "kv_len", torch.int32, (B,))
    _expect(out, "out", torch.bfloat16, (B, H, d))
    _expect(lse, "lse", torch.float32, (B, H))


def attn_decode(q, k, v, k_scale, v_scale, *, kv_len=None, softmax_scale=0.0, kv_fmt=E4M3, num_splits=0, out=None,
                lse=None, workspace=None):
    """Decode attention: q bf16 [B,H,d]; k/v codes [B,H_kv,L,d]; scales [B,H_kv,L,d/32]; kv_len int32 [B] or None.
    Returns O bf16 [B,H,d]."""
    _need_cuda(q, k, v, k_scale, v_scale, kv_len, out, lse, workspace)
    if q.dtype != torch.bfloat16:
        raise ValueError("decode query must be bfloat16")
    _check_decode_tensors(q, k, v, k_scale, v_scale, kv_len, out, lse)
    B, H, d = q.shape
    o = out if out is not None else torch.empty((B, H, d), dtype=torch.bfloat16, device=q.device)
    a = _decode_args(q, k, v, k_scale, v_scale, kv_len, o, lse, softmax_scale, kv_fmt, num_splits)
    need = lib().rk_attn_decode_workspace_bytes(C.byref(a))
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    a.workspace, a.workspace_bytes = _ptr(workspace), workspace.numel()
    check(lib().rk_attn_decode(C.byref(a), _stream()), "rk_attn_decode")
    return o


def last_device_status():
    return lib().rk_last_device_status()


def shard_range(n_units, rank, world):
    """Contiguous block partition of n_units independent (batch, KV-head) units over `world` ranks (rk_shard_units)."""
    lo, hi = C.c_int64(), C.c_int64()
    check(lib().rk_shard_units(n_units, rank, world, C.byref(lo), C.byref(hi)), "rk_shard_units")
    return lo.value, hi.value
