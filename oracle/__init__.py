"""ctypes bindings of the CPU oracle (oracle/rk_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped library never imports this package.
"""
import ctypes as C
import os
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB = None

E4M3, E5M2, E2M3, E3M2, E2M1 = 0, 1, 2, 3, 4


def reference_dir():
    """Where the reference's source tree lies: $RK_REFERENCE_DIR, else a directory named `reference` beside this
    repository's checkout.  It need not exist (the prebuilt oracle/_ref files are used then)."""
    return os.environ.get("RK_REFERENCE_DIR") or str(_HERE.parent.parent / "reference")


def build(force=False):
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    so = _HERE / "liboracle.so"
    src = _HERE / "rk_oracle.cpp"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True, stdout=subprocess.DEVNULL)
    ref = reference_dir()
    if os.path.isdir(ref) and (force or not (_HERE / "_ref" / "libref_codec.so").exists()):
        subprocess.run(["make", "-C", str(_HERE), "ref", "REF=" + ref], check=True, stdout=subprocess.DEVNULL)


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32), ("d", C.c_int32),
        ("q_pos0", C.c_int32), ("causal", C.c_int32), ("window", C.c_int32),
        ("softcap", C.c_float), ("softmax_scale", C.c_float),
        ("q_fmt", C.c_int32), ("kv_fmt", C.c_int32), ("v_scale_axis", C.c_int32), ("block_n", C.c_int32),
        ("nthreads", C.c_int32),
        ("slice_begin", C.c_int64), ("slice_end", C.c_int64),
        ("o_f32", C.c_void_p), ("o_bf16", C.c_void_p), ("lse", C.c_void_p),
        ("dump_slice", C.c_int64),
        ("dump_s", C.c_void_p), ("dump_p_codes", C.c_void_p), ("dump_p_scales", C.c_void_p),
        ("dump_m", C.c_void_p), ("dump_l", C.c_void_p),
        ("bf16_faithful", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("kv_len", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("Hkv", C.c_int32), ("L", C.c_int32), ("d", C.c_int32),
        ("softmax_scale", C.c_float), ("kv_fmt", C.c_int32), ("nthreads", C.c_int32),
        ("unit_begin", C.c_int64), ("unit_end", C.c_int64),
        ("o_f32", C.c_void_p), ("o_bf16", C.c_void_p), ("lse", C.c_void_p),
    ]


def lib():
    global _LIB
    if _LIB is None:
        build()
        L = C.CDLL(str(_HERE / "liboracle.so"))
        L.rko_decode_elem.restype = C.c_float
        L.rko_decode_elem.argtypes = [C.c_uint8, C.c_int]
        L.rko_encode_elem_rne.restype = C.c_uint8
        L.rko_encode_elem_rne.argtypes = [C.c_float, C.c_int]
        L.rko_e8m0_decode.restype = C.c_float
        L.rko_e8m0_decode.argtypes = [C.c_uint8]
        L.rko_f32_to_bf16.restype = C.c_uint16
        L.rko_f32_to_bf16.argtypes = [C.c_float]
        L.rko_p_block_scale_code.restype = C.c_uint8
        L.rko_p_block_scale_code.argtypes = [C.c_float]
        L.rko_p_code.restype = C.c_uint8
        L.rko_p_code.argtypes = [C.c_float, C.c_uint8]
        for n in ("rko_quantize_rows", "rko_quantize_cols"):
            getattr(L, n).restype = None
            getattr(L, n).argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        for n in ("rko_dequant_rows", "rko_dequant_cols"):
            getattr(L, n).restype = None
            getattr(L, n).argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
        L.rko_quantize_rows_mxgolden.restype = None
        L.rko_quantize_rows_mxgolden.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        L.rko_rope_rows.restype = None
        L.rko_rope_rows.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.rko_mx_gemm_hw.restype = None
        L.rko_mx_gemm_hw.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p, C.c_int]
        L.rko_rmsnorm_rows.restype = None
        L.rko_rmsnorm_rows.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_float, C.c_void_p]
        L.rko_rebase_v.restype = None
        L.rko_rebase_v.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
        L.rko_attn_prefill.restype = C.c_int
        L.rko_attn_prefill.argtypes = [C.POINTER(PrefillArgs)]
        L.rko_attn_decode.restype = C.c_int
        L.rko_attn_decode.argtypes = [C.POINTER(DecodeArgs)]
        L.rko_attn_fp32_ref.restype = None
        L.rko_attn_fp32_ref.argtypes = [C.c_void_p] * 3 + [C.c_int] * 9 + [C.c_float, C.c_float, C.c_void_p, C.c_int]
        L.rko_hardware_threads.restype = C.c_int
        _LIB = L
    return _LIB


def ref_codec():
    """The reference's own codec header behind a C shim, or None when oracle/_ref was never built."""
    so = _HERE / "_ref" / "libref_codec.so"
    if not so.exists():
        return None
    R = C.CDLL(str(so))
    R.ref_fp8_e4m3_decode.restype = C.c_float
    R.ref_fp8_e4m3_decode.argtypes = [C.c_uint8]
    R.ref_fp8_e4m3_to_code.restype = C.c_uint8
    R.ref_fp8_e4m3_to_code.argtypes = [C.c_float]
    R.ref_fpe8m0_decode.restype = C.c_float
    R.ref_fpe8m0_decode.argtypes = [C.c_uint8]
    R.ref_fp6_e3m2_decode.restype = C.c_float
    R.ref_fp6_e3m2_decode.argtypes = [C.c_uint8]
    R.ref_f32_to_bf16_rne.restype = C.c_uint16
    R.ref_f32_to_bf16_rne.argtypes = [C.c_float]
    if hasattr(R, "ref_fp4_e2m1_decode"):            # shims built before the FP4 format was added lack these two
        R.ref_fp4_e2m1_decode.restype = C.c_float
        R.ref_fp4_e2m1_decode.argtypes = [C.c_uint8]
        R.ref_bf16_bits_to_fp4_e2m1_code.restype = C.c_uint8
        R.ref_bf16_bits_to_fp4_e2m1_code.argtypes = [C.c_uint16]
    return R


def ref_requant():
    """The reference attention kernel's own P-requantization helpers behind a C shim (oracle/_ref/libref_requant.so),
    or None when oracle/_ref was never built."""
    so = _HERE / "_ref" / "libref_requant.so"
    if not so.exists():
        return None
    R = C.CDLL(str(so))
    R.ref_bf16_to_e4m3_scaled.restype = C.c_uint8
    R.ref_bf16_to_e4m3_scaled.argtypes = [C.c_uint16, C.c_int]
    R.ref_bf16_floor_log2.restype = C.c_int
    R.ref_bf16_floor_log2.argtypes = [C.c_uint16]
    for n in ("ref_bf16_to_e4m3_trunc", "ref_bf16_to_e4m3_rne"):
        getattr(R, n).restype = C.c_uint8
        getattr(R, n).argtypes = [C.c_uint16]
    return R


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def hardware_threads():
    return lib().rko_hardware_threads()


def quantize_mxgolden(x):
    """The reference's other rule (requant post-pass of lib/golden/mx_golden.cpp) on fp32 rows [rows, cols], cols a
    multiple of 32: scale = floor(log2 amax) - 8, elements RNE with subnormals flushed.  Oracle mode only."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    codes = np.empty((rows, cols), np.uint8)
    scales = np.empty((rows, cols // 32), np.uint8)
    lib().rko_quantize_rows_mxgolden(_p(x), rows, cols, _p(codes), _p(scales))
    return codes, scales


def ref_mx_golden_path():
    """Path of the reference's mx_golden program built under oracle/_ref, or None."""
    exe = _HERE / "_ref" / "mx_golden"
    return str(exe) if exe.exists() else None


def rope(x, pos, cos_half, sin_half):
    """RoPE (rotate-half) of fp32 rows [rows, d]; row r uses cache row pos[r] of cos_half / sin_half [n_pos, d/2]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    c = np.ascontiguousarray(cos_half, dtype=np.float32)
    s = np.ascontiguousarray(sin_half, dtype=np.float32)
    rows, d = x.shape
    out = np.empty_like(x)
    lib().rko_rope_rows(_p(x), rows, d, _p(pos), _p(c), _p(s), _p(out))
    return out


def mx_gemm_hw(A, B, SA, SB, nthreads=0):
    """MX matmul in the mesh's accumulate semantics (lib/golden/mx_golden.cpp:114-144).  A [M,K], B [K,N] E4M3 codes,
    SA [K/32,M], SB [K/32,N] E8M0 codes -> C bf16 bits uint16 [M,N]."""
    A, B, SA, SB = [np.ascontiguousarray(t, np.uint8) for t in (A, B, SA, SB)]
    M, K = A.shape
    N = B.shape[1]
    Cc = np.empty((M, N), np.uint16)
    lib().rko_mx_gemm_hw(_p(A), _p(B), _p(SA), _p(SB), M, N, K, _p(Cc), nthreads or hardware_threads())
    return Cc


def rmsnorm(x, gamma, eps):
    """Row RMSNorm of fp32 [rows, K] in the reference's scalar fp32 order (lib/golden/golden.py:203-216)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    gamma = np.ascontiguousarray(gamma, dtype=np.float32)
    rows, K = x.shape
    out = np.empty_like(x)
    lib().rko_rmsnorm_rows(_p(x), rows, K, _p(gamma), float(np.float32(eps)), _p(out))
    return out


def quantize(x, fmt=E4M3, axis=-1, nthreads=1):
    """MX block-32 quantization of a 2-D fp32 array under the lib/golden rule.

    axis=-1: blocks along the last axis, scales [rows, ceil(cols/32)];
    axis=0 : blocks along the first axis, scales [ceil(rows/32), cols]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    codes = np.empty((rows, cols), np.uint8)
    if axis in (-1, 1):
        scales = np.empty((rows, (cols + 31) // 32), np.uint8)
        lib().rko_quantize_rows(_p(x), rows, cols, fmt, _p(codes), _p(scales), nthreads)
    else:
        scales = np.empty(((rows + 31) // 32, cols), np.uint8)
        lib().rko_quantize_cols(_p(x), rows, cols, fmt, _p(codes), _p(scales), nthreads)
    return codes, scales


def dequant(codes, scales, fmt=E4M3, axis=-1):
    codes = np.ascontiguousarray(codes, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint8)
    rows, cols = codes.shape
    out = np.empty((rows, cols), np.float32)
    fn = lib().rko_dequant_rows if axis in (-1, 1) else lib().rko_dequant_cols
    fn(_p(codes), _p(scales), rows, cols, fmt, _p(out))
    return out


def rebase_v(codes, scales, fmt=E4M3):
    """[S,d] codes + [S,d/32] scales -> [S,d] codes + [ceil(S/32),d] scales (blocks along keys)."""
    codes = np.ascontiguousarray(codes, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint8)
    S, d = codes.shape
    oc = np.empty((S, d), np.uint8)
    osc = np.empty(((S + 31) // 32, d), np.uint8)
    lib().rko_rebase_v(_p(codes), _p(scales), S, d, fmt, _p(oc), _p(osc))
    return oc, osc


def attn_prefill(q, k, v, qs, ks, vs, *, causal, softmax_scale, q_pos0=0, window=0, softcap=0.0,
                 q_fmt=E4M3, kv_fmt=E4M3, v_scale_axis=1, block_n=128, nthreads=0, slices=None,
                 dump_slice=-1, want_lse=False, bf16_faithful=False):
    """MX prefill attention oracle. q [B,H,Sq,d] codes, k/v [B,Hkv,Skv,d] codes, scales as the C ABI takes them.

    bf16_faithful: re-round every intermediate to bf16 where the reference's Python model does (its numerics, not
    the build target's fp32 softmax).  Returns dict(o_f32, o_bf16, lse?, dumps?)."""
    q, k, v, qs, ks, vs = [np.ascontiguousarray(t, np.uint8) for t in (q, k, v, qs, ks, vs)]
    B, H, Sq, d = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    a = PrefillArgs()
    o32 = np.zeros((B, H, Sq, d), np.float32)
    o16 = np.zeros((B, H, Sq, d), np.uint16)
    lse = np.zeros((B, H, Sq), np.float32) if want_lse else None
    a.q, a.k, a.v, a.q_scale, a.k_scale, a.v_scale = _p(q), _p(k), _p(v), _p(qs), _p(ks), _p(vs)
    a.B, a.H, a.Hkv, a.Sq, a.Skv, a.d = B, H, Hkv, Sq, Skv, d
    a.q_pos0, a.causal, a.window = q_pos0, int(causal), window
    a.softcap, a.softmax_scale = softcap, softmax_scale
    a.q_fmt, a.kv_fmt, a.v_scale_axis, a.block_n = q_fmt, kv_fmt, v_scale_axis, block_n
    a.nthreads = nthreads or hardware_threads()
    a.slice_begin, a.slice_end = (slices if slices else (0, 0))
    a.o_f32, a.o_bf16, a.lse = _p(o32), _p(o16), _p(lse)
    a.bf16_faithful = int(bool(bf16_faithful))
    out = {"o_f32": o32, "o_bf16": o16}
    a.dump_slice = dump_slice
    if dump_slice >= 0:
        out["s"] = np.zeros((Sq, Skv), np.float32)
        out["p_codes"] = np.zeros((Sq, Skv), np.uint8)
        out["p_scales"] = np.zeros((Sq, (Skv + 31) // 32), np.uint8)
        out["m"] = np.zeros(Sq, np.float32)
        out["l"] = np.zeros(Sq, np.float32)
        a.dump_s, a.dump_p_codes, a.dump_p_scales = _p(out["s"]), _p(out["p_codes"]), _p(out["p_scales"])
        a.dump_m, a.dump_l = _p(out["m"]), _p(out["l"])
    rc = lib().rko_attn_prefill(C.byref(a))
    if rc != 0:
        raise ValueError("oracle prefill: bad arguments")
    if want_lse:
        out["lse"] = lse
    return out


def attn_decode(q_bf16, k, v, ks, vs, *, softmax_scale, kv_len=None, kv_fmt=E4M3, nthreads=0, units=None,
                want_lse=False):
    """Decode attention oracle. q_bf16 uint16 [B,H,d]; k/v codes [B,Hkv,L,d]; scales [B,Hkv,L,d/32]."""
    q_bf16 = np.ascontiguousarray(q_bf16, np.uint16)
    k, v, ks, vs = [np.ascontiguousarray(t, np.uint8) for t in (k, v, ks, vs)]
    B, H, d = q_bf16.shape
    Hkv, L = k.shape[1], k.shape[2]
    a = DecodeArgs()
    o32 = np.zeros((B, H, d), np.float32)
    o16 = np.zeros((B, H, d), np.uint16)
    lse = np.zeros((B, H), np.float32) if want_lse else None
    kl = None if kv_len is None else np.ascontiguousarray(kv_len, np.int32)
    a.q, a.k, a.v, a.k_scale, a.v_scale, a.kv_len = _p(q_bf16), _p(k), _p(v), _p(ks), _p(vs), _p(kl)
    a.B, a.H, a.Hkv, a.L, a.d = B, H, Hkv, L, d
    a.softmax_scale, a.kv_fmt = softmax_scale, kv_fmt
    a.nthreads = nthreads or hardware_threads()
    a.unit_begin, a.unit_end = (units if units else (0, 0))
    a.o_f32, a.o_bf16, a.lse = _p(o32), _p(o16), _p(lse)
    if lib().rko_attn_decode(C.byref(a)) != 0:
        raise ValueError("oracle decode: bad arguments")
    out = {"o_f32": o32, "o_bf16": o16}
    if want_lse:
        out["lse"] = lse
    return out


def attn_fp32_ref(Q, K, V, *, causal, softmax_scale, q_pos0=0, window=0, softcap=0.0, nthreads=0):
    Q, K, V = [np.ascontiguousarray(t, np.float32) for t in (Q, K, V)]
    B, H, Sq, d = Q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    O = np.zeros((B, H, Sq, d), np.float32)
    lib().rko_attn_fp32_ref(_p(Q), _p(K), _p(V), B, H, Hkv, Sq, Skv, d, q_pos0, int(causal), window,
                            softcap, softmax_scale, _p(O), nthreads or hardware_threads())
    return O
