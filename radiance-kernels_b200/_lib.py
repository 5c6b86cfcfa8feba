"""ctypes binding of librk_mx_attn.so (the same stub a foreign host would write)."""
import ctypes as C
import pathlib

_HERE = pathlib.Path(__file__).resolve().parent
_LIB = None


class RkError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        msg = lib().rk_error_string(code).decode()
        super().__init__(f"{where}: {msg} (code {code})")


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("o", C.c_void_p), ("lse", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("H_kv", C.c_int32), ("S_q", C.c_int32), ("S_kv", C.c_int32), ("d", C.c_int32),
        ("q_pos0", C.c_int32), ("causal", C.c_int32), ("window", C.c_int32),
        ("softcap", C.c_float), ("softmax_scale", C.c_float),
        ("q_fmt", C.c_int32), ("kv_fmt", C.c_int32), ("v_scale_axis", C.c_int32), ("block_n", C.c_int32),
        ("q_scale_layout", C.c_int32), ("k_scale_layout", C.c_int32), ("v_scale_layout", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_packed", C.c_int32), ("kv_packed", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("kv_len", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("H_kv", C.c_int32), ("L", C.c_int32), ("d", C.c_int32),
        ("softmax_scale", C.c_float), ("kv_fmt", C.c_int32), ("num_splits", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


# every symbol include/rk_mx_attn.h declares: (restype, argtypes)
SYMBOLS = {
    "rk_error_string": (C.c_char_p, [C.c_int]),
    "rk_version": (C.c_int, []),
    "rk_mx_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_mx_quantize_bf16": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_mx_quantize_keys": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_mx_quantize_ex": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "rk_mx_quantize_keys_ex": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "rk_import_kt_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_mx_rebase_v": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_mx_packed_rows_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int]),
    "rk_mx_pack_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "rk_mx_packed_vt_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int]),
    "rk_mx_pack_vt": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "rk_attn_prefill_block_n": (C.c_int, [C.POINTER(PrefillArgs)]),
    "rk_attn_prefill_workspace_bytes": (C.c_size_t, [C.POINTER(PrefillArgs)]),
    "rk_attn_prefill": (C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    "rk_attn_prefill_host_arena_bytes": (C.c_size_t, [C.POINTER(PrefillArgs)]),
    "rk_attn_prefill_host": (C.c_int, [C.POINTER(PrefillArgs), C.c_void_p, C.c_size_t, C.c_void_p]),
    "rk_attn_decode_num_splits": (C.c_int, [C.POINTER(DecodeArgs)]),
    "rk_attn_decode_workspace_bytes": (C.c_size_t, [C.POINTER(DecodeArgs)]),
    "rk_attn_decode": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "rk_attn_decode_noalloc": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "rk_attn_decode_noalloc_status": (C.c_int, []),
    "rk_rope_mx_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                      C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_rmsnorm_mx_quantize": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int32, C.c_void_p, C.c_float, C.c_int32, C.c_int32,
                                         C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_mx_gemm_hw": (C.c_int, [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_void_p, C.c_void_p]),
    "rk_kv_cache_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "rk_shard_units": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "rk_profile_set_events": (None, [C.c_void_p, C.c_void_p]),
    "rk_last_device_status": (C.c_int, []),
}


def build_library(force=False, verbose=False):
    import importlib.util
    spec = importlib.util.spec_from_file_location("_rk_build", _HERE / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(force=force, verbose=verbose)


def lib():
    """The loaded C-ABI library.  Raises if it was never built: there is no fallback."""
    global _LIB
    if _LIB is None:
        so = _HERE / "librk_mx_attn.so"
        if not so.exists():
            raise RuntimeError(f"{so} is missing: run `python radiance-kernels_b200/build.py` (needs nvcc)")
        L = C.CDLL(str(so))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)   # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        L.rk_debug_verify_encoder.restype = C.c_int
        L.rk_debug_verify_encoder.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.rk_debug_set_prefill_dump.restype = None
        L.rk_debug_set_prefill_dump.argtypes = [C.c_void_p]
        L.rk_debug_set_decode_path.restype = None
        L.rk_debug_set_decode_path.argtypes = [C.c_int]
        L.rk_debug_mxfp8_mma_loop.restype = C.c_int
        L.rk_debug_mxfp8_mma_loop.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.rk_debug_wait_runs_out.restype = C.c_int
        L.rk_debug_wait_runs_out.argtypes = [C.c_int, C.c_int, C.c_void_p]
        L.rk_debug_set_prefill_perturb.restype = None
        L.rk_debug_set_prefill_perturb.argtypes = [C.c_int]
        _LIB = L
    return _LIB


def check(code, where):
    if code != 0:
        raise RkError(code, where)
