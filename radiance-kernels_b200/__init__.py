"""B200-native MX flash-attention path of radiance-kernels.

Host-side mirror of the C ABI in include/rk_mx_attn.h.  Every function here
launches the CUDA kernels of librk_mx_attn.so on torch CUDA tensors; there is
no CPU path and no fallback: a missing library or a missing GPU raises.
"""
from ._lib import lib, build_library, RkError, check  # noqa: F401
from .api import (  # noqa: F401
    E4M3, E5M2, E2M3, E3M2, E2M1, V_SCALES_ALONG_KEYS, V_SCALES_ALONG_D, SCALES_ROWMAJOR, SCALES_GROUPMAJOR, SCALES_SF_ATOMS,
    mx_quantize, mx_quantize_keys, mx_rebase_v, mx_quantize_ex, mx_quantize_keys_ex, import_kt_blocks,
    attn_prefill, attn_prefill_workspace_bytes, attn_prefill_host, PrefillHostRunner, mx_pack_rows, mx_pack_vt, attn_prefill_packed,
    attn_decode, attn_decode_workspace_bytes, attn_decode_num_splits, kv_cache_append, rope_mx_quantize, rmsnorm_mx_quantize, mx_gemm_hw,
    last_device_status, shard_range,
)
