"""CPU checks of the C-ABI library: it loads, exports every symbol the header declares, and rejects bad
arguments with the documented codes before touching the GPU.  No compute is launched here."""
import ctypes as C
import os
import re

import pytest

import radiance_kernels_b200 as rk
from radiance_kernels_b200._lib import SYMBOLS, DecodeArgs, PrefillArgs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "rk_mx_attn.h")).read()
    return sorted(set(re.findall(r"RK_API\s+[\w\s\*]+?\b(rk_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = rk.lib()
    names = header_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/rk_mx_attn.h but not exported"
    assert sorted(SYMBOLS) == names, "python binding table and header disagree"


def test_error_strings_and_version():
    L = rk.lib()
    assert L.rk_version() >= 100
    assert L.rk_error_string(0) == b"ok"
    for code in range(-9, 0):
        assert L.rk_error_string(code) not in (b"", b"unknown error")


def _pargs(**kw):
    a = PrefillArgs()
    a.B, a.H, a.H_kv, a.S_q, a.S_kv, a.d = 1, 4, 2, 128, 128, 128
    a.v_scale_axis = 1
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_prefill_argument_errors():
    L = rk.lib()
    assert L.rk_attn_prefill(None, None) == -1
    assert L.rk_attn_prefill(C.byref(_pargs(d=96)), None) == -2
    assert L.rk_attn_prefill(C.byref(_pargs(H=3)), None) == -2          # H % H_kv
    assert L.rk_attn_prefill(C.byref(_pargs(S_kv=0)), None) == -2
    assert L.rk_attn_prefill(C.byref(_pargs(v_scale_axis=7)), None) == -3
    assert L.rk_attn_prefill(C.byref(_pargs(q_fmt=9)), None) == -3
    assert L.rk_attn_prefill(C.byref(_pargs(block_n=64)), None) == -6
    assert L.rk_attn_prefill(C.byref(_pargs()), None) == -1               # valid shape, null tensors
    a = _pargs()
    for f in ("q", "k", "v", "q_scale", "k_scale", "v_scale", "o"):
        setattr(a, f, 4096)
    a.q = 4096 + 8
    assert L.rk_attn_prefill(C.byref(a), None) == -5                      # misaligned q
    a.q = 4096
    assert L.rk_attn_prefill(C.byref(a), None) == -4                      # no workspace
    assert L.rk_attn_prefill_block_n(C.byref(a)) == 128


def test_prefill_workspace_size():
    # q/k/v scale atoms (512 B per 128x128 tile chunk) + re-blocked V codes, each rounded to 1 KiB
    B, H, Hkv, S, d = 2, 4, 2, 300, 256
    nt, dch = 3, 2
    want = B * H * nt * dch * 512 + 2 * (B * Hkv * nt * dch * 512)
    want += (B * Hkv * S * d + 1023) // 1024 * 1024
    assert rk.attn_prefill_workspace_bytes(B, H, Hkv, S, S, d, rk.V_SCALES_ALONG_D) == want
    assert rk.attn_prefill_workspace_bytes(B, H, Hkv, S, S, d, rk.V_SCALES_ALONG_KEYS) == want - (B * Hkv * S * d + 1023) // 1024 * 1024
    assert rk.attn_prefill_workspace_bytes(B, H, Hkv, S, S, 96) == 0


def test_decode_argument_errors():
    L = rk.lib()
    a = DecodeArgs()
    a.B, a.H, a.H_kv, a.L, a.d = 2, 8, 2, 1024, 128
    assert L.rk_attn_decode(None, None) == -1
    assert L.rk_attn_decode(C.byref(a), None) == -1       # null tensors
    a.d = 64
    assert L.rk_attn_decode(C.byref(a), None) == -2
    a.d, a.H = 128, 6                                     # group of 3
    assert L.rk_attn_decode(C.byref(a), None) == -2
    a.H, a.L = 8, 1022
    assert L.rk_attn_decode(C.byref(a), None) == -2
    a.L, a.kv_fmt = 1024, 5                               # no such format
    assert L.rk_attn_decode(C.byref(a), None) == -3
    a.kv_fmt, a.num_splits = 0, 3
    assert L.rk_attn_decode_num_splits(C.byref(a)) == 3
    assert L.rk_attn_decode_workspace_bytes(C.byref(a)) == 2 * 8 * 3 * 130 * 4
    a.num_splits = 100
    assert L.rk_attn_decode(C.byref(a), None) == -2


def test_quantizer_argument_errors():
    L = rk.lib()
    assert L.rk_mx_quantize(None, 4, 32, 0, None, None, None) == -1
    assert L.rk_mx_quantize(4096, 4, 48, 0, 4096, 4096, None) == -2
    assert L.rk_mx_quantize(4096, 4, 64, 5, 4096, 4096, None) == -3
    assert L.rk_mx_quantize(4100, 4, 64, 0, 4096, 4096, None) == -5


def test_producer_and_cache_entry_points_reject_bad_arguments():
    L = rk.lib()
    ok = 4096                                              # an aligned, non-null stand-in pointer; nothing is launched
    # bf16 quantizer: same rules as the fp32 one
    assert L.rk_mx_quantize_bf16(None, 4, 32, 0, None, None, None) == -1
    assert L.rk_mx_quantize_bf16(ok, 4, 48, 0, ok, ok, None) == -2
    assert L.rk_mx_quantize_bf16(ok, 4, 64, 5, ok, ok, None) == -3
    assert L.rk_mx_quantize_bf16(ok + 2, 4, 64, 0, ok, ok, None) == -5
    # RoPE + quantizer: d must be a multiple of 64, positions inside the caches
    assert L.rk_rope_mx_quantize(None, 4, 128, None, 4, 0, ok, ok, 16, 0, ok, ok, None) == -1
    assert L.rk_rope_mx_quantize(ok, 4, 96, None, 4, 0, ok, ok, 16, 0, ok, ok, None) == -2
    assert L.rk_rope_mx_quantize(ok, 4, 128, None, 0, 0, ok, ok, 16, 0, ok, ok, None) == -2      # no pos list and no seq_len
    assert L.rk_rope_mx_quantize(ok, 4, 128, None, 12, 8, ok, ok, 16, 0, ok, ok, None) == -2     # pos0 + seq_len > n_pos
    assert L.rk_rope_mx_quantize(ok, 4, 128, None, 4, 0, ok, ok, 16, 7, ok, ok, None) == -3
    assert L.rk_rope_mx_quantize(ok + 4, 4, 128, None, 4, 0, ok, ok, 16, 0, ok, ok, None) == -5
    # KV-cache append
    assert L.rk_kv_cache_append(None, ok, 1, 1, 128, 128, ok, 0, ok, ok, ok, ok, None) == -1
    assert L.rk_kv_cache_append(ok, ok, 1, 1, 128, 100, ok, 0, ok, ok, ok, ok, None) == -2
    assert L.rk_kv_cache_append(ok, ok, 1, 1, 0, 128, ok, 0, ok, ok, ok, ok, None) == -2
    assert L.rk_kv_cache_append(ok, ok, 1, 1, 128, 128, ok, 5, ok, ok, ok, ok, None) == -3
    assert L.rk_kv_cache_append(ok + 4, ok, 1, 1, 128, 128, ok, 0, ok, ok, ok, ok, None) == -5


def test_dense_operand_entry_points_reject_bad_arguments():
    L = rk.lib()
    ok = 4096
    assert L.rk_mx_packed_rows_bytes(10, 128, 2) == 10 * 96 and L.rk_mx_packed_rows_bytes(10, 64, 4) == 10 * 64
    assert L.rk_mx_packed_rows_bytes(10, 128, 0) == 0                      # E4M3 has no dense form
    assert L.rk_mx_packed_vt_bytes(3, 333, 64, 3) == 3 * 64 * 384 * 6 // 8
    assert L.rk_mx_pack_rows(None, 4, 128, 2, ok, None) == -1
    assert L.rk_mx_pack_rows(ok, 4, 100, 2, ok, None) == -2
    assert L.rk_mx_pack_rows(ok, 4, 128, 1, ok, None) == -3
    assert L.rk_mx_pack_rows(ok + 4, 4, 128, 2, ok, None) == -5
    assert L.rk_mx_pack_vt(ok, 1, 0, 128, 4, ok, None) == -2
    assert L.rk_mx_pack_vt(ok, 1, 128, 128, 0, ok, None) == -3
    assert L.rk_attn_prefill(C.byref(_pargs(q_packed=1)), None) == -3               # E4M3 queries cannot be dense
    assert L.rk_attn_prefill(C.byref(_pargs(kv_fmt=3, kv_packed=1, v_scale_axis=1)), None) == -3   # dense V must be blocked along the keys
    # dense operands need no packing space in the workspace
    a, b = _pargs(q_fmt=2, kv_fmt=3, v_scale_axis=0), _pargs(q_fmt=2, kv_fmt=3, v_scale_axis=0, q_packed=1, kv_packed=1)
    assert L.rk_attn_prefill_workspace_bytes(C.byref(b)) < L.rk_attn_prefill_workspace_bytes(C.byref(a))
    for f in ("q", "k", "v", "q_scale", "k_scale", "v_scale", "o"):
        setattr(b, f, ok)
    assert L.rk_attn_prefill_host(C.byref(b), ok, 1 << 30, None) == -6              # the host entry point takes bytes only


def test_no_cpu_fallback():
    """The product path has no CPU route: calling it with CPU tensors raises instead of computing."""
    import torch
    x = torch.zeros(4, 64)
    with pytest.raises(ValueError):
        rk.mx_quantize(x)


def test_shard_range_covers_units_once():
    for n in (1, 7, 16, 512):
        for world in (1, 2, 3, 8):
            got = []
            for r in range(world):
                lo, hi = rk.shard_range(n, r, world)
                got += list(range(lo, hi))
            assert got == list(range(n))


def test_shard_units_argument_errors():
    L = rk.lib()
    lo, hi = C.c_int64(), C.c_int64()
    assert L.rk_shard_units(16, 0, 4, None, C.byref(hi)) == -1
    assert L.rk_shard_units(16, 4, 4, C.byref(lo), C.byref(hi)) == -2
    assert L.rk_shard_units(16, 0, 0, C.byref(lo), C.byref(hi)) == -2
    assert L.rk_shard_units(3, 3, 8, C.byref(lo), C.byref(hi)) == 0 and (lo.value, hi.value) == (3, 3)   # more ranks than units


def test_front_end_rejects_wrong_dtypes_and_shapes():
    """The Python front end checks dtype and exact shape of every tensor against B/H/H_kv/S/d before a pointer
    reaches the library (the checks run on CPU tensors here; nothing is launched)."""
    import torch
    from radiance_kernels_b200 import api
    B, H, Hkv, S, d = 1, 4, 2, 64, 128
    u8 = lambda *sh: torch.zeros(sh, dtype=torch.uint8)
    good = dict(q=u8(B, H, S, d), k=u8(B, Hkv, S, d), v=u8(B, Hkv, S, d), q_scale=u8(B, H, S, 4), k_scale=u8(B, Hkv, S, 4),
                v_scale=u8(B, Hkv, S, 4), o=torch.zeros(B, H, S, d, dtype=torch.bfloat16), lse=torch.zeros(B, H, S))
    api._check_prefill_tensors(**good, v_scale_axis=rk.V_SCALES_ALONG_D)
    bad_cases = [("k", u8(B, Hkv, S, 64)), ("q_scale", u8(B, H, S, 3)), ("v_scale", u8(B, Hkv, 2, d)),
                 ("q", torch.zeros(B, H, S, d, dtype=torch.int8)), ("o", torch.zeros(B, H, S, d)),
                 ("lse", torch.zeros(B, H, S + 1)), ("v", u8(B, H, S, d))]
    for name, t in bad_cases:
        with pytest.raises(ValueError):
            api._check_prefill_tensors(**{**good, name: t}, v_scale_axis=rk.V_SCALES_ALONG_D)
    with pytest.raises(ValueError):
        api._check_prefill_tensors(**good, v_scale_axis=rk.V_SCALES_ALONG_KEYS)     # v_scale has the other layout
    with pytest.raises(ValueError):
        api._check_prefill_tensors(**good, v_scale_axis=5)
    L = 256
    dq = torch.zeros(B, H, d, dtype=torch.bfloat16)
    dgood = dict(q=dq, k=u8(B, Hkv, L, d), v=u8(B, Hkv, L, d), k_scale=u8(B, Hkv, L, 4), v_scale=u8(B, Hkv, L, 4),
                 kv_len=torch.zeros(B, dtype=torch.int32), out=torch.zeros(B, H, d, dtype=torch.bfloat16), lse=torch.zeros(B, H))
    api._check_decode_tensors(**dgood)
    for name, t in [("v", u8(B, Hkv, L, 64)), ("k_scale", u8(B, Hkv, L, 8)), ("kv_len", torch.zeros(B, dtype=torch.int64)),
                    ("out", torch.zeros(B, H, d)), ("lse", torch.zeros(B, H, 2))]:
        with pytest.raises(ValueError):
            api._check_decode_tensors(**{**dgood, name: t})
