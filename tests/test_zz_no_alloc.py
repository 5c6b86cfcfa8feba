"""The allocation-free decode entry point (rk_attn_decode_noalloc), for hosts that may not allocate device
memory where they call the library (a plugin inside a memory pool it does not own, a serving loop whose
allocator is locked during a step).  It must give what rk_attn_decode gives, call after call, although its
split partials live in one fixed array inside the library image that every call reuses.

Collected last on purpose (file name): if it fails under `-x`, every other test has already run."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from radiance_kernels_b200._lib import DecodeArgs
from helpers import MAX_ABS, REL_L2, errors, np_

pytestmark = pytest.mark.gpu


def _case(B, H, Hkv, L, seed, lens=None):
    d = 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, d, generator=g, device="cuda").bfloat16()
    kc, ks = rk.mx_quantize(torch.randn(B, Hkv, L, d, generator=g, device="cuda"))
    vc, vs = rk.mx_quantize(torch.randn(B, Hkv, L, d, generator=g, device="cuda"))
    kl = None if lens is None else torch.tensor(lens, dtype=torch.int32, device="cuda")
    return q, kc, vc, ks, vs, kl


def _noalloc(q, kc, vc, ks, vs, kl, num_splits=0):
    B, H, d = q.shape
    o = torch.empty(B, H, d, dtype=torch.bfloat16, device="cuda")      # the caller still owns inputs and outputs
    a = DecodeArgs()
    a.q, a.k, a.v, a.k_scale, a.v_scale = (C.c_void_p(t.data_ptr()) for t in (q, kc, vc, ks, vs))
    a.kv_len = None if kl is None else C.c_void_p(kl.data_ptr())
    a.o = C.c_void_p(o.data_ptr())
    a.B, a.H, a.H_kv, a.L, a.d = B, H, kc.shape[1], kc.shape[2], d
    a.num_splits = num_splits
    rc = rk.lib().rk_attn_decode_noalloc(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, o


def test_noalloc_decode_matches_workspace_decode_twice_in_a_row():
    # two different problems back to back: the second call must not be disturbed by what the first left behind
    for args in (dict(B=2, H=8, Hkv=2, L=2048, seed=21), dict(B=3, H=16, Hkv=4, L=1000, seed=22, lens=[1000, 3, 517])):
        q, kc, vc, ks, vs, kl = _case(**args)
        want = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl)
        ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(kc), np_(vc), np_(ks), np_(vs), softmax_scale=128 ** -0.5,
                                 kv_len=None if kl is None else np_(kl))
        for _ in range(2):
            rc, got = _noalloc(q, kc, vc, ks, vs, kl)
            assert rc == 0
            torch.cuda.synchronize()
            ma, rl = errors(np_(got.float()), np_(want.float()))
            assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)
            ma, rl = errors(np_(got.float()), ref["o_f32"])          # and against the CPU oracle itself
            assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)
            assert rk.lib().rk_attn_decode_noalloc_status() == 0     # this path's own status word
    assert rk.last_device_status() == 0


def test_noalloc_decode_rejects_what_does_not_fit():
    q, kc, vc, ks, vs, kl = _case(1, 8, 1, 256, seed=23)
    # pretend a huge batch: B * H * splits * 130 floats beyond the 5 MiB array -> RK_ERR_TOO_LARGE, nothing launched
    a = DecodeArgs()
    a.q, a.k, a.v, a.k_scale, a.v_scale = (C.c_void_p(t.data_ptr()) for t in (q, kc, vc, ks, vs))
    a.o = C.c_void_p(q.data_ptr())
    a.B, a.H, a.H_kv, a.L, a.d = 4096, 32, 8, 256, 128
    a.num_splits = 2
    assert rk.lib().rk_attn_decode_noalloc(C.byref(a), None) == -9
    a.num_splits = 0
    assert rk.lib().rk_attn_decode_noalloc(C.byref(a), None) == -9
