"""Failure detection without a GPU fault: a bounded device-side wait is made to run out (an mbarrier nobody ever
arrives at, limit one millisecond) and the library must report it, keep later launches from producing results
while the status word is set, and work again once the word has been read.  Plus the schedule-perturbation check
the reference uses to hunt missing barriers (a delay in one role must not change a bit of O:
kernels/flash_attention_mx_stable/README.md:27-35)."""
import ctypes as C

import pytest
import torch

import radiance_kernels_b200 as rk
from radiance_kernels_b200._lib import DecodeArgs
from helpers import quantize_inputs, randn_qkv

pytestmark = pytest.mark.gpu

WAIT_GAVE_UP = 901          # the code the test-hook kernel records


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_bounded_wait_runs_out_and_is_reported_and_clears():
    L = rk.lib()
    assert rk.last_device_status() == 0
    Q, K, V = randn_qkv(1, 2, 2, 256, 256, 128, seed=90)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V)
    good = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
    torch.cuda.synchronize()

    assert L.rk_debug_wait_runs_out(1000, 0, _stream()) == 0            # the kernel returns by itself
    torch.cuda.synchronize()
    try:
        # while the word is set, launches return at once and write nothing
        sentinel = torch.full_like(good, 7.0)
        out = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, out=sentinel.clone())
        torch.cuda.synchronize()
        assert torch.equal(out, sentinel)
        status = rk.last_device_status()
    except BaseException:
        rk.last_device_status()                                         # never leave the word set for the tests that follow
        raise
    assert status == WAIT_GAVE_UP                                       # reported once ...
    assert rk.last_device_status() == 0                                 # ... and cleared by the read
    again = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(again, good)
    assert rk.last_device_status() == 0


def test_noalloc_decode_status_word_is_observable():
    L = rk.lib()
    g = torch.Generator(device="cuda").manual_seed(91)
    q = torch.randn(1, 8, 128, generator=g, device="cuda").bfloat16()
    kc, ks = rk.mx_quantize(torch.randn(1, 2, 512, 128, generator=g, device="cuda"))
    vc, vs = rk.mx_quantize(torch.randn(1, 2, 512, 128, generator=g, device="cuda"))
    want = rk.attn_decode(q, kc, vc, ks, vs)

    def call():
        o = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda")
        a = DecodeArgs()
        a.q, a.k, a.v, a.k_scale, a.v_scale = (C.c_void_p(t.data_ptr()) for t in (q, kc, vc, ks, vs))
        a.o = C.c_void_p(o.data_ptr())
        a.B, a.H, a.H_kv, a.L, a.d = 1, 8, 2, 512, 128
        assert L.rk_attn_decode_noalloc(C.byref(a), _stream()) == 0
        torch.cuda.synchronize()
        return o

    assert L.rk_attn_decode_noalloc_status() == 0
    assert L.rk_debug_wait_runs_out(1000, 1, _stream()) == 0
    call()                                                              # runs on a set word: its result is not valid
    assert L.rk_attn_decode_noalloc_status() == WAIT_GAVE_UP
    assert rk.last_device_status() == 0                                 # the other word never saw it
    assert L.rk_attn_decode_noalloc_status() == 0
    got = call()
    assert (got.float() - want.float()).abs().max() < 2e-2


@pytest.mark.parametrize("shape", [(2, 4, 2, 1024, 128, False), (1, 2, 1, 640, 64, False), (1, 4, 4, 512, 128, True)])
def test_schedule_perturbation_leaves_every_bit_of_o(shape):
    """A few hundred nanoseconds of sleep at every key tile in one warp role at a time (softmax of query tile A,
    of tile B, correction, TMA producer, Q K^T issuer, P V issuer): if a hand-off between roles lacked a barrier the delayed
    role would read or overwrite something too early and O would change."""
    B, H, Hkv, S, d, cap = shape
    L = rk.lib()
    Q, K, V = randn_qkv(B, H, Hkv, S, S, d, seed=92)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V)
    kw = dict(causal=True, softcap=30.0 if cap else 0.0)
    base = rk.attn_prefill(qc, kc, vc, qs, ks, vs, **kw)
    try:
        for role in (1, 2, 3, 4, 5, 6):
            L.rk_debug_set_prefill_perturb(role)
            for _ in range(2):
                assert torch.equal(rk.attn_prefill(qc, kc, vc, qs, ks, vs, **kw), base), role
    finally:
        L.rk_debug_set_prefill_perturb(0)
    assert rk.last_device_status() == 0


def test_tensor_pipe_ceiling_loop_never_runs_into_its_waits():
    """The GEMM-only loop bench.py measures the tensor-pipe ceiling with paces itself through two alternating
    mbarriers (one barrier per batch in flight: a barrier that completes two phases before its waiter looks reads as
    "not yet", and a single pacing barrier did that about once in 10 000 launches).  A few thousand launches, short
    and long, must leave the device status word at zero."""
    import ctypes as C
    L = rk.lib()
    if not hasattr(L, "rk_debug_mxfp8_mma_loop"):
        pytest.skip("measurement aid not exported")
    L.rk_debug_mxfp8_mma_loop.restype = C.c_int
    L.rk_debug_mxfp8_mma_loop.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    tiles = torch.randint(0, 0x7E, (2, 128 * 128), dtype=torch.uint8, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for iters, n in ((64, 500), (200, 1500), (1024, 500), (8192, 100)):
        for _ in range(n):
            assert L.rk_debug_mxfp8_mma_loop(C.c_void_p(tiles[0].data_ptr()), C.c_void_p(tiles[1].data_ptr()), iters, st) == 0
        torch.cuda.synchronize()
        assert rk.last_device_status() == 0, iters
