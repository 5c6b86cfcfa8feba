"""Decode attention over an MXFP8 KV cache against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import MAX_ABS, REL_L2, errors, np_

pytestmark = pytest.mark.gpu


def run(B, H, Hkv, L, lens=None, seed=0, num_splits=0, want_lse=False, vmul=1.0, kv_fmt=rk.E4M3):
    d = 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, d, generator=g, device="cuda").bfloat16()
    K = torch.randn(B, Hkv, L, d, generator=g, device="cuda")
    V = torch.randn(B, Hkv, L, d, generator=g, device="cuda") * vmul
    kc, ks = rk.mx_quantize(K, kv_fmt)
    vc, vs = rk.mx_quantize(V, kv_fmt)
    kl = None if lens is None else torch.tensor(lens, dtype=torch.int32, device="cuda")
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda") if want_lse else None
    o = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl, num_splits=num_splits, lse=lse, kv_fmt=kv_fmt)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(kc), np_(vc), np_(ks), np_(vs), softmax_scale=d ** -0.5,
                             kv_len=None if lens is None else np.array(lens, np.int32), want_lse=want_lse, kv_fmt=kv_fmt)
    got = np_(o.float())
    assert np.isfinite(got).all()
    ma, rl = errors(got, ref["o_f32"])
    big = max(1.0, float(np.abs(ref["o_f32"]).max()))        # output magnitudes follow V's: the absolute bound with them
    assert ma <= MAX_ABS * big and rl <= REL_L2, (ma, rl)
    if want_lse:
        assert np.abs(np_(lse) - ref["lse"]).max() < 2e-3
    return got, ref


@pytest.mark.parametrize("grp", [1, 2, 4, 8])
def test_group_sizes(grp):
    run(2, 2 * grp, 2, 1024, seed=grp)


@pytest.mark.parametrize("grp", [1, 4, 8])
def test_e5m2_cache(grp):
    """An E5M2 cache (what rk_kv_cache_append writes with fmt = RK_FMT_E5M2): the tcgen05 kernel feeds the raw tiles
    to block-scaled MMAs, so the cache format is one field of the instruction descriptor."""
    run(2, 2 * grp, 2, 2048, seed=60 + grp, kv_fmt=rk.E5M2, want_lse=True)
    run(2, 2 * grp, 2, 1000, lens=[1000, 37], seed=70 + grp, kv_fmt=rk.E5M2)


@pytest.mark.parametrize("fmt", [rk.E2M3, rk.E3M2, rk.E2M1])
def test_six_and_four_bit_caches(fmt):
    """Caches in the 6-bit and 4-bit formats rk_kv_cache_append can write (one code per byte): the tensor core does
    not read that form, so these go through the kernel whose threads convert the codes (hardware conversions to f16 for
    K, bit placement into bf16 for V)."""
    run(2, 8, 2, 2048, seed=80 + fmt, kv_fmt=fmt, want_lse=True)
    run(2, 16, 2, 1000, lens=[1000, 37], seed=90 + fmt, kv_fmt=fmt)
    run(1, 2, 2, 512, seed=95 + fmt, kv_fmt=fmt, vmul=300.0)            # large V block scales


def test_e5m2_cache_through_the_converting_kernel():
    """The same E5M2 cache through the mma.sync kernel (test hook), which is templated on the cache format."""
    try:
        rk.lib().rk_debug_set_decode_path(1)
        run(2, 8, 2, 2048, seed=61, kv_fmt=rk.E5M2, want_lse=True)
    finally:
        rk.lib().rk_debug_set_decode_path(0)


def test_llama_shape_small_batch():
    """32 query heads on 8 KV heads, d=128 (the benchmark's head geometry) at a length the oracle finishes fast."""
    run(2, 32, 8, 4096, seed=1)


def test_ragged_kv_len_and_splits():
    run(3, 8, 2, 4096, lens=[4096, 1, 2500], seed=2)
    run(2, 8, 2, 1000, lens=[1000, 37], seed=3)
    run(1, 4, 1, 2048, num_splits=1, seed=4)
    run(1, 4, 1, 2048, num_splits=16, seed=4)       # more splits than needed: some are short or empty
    run(1, 4, 1, 132, lens=[129], num_splits=2, seed=5)


def test_empty_and_tiny_sequences():
    """kv_len 0 gives O = 0 and LSE = -inf (the l <= 0 guard); lengths below one key tile and one key short of it."""
    g = torch.Generator(device="cuda").manual_seed(12)
    q = torch.randn(4, 8, 128, generator=g, device="cuda").bfloat16()
    K = torch.randn(4, 2, 256, 128, generator=g, device="cuda")
    V = torch.randn(4, 2, 256, 128, generator=g, device="cuda")
    kc, ks = rk.mx_quantize(K); vc, vs = rk.mx_quantize(V)
    lens = [0, 5, 127, 129]
    kl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    lse = torch.empty(4, 8, dtype=torch.float32, device="cuda")
    o = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl, lse=lse)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(kc), np_(vc), np_(ks), np_(vs), softmax_scale=128 ** -0.5,
                             kv_len=np.array(lens, np.int32), want_lse=True)
    got = np_(o.float())
    assert np.all(got[0] == 0.0) and np.all(np.isneginf(np_(lse)[0]))
    ma, rl = errors(got, ref["o_f32"])
    assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)
    assert np.abs(np_(lse)[1:] - ref["lse"][1:]).max() < 2e-3


def test_split_count_does_not_change_result_much():
    a, _ = run(1, 8, 2, 8192, num_splits=1, seed=6)
    b, _ = run(1, 8, 2, 8192, num_splits=8, seed=6)
    assert np.abs(a - b).max() < 4e-3


def test_lse_output():
    run(1, 8, 2, 1024, want_lse=True, seed=7)


@pytest.mark.parametrize("top_code", [134, 135, 200, 60])
def test_v_scale_codes_at_and_beyond_the_bf16_folding_edge(top_code):
    """V block scales whose largest code is 134 (the last one a fixed 2^120 folding constant can take in bf16), 135,
    200 and a very small 60, mixed with codes up to 24 below it inside every block of 32 keys: both decode kernels
    must re-centre the factor they fold into P and match the oracle.  Output magnitudes follow the scale, so the
    absolute bound is relative to the reference's largest value."""
    g = torch.Generator(device="cuda").manual_seed(40 + top_code)
    q = torch.randn(2, 8, 128, generator=g, device="cuda").bfloat16()
    kc, ks, vc, vs = _quantized_cache(2, 2, 1024, seed=41 + top_code)
    vs = torch.randint(top_code - 24, top_code + 1, vs.shape, generator=g, dtype=torch.uint8, device="cuda")
    vs[:, :, 5::97] = top_code                      # the top code is present in every sequence
    (legacy, tc), ref = _check(q, kc, ks, vc, vs)
    big = float(np.abs(ref["o_f32"]).max())
    assert np.abs(legacy - tc).max() <= 1e-2 * max(1.0, big)      # one bf16 step of the output at that magnitude


def test_full_length_one_sequence():
    """KV length 32768 (the benchmark's per-sequence length) for one sequence, all 8 KV heads."""
    run(1, 32, 8, 32768, seed=9)


def _quantized_cache(B, Hkv, L, seed, kmul=1.0, vscale_spread=0):
    d = 128
    g = torch.Generator(device="cuda").manual_seed(seed)
    K = torch.randn(B, Hkv, L, d, generator=g, device="cuda") * kmul
    V = torch.randn(B, Hkv, L, d, generator=g, device="cuda")
    if vscale_spread:       # per-key magnitudes spread over 2^+-spread: block scales differ widely inside a 32-key block
        e = torch.randint(-vscale_spread, vscale_spread + 1, (B, Hkv, L, 1), generator=g, device="cuda").float()
        V = V * torch.exp2(e)
    kc, ks = rk.mx_quantize(K)
    vc, vs = rk.mx_quantize(V)
    return kc, ks, vc, vs


def _check(q, kc, ks, vc, vs, lens=None, num_splits=0):
    d = 128
    kl = None if lens is None else torch.tensor(lens, dtype=torch.int32, device="cuda")
    ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(kc), np_(vc), np_(ks), np_(vs), softmax_scale=d ** -0.5,
                             kv_len=None if lens is None else np.array(lens, np.int32))
    outs = []
    for path in (1, 0):                       # 1 = the mma.sync kernel, 0 = chosen by shape (tcgen05 for these shapes)
        rk.lib().rk_debug_set_decode_path(path)
        try:
            o = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl, num_splits=num_splits)
            torch.cuda.synchronize()
        finally:
            rk.lib().rk_debug_set_decode_path(0)
        assert rk.last_device_status() == 0
        got = np_(o.float())
        assert np.isfinite(got).all(), f"path {path}: non-finite output"
        ma, rl = errors(got, ref["o_f32"])
        # the absolute bound is stated for outputs of order one; scale it with the reference's magnitude
        assert ma <= MAX_ABS * max(1.0, float(np.abs(ref["o_f32"]).max())) and rl <= REL_L2, (path, ma, rl)
        outs.append(got)
    return outs, ref


def test_both_decode_kernels_match_the_oracle():
    g = torch.Generator(device="cuda").manual_seed(21)
    q = torch.randn(2, 8, 128, generator=g, device="cuda").bfloat16()
    kc, ks, vc, vs = _quantized_cache(2, 2, 2048, seed=22)
    (legacy, tc), ref = _check(q, kc, ks, vc, vs)
    assert np.abs(legacy - tc).max() < 4e-3


def test_tc_decode_peaked_rows_and_growing_maxima():
    """Large logits: a few keys dominate, the running maximum keeps growing along the sequence (keys scaled up
    towards the end), so O is rescaled several times and most p are far below the block maximum."""
    g = torch.Generator(device="cuda").manual_seed(23)
    q = (torch.randn(1, 4, 128, generator=g, device="cuda") * 4.0).bfloat16()
    kc, ks, vc, vs = _quantized_cache(1, 1, 4096, seed=24)
    K = torch.randn(1, 1, 4096, 128, generator=g, device="cuda") * torch.linspace(0.2, 3.0, 4096, device="cuda").view(1, 1, -1, 1)
    kc, ks = rk.mx_quantize(K)
    _check(q, kc, ks, vc, vs, num_splits=1)
    _check(q, kc, ks, vc, vs, num_splits=4)


def test_tc_decode_v_scales_spread_inside_a_block():
    g = torch.Generator(device="cuda").manual_seed(25)
    q = torch.randn(1, 8, 128, generator=g, device="cuda").bfloat16()
    kc, ks, vc, vs = _quantized_cache(1, 2, 1024, seed=26, vscale_spread=12)
    _check(q, kc, ks, vc, vs)


def test_decode_ignores_poisoned_cache_past_kv_len():
    """Keys at and beyond kv_len hold NaN codes and NaN scales (0x7F / 0xFF): they must not reach the result."""
    g = torch.Generator(device="cuda").manual_seed(27)
    q = torch.randn(2, 8, 128, generator=g, device="cuda").bfloat16()
    kc, ks, vc, vs = _quantized_cache(2, 2, 1024, seed=28)
    lens = [700, 130]
    clean = [t.clone() for t in (kc, ks, vc, vs)]
    for b, n in enumerate(lens):
        kc[b, :, n:] = 0x7F; vc[b, :, n:] = 0x7F; ks[b, :, n:] = 0xFF; vs[b, :, n:] = 0xFF
    kl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(clean[0]), np_(clean[2]), np_(clean[1]), np_(clean[3]),
                             softmax_scale=128 ** -0.5, kv_len=np.array(lens, np.int32))
    o = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    got = np_(o.float())
    assert np.isfinite(got).all()
    ma, rl = errors(got, ref["o_f32"])
    assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)


@pytest.mark.parametrize("fmt", [rk.E4M3, rk.E3M2, rk.E2M1])
def test_kv_cache_append_then_decode_in_a_loop(fmt):
    """Tokens appended one at a time give the cache that quantizing the whole tensor gives (bit for bit, and equal
    to the CPU oracle's rows); decode over the growing cache matches the oracle at every length tried.  Every format
    the append kernel writes is one the decode entry point reads."""
    B, Hkv, H, L, d, T = 2, 2, 8, 160, 128, 150
    g = torch.Generator(device="cuda").manual_seed(31)
    K = torch.randn(B, Hkv, L, d, generator=g, device="cuda")
    V = torch.randn(B, Hkv, L, d, generator=g, device="cuda") * 3.0
    q = torch.randn(B, H, d, generator=g, device="cuda").bfloat16()
    kc_all, ks_all = rk.mx_quantize(K, fmt)
    vc_all, vs_all = rk.mx_quantize(V, fmt)
    kc = torch.full((B, Hkv, L, d), 0x7F, dtype=torch.uint8, device="cuda")      # unwritten rows are poison
    vc = torch.full_like(kc, 0x7F)
    ks = torch.full((B, Hkv, L, d // 32), 0xFF, dtype=torch.uint8, device="cuda")
    vs = torch.full_like(ks, 0xFF)
    lens = [0, 0]
    for t in range(T):
        pos = torch.tensor([t, t if t < 100 else -1], dtype=torch.int32, device="cuda")   # sequence 1 stops at 100 tokens
        rk.kv_cache_append(K[:, :, t].contiguous(), V[:, :, t].contiguous(), pos, kc, ks, vc, vs, fmt=fmt)
        lens = [t + 1, min(t + 1, 100)]
        if t in (0, 31, 99, 127, 128, T - 1):
            kl = torch.tensor(lens, dtype=torch.int32, device="cuda")
            o = rk.attn_decode(q, kc, vc, ks, vs, kv_len=kl, kv_fmt=fmt)
            torch.cuda.synchronize()
            assert rk.last_device_status() == 0
            ref = oracle.attn_decode(np_(q.view(torch.uint16)), np_(kc_all), np_(vc_all), np_(ks_all), np_(vs_all),
                                     softmax_scale=d ** -0.5, kv_len=np.array(lens, np.int32), kv_fmt=fmt)
            got = np_(o.float())
            assert np.isfinite(got).all()
            ma, rl = errors(got, ref["o_f32"])
            assert ma <= MAX_ABS * 3.0 and rl <= REL_L2, (t, ma, rl)
    assert torch.equal(kc[0, :, :T], kc_all[0, :, :T]) and torch.equal(ks[0, :, :T], ks_all[0, :, :T])
    assert torch.equal(vc[0, :, :T], vc_all[0, :, :T]) and torch.equal(vs[0, :, :T], vs_all[0, :, :T])
    assert torch.equal(kc[1, :, :100], kc_all[1, :, :100]) and bool((kc[1, :, 100:] == 0x7F).all())
    oc, os_ = oracle.quantize(np_(V[0, 0, :T]), axis=1, fmt=fmt)
    assert np.array_equal(np_(vc[0, 0, :T]), oc) and np.array_equal(np_(vs[0, 0, :T]), os_)
