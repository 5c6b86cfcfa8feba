"""Parity at the full shapes the benchmark configurations name: the whole tensor runs on the GPU through the C ABI,
a few (batch, head) slices -- first, last and one from the middle of the work order -- are checked against the CPU
oracle (same block_n, same P rule), and every element is checked through size-independent properties: finite, and
inside the convex hull of the V rows (|O| <= max |V|)."""
import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import MAX_ABS, REL_L2, errors, np_, randn_qkv

pytestmark = pytest.mark.gpu


def _check_head_slices(qc, qs, kc, ks, vc, vs, o, slices, *, softcap=0.0, q_fmt=rk.E4M3, kv_fmt=rk.E4M3):
    """slices: (b, h) pairs.  Each is copied out with its own KV head, so that one oracle call runs them on
    separate threads."""
    B, H, S, d = qc.shape
    grp = H // kc.shape[1]
    pick = lambda t, idx: np.stack([np_(t[b, h]) for b, h in idx])[None]
    kv = [(b, h // grp) for b, h in slices]
    ref = oracle.attn_prefill(pick(qc, slices), pick(kc, kv), pick(vc, kv), pick(qs, slices), pick(ks, kv), pick(vs, kv),
                              causal=True, softmax_scale=d ** -0.5, softcap=softcap, q_fmt=q_fmt, kv_fmt=kv_fmt,
                              block_n=128)
    for i, (b, h) in enumerate(slices):
        ma, rl = errors(np_(o[b, h].float()), ref["o_f32"][0, i])
        assert ma <= MAX_ABS and rl <= REL_L2, ((b, h), ma, rl)


def _run_prefill(B, H, Hkv, S, d, *, seed, mul=1.0, softcap=0.0, q_fmt=rk.E4M3, kv_fmt=rk.E4M3, slices):
    Q, K, V = randn_qkv(B, H, Hkv, S, S, d, seed=seed, mul=mul)
    qc, qs = rk.mx_quantize(Q, q_fmt)
    kc, ks = rk.mx_quantize(K, kv_fmt)
    vc, vs = rk.mx_quantize(V, kv_fmt)
    vmax = float(V.abs().max())
    del Q, K, V
    o = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, softcap=softcap, q_fmt=q_fmt, kv_fmt=kv_fmt)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    assert torch.isfinite(o.float()).all()
    assert float(o.float().abs().max()) <= vmax * 1.01
    _check_head_slices(qc, qs, kc, ks, vc, vs, o, slices, softcap=softcap, q_fmt=q_fmt, kv_fmt=kv_fmt)


def test_gqa_prefill_b4_h32_kv8_s8192_d128():
    """MXFP8 causal GQA prefill: B=4, 32 query heads on 8 KV heads, S=8192, d=128."""
    _run_prefill(4, 32, 8, 8192, 128, seed=21, slices=[(0, 0), (1, 13), (3, 31)])


def test_gemma_prefill_b2_h16_kv8_s8192_d256_softcap50():
    """Gemma-style: B=2, 16 query heads on 8 KV heads, S=8192, d=256, logits capped at 50 tanh(x/50), inputs x 0.5."""
    _run_prefill(2, 16, 8, 8192, 256, seed=22, mul=0.5, softcap=50.0, slices=[(0, 0), (1, 15)])


def test_gemma_prefill_mxfp6_e2m3_q_e3m2_kv():
    """The MXFP6 variant of the same shape: E2M3 queries, E3M2 keys and values."""
    _run_prefill(2, 16, 8, 8192, 256, seed=23, mul=0.5, softcap=50.0, q_fmt=rk.E2M3, kv_fmt=rk.E3M2,
                 slices=[(0, 1), (1, 14)])


def test_gqa_prefill_mxfp4_e2m1_b4_h32_kv8_s8192_d128():
    """The FP4 variant at the GQA shape: E2M1 queries, keys and values (P stays E4M3)."""
    _run_prefill(4, 32, 8, 8192, 128, seed=25, mul=0.5, q_fmt=rk.E2M1, kv_fmt=rk.E2M1, slices=[(0, 3), (3, 28)])


def test_decode_batch64_h32_kv8_l32768():
    """Llama decode: batch 64, 32 query heads on 8 KV heads, d=128, KV length 32768 for every sequence.  Three
    (batch, KV head) units against the oracle; all outputs finite and inside the hull of the decoded V."""
    B, H, Hkv, L, d = 64, 32, 8, 32768, 128
    g = torch.Generator(device="cuda").manual_seed(24)
    q = torch.randn(B, H, d, generator=g, device="cuda").bfloat16()
    K = torch.randn(B, Hkv, L, d, generator=g, device="cuda")         # 8.6 GB of fp32, freed right after quantization
    kc, ks = rk.mx_quantize(K)
    del K
    V = torch.randn(B, Hkv, L, d, generator=g, device="cuda")
    vc, vs = rk.mx_quantize(V)
    vmax = float(V.abs().max())
    del V
    o = rk.attn_decode(q, kc, vc, ks, vs)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    of = o.float()
    assert torch.isfinite(of).all()
    assert float(of.abs().max()) <= vmax * 1.01
    grp = H // Hkv
    for b, hkv in ((0, 0), (37, 5), (63, 7)):
        qh = q[b:b + 1, hkv * grp:(hkv + 1) * grp]
        ref = oracle.attn_decode(np_(qh.contiguous().view(torch.uint16)), np_(kc[b:b + 1, hkv:hkv + 1]),
                                 np_(vc[b:b + 1, hkv:hkv + 1]), np_(ks[b:b + 1, hkv:hkv + 1]), np_(vs[b:b + 1, hkv:hkv + 1]),
                                 softmax_scale=d ** -0.5)
        ma, rl = errors(np_(of[b, hkv * grp:(hkv + 1) * grp]), ref["o_f32"][0])
        assert ma <= MAX_ABS and rl <= REL_L2, ((b, hkv), ma, rl)
