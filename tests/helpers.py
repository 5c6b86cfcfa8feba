"""Shared helpers of the GPU parity tests: seeded synthetic inputs, the oracle call with the
kernel's block_n, and the tolerance of the build target (max-abs 2e-2, relative L2 1e-2)."""
import numpy as np
import torch

import oracle
import radiance_kernels_b200 as rk

MAX_ABS = 2e-2
REL_L2 = 1e-2


def randn_qkv(B, H, Hkv, Sq, Skv, d, seed, mul=1.0, qmul=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    Q = torch.randn(B, H, Sq, d, generator=g, device="cuda") * (mul * qmul)
    K = torch.randn(B, Hkv, Skv, d, generator=g, device="cuda") * mul
    V = torch.randn(B, Hkv, Skv, d, generator=g, device="cuda") * mul
    return Q, K, V


def np_(t):
    return t.detach().cpu().numpy()


def errors(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.abs(got - want).max()), float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def quantize_inputs(Q, K, V, v_axis=rk.V_SCALES_ALONG_D, fmt=rk.E4M3):
    qc, qs = rk.mx_quantize(Q, fmt)
    kc, ks = rk.mx_quantize(K, fmt)
    vc, vs = rk.mx_quantize(V, fmt) if v_axis == rk.V_SCALES_ALONG_D else rk.mx_quantize_keys(V, fmt)
    return qc, qs, kc, ks, vc, vs


def prefill_vs_oracle(B, H, Hkv, Sq, Skv, d, *, causal, seed=0, softcap=0.0, window=0, q_pos0=0, mul=1.0, qmul=1.0,
                      v_axis=rk.V_SCALES_ALONG_D, fmt=rk.E4M3, want_lse=False):
    Q, K, V = randn_qkv(B, H, Hkv, Sq, Skv, d, seed, mul, qmul)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V, v_axis, fmt)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device="cuda") if want_lse else None
    o = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=causal, softcap=softcap, window=window, q_pos0=q_pos0,
                        v_scale_axis=v_axis, q_fmt=fmt, kv_fmt=fmt, lse=lse)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    ref = oracle.attn_prefill(np_(qc), np_(kc), np_(vc), np_(qs), np_(ks), np_(vs), causal=causal,
                              softmax_scale=d ** -0.5, q_pos0=q_pos0, window=window, softcap=softcap,
                              q_fmt=fmt, kv_fmt=fmt, v_scale_axis=v_axis, block_n=128, want_lse=want_lse)
    got = np_(o.float())
    assert np.isfinite(got).all()
    out = {"got": got, "ref": ref, "err": errors(got, ref["o_f32"])}
    if want_lse:
        out["lse"] = np_(lse)
    return out
