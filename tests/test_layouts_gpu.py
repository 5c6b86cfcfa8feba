"""Operand layouts at the boundary: the reference's group-major Q scales, its per-block K^T tiles, and the
scale-factor atoms the tensor core reads, all accepted as they lie and all giving the bits of the row-major call."""
import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import MAX_ABS, REL_L2, errors, np_, randn_qkv

pytestmark = pytest.mark.gpu


def _atoms_from_rowmajor(scales, S, d):
    """numpy restatement of the atom layout: scales [n, S, d/32] -> [n, ceil(S/128), ceil(d/128), 512]."""
    n = scales.shape[0]
    nt, dch = (S + 127) // 128, (d + 127) // 128
    out = np.full((n, nt, dch, 512), 0x7F, np.uint8)
    for r in range(S):
        for b in range(d // 32):
            out[:, r // 128, b // 4, ((r % 128) % 32) * 16 + ((r % 128) // 32) * 4 + (b % 4)] = scales[:, r, b]
    return out


@pytest.mark.parametrize("S,d,dtype", [(256, 128, torch.float32), (200, 64, torch.float32), (130, 256, torch.bfloat16)])
def test_quantizer_scale_layouts(S, d, dtype):
    g = torch.Generator(device="cuda").manual_seed(S + d)
    x = (torch.randn(3, S, d, generator=g, device="cuda") * 3.0).to(dtype)
    c0, s0 = rk.mx_quantize(x)
    for layout in (rk.SCALES_ROWMAJOR, rk.SCALES_GROUPMAJOR, rk.SCALES_SF_ATOMS):
        c, s = rk.mx_quantize_ex(x, scale_layout=layout)
        assert torch.equal(c, c0)
        if layout == rk.SCALES_ROWMAJOR:
            assert torch.equal(s, s0)
        elif layout == rk.SCALES_GROUPMAJOR:
            assert torch.equal(s, s0.transpose(1, 2).contiguous())
        else:
            assert np.array_equal(np_(s), _atoms_from_rowmajor(np_(s0), S, d))


@pytest.mark.parametrize("S,d", [(256, 128), (200, 64), (96, 256)])
def test_key_axis_quantizer_atoms(S, d):
    g = torch.Generator(device="cuda").manual_seed(7 * S + d)
    x = torch.randn(2, S, d, generator=g, device="cuda")
    c0, s0 = rk.mx_quantize_keys(x)                         # [2, ceil(S/32), d]
    c, s = rk.mx_quantize_keys_ex(x, scale_layout=rk.SCALES_SF_ATOMS)
    assert torch.equal(c, c0)
    s0n, sn = np_(s0), np_(s)
    want = np.full(sn.shape, 0x7F, np.uint8)
    for kb in range(s0n.shape[1]):
        for n in range(d):
            want[:, kb // 4, n // 128, ((n % 128) % 32) * 16 + ((n % 128) // 32) * 4 + (kb % 4)] = s0n[:, kb, n]
    assert np.array_equal(sn, want)


@pytest.mark.parametrize("B,H,Hkv,Sq,Skv,d", [(1, 4, 2, 384, 384, 128), (2, 2, 1, 200, 333, 64), (1, 2, 2, 256, 256, 256)])
def test_prefill_accepts_group_major_scales_and_atoms(B, H, Hkv, Sq, Skv, d):
    Q, K, V = randn_qkv(B, H, Hkv, Sq, Skv, d, seed=70 + d, mul=0.5 if d == 256 else 1.0)
    qc, qs = rk.mx_quantize(Q); kc, ks = rk.mx_quantize(K); vc, vs = rk.mx_quantize_keys(V)
    base = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, v_scale_axis=rk.V_SCALES_ALONG_KEYS, q_pos0=Skv - Sq)
    gm = rk.attn_prefill(qc, kc, vc, qs.transpose(2, 3).contiguous(), ks.transpose(2, 3).contiguous(), vs, causal=True,
                         v_scale_axis=rk.V_SCALES_ALONG_KEYS, q_pos0=Skv - Sq, q_scale_layout=rk.SCALES_GROUPMAJOR,
                         k_scale_layout=rk.SCALES_GROUPMAJOR)
    assert torch.equal(base, gm)
    _, qa = rk.mx_quantize_ex(Q, scale_layout=rk.SCALES_SF_ATOMS)
    _, ka = rk.mx_quantize_ex(K, scale_layout=rk.SCALES_SF_ATOMS)
    _, va = rk.mx_quantize_keys_ex(V, scale_layout=rk.SCALES_SF_ATOMS)
    at = rk.attn_prefill(qc, kc, vc, qa, ka, va, causal=True, v_scale_axis=rk.V_SCALES_ALONG_KEYS, q_pos0=Skv - Sq,
                         q_scale_layout=rk.SCALES_SF_ATOMS, k_scale_layout=rk.SCALES_SF_ATOMS,
                         v_scale_layout=rk.SCALES_SF_ATOMS)
    assert torch.equal(base, at)
    assert rk.last_device_status() == 0


def test_import_of_reference_kt_blocks_and_full_reference_layout():
    """The reference GQA shape (8 query heads on 2 KV heads, Sq=64 Sk=256 d=64, q_pos0=64, Bk=64,
    kernels/regen_data.sh:31-32) fed in the layout its generator emits
    (kernels/flash_attention_mx_gqa/fa_gen_data.py:97-120)."""
    n_q, n_kv, Sq, Sk, d, q_pos0, Bk = 8, 2, 64, 256, 64, 64, 64
    nbu = min(Sk // Bk, (q_pos0 + Sq - 1) // Bk + 1)
    skv = nbu * Bk
    g = torch.Generator(device="cuda").manual_seed(5)
    Q = torch.randn(1, n_q, Sq, d, generator=g, device="cuda")
    K = torch.randn(1, n_kv, skv, d, generator=g, device="cuda")
    V = torch.randn(1, n_kv, skv, d, generator=g, device="cuda")
    qc, qs = rk.mx_quantize(Q); kc, ks = rk.mx_quantize(K); vc, vs = rk.mx_quantize_keys(V)
    # the reference's arrays
    A_scales_row = qs[0].transpose(1, 2).contiguous()                                  # [NQ][GK][SQ]
    B_blocks = kc[0].view(n_kv, nbu, Bk, d).transpose(2, 3).contiguous().view(n_kv * nbu * d, Bk)
    B_scales = ks[0].view(n_kv, nbu, Bk, d // 32).transpose(2, 3).contiguous().view(n_kv * nbu * (d // 32), Bk)
    k2, ks2 = rk.import_kt_blocks(B_blocks, B_scales, n_kv, nbu, Bk, d)
    assert torch.equal(k2, kc[0]) and torch.equal(ks2, ks[0])
    o = rk.attn_prefill(qc, k2[None], vc, A_scales_row[None], ks2[None], vs, causal=True, q_pos0=q_pos0,
                        v_scale_axis=rk.V_SCALES_ALONG_KEYS, q_scale_layout=rk.SCALES_GROUPMAJOR)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    ref = oracle.attn_prefill(np_(qc), np_(kc), np_(vc), np_(qs), np_(ks), np_(vs), causal=True, softmax_scale=d ** -0.5,
                              q_pos0=q_pos0, v_scale_axis=rk.V_SCALES_ALONG_KEYS, block_n=128)
    ma, rl = errors(np_(o.float()), ref["o_f32"])
    assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)
