"""Prefill attention on the GPU against the CPU oracle (same block_n, same P rule), through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import MAX_ABS, REL_L2, errors, np_, prefill_vs_oracle, quantize_inputs, randn_qkv

pytestmark = pytest.mark.gpu


def _check(r):
    ma, rl = r["err"]
    assert ma <= MAX_ABS and rl <= REL_L2, (ma, rl)


def test_config1_single_head_noncausal_d64():
    """B=1 H=1 S=256 d=64 non-causal: the reference's own CPU-runnable case."""
    for seed in (0, 1, 2):
        _check(prefill_vs_oracle(1, 1, 1, 256, 256, 64, causal=False, seed=seed))


def test_single_tile_d128():
    _check(prefill_vs_oracle(1, 1, 1, 128, 128, 128, causal=False))


def test_causal_mha_d128():
    _check(prefill_vs_oracle(2, 4, 4, 1024, 1024, 128, causal=True, seed=1))


def test_causal_gqa_d128_group4():
    _check(prefill_vs_oracle(1, 8, 2, 768, 768, 128, causal=True, seed=2))


def test_reference_gqa_shape():
    """The reference's GQA kernel shape: 8 query heads on 2 KV heads, Sq=64 Sk=256 d=64, q_pos0=64
    (kernels/regen_data.sh:31-32)."""
    _check(prefill_vs_oracle(1, 8, 2, 64, 256, 64, causal=True, q_pos0=64, seed=0))


def test_gemma_softcap_d256():
    _check(prefill_vs_oracle(1, 4, 2, 512, 512, 256, causal=True, softcap=50.0, mul=0.5, seed=3))


def test_gemma_reference_style_cap_bites_window():
    """Q scaled by 50 so the cap saturates, sliding window 128, d=256, 8:4 heads
    (kernels/flash_attention_mx_gemma/fa_gen_data.py:77-79, kernels/regen_data.sh:33-34)."""
    _check(prefill_vs_oracle(1, 8, 4, 256, 512, 256, causal=True, softcap=50.0, qmul=50.0, q_pos0=256, window=128))


@pytest.mark.parametrize("d", [128, 256])
def test_softcap_scores_on_both_sides_of_the_series_limit(d):
    """The capped kernels evaluate tanh by its series while a warp's scores of a key tile stay below cap / 8 and by
    the exponential form otherwise: with Q scaled by 1.6 the largest |score| of a tile lies around that limit
    (6.25 at cap 50), so both forms run inside one launch and must meet the oracle's tanh."""
    _check(prefill_vs_oracle(1, 4, 2, 640, 640, d, causal=True, softcap=50.0, qmul=1.6, seed=23))
    _check(prefill_vs_oracle(1, 2, 2, 384, 384, d, causal=False, softcap=30.0, qmul=1.0, seed=24))


def test_sliding_window_d128():
    _check(prefill_vs_oracle(1, 2, 1, 640, 640, 128, causal=True, window=200, seed=4))


@pytest.mark.parametrize("d,S,window,q_pos0,softcap", [(128, 1536, 300, 0, 0.0), (128, 1100, 128, 700, 0.0),
                                                      (256, 1280, 200, 0, 50.0), (128, 900, 1, 0, 0.0)])
def test_sliding_window_skips_key_tiles_below_the_window(d, S, window, q_pos0, softcap):
    """Long sequences with a short window: most key tiles lie wholly below the window and are never loaded; the
    result must equal the oracle's, which masks them (both kernels: d = 128 pairs of query tiles, d = 256)."""
    _check(prefill_vs_oracle(1, 2, 1, S, S + q_pos0, d, causal=True, window=window, q_pos0=q_pos0, softcap=softcap,
                             mul=0.5 if d == 256 else 1.0, seed=60 + window))


def test_ragged_lengths_and_offset():
    _check(prefill_vs_oracle(1, 2, 2, 200, 333, 128, causal=True, q_pos0=133, seed=5))
    _check(prefill_vs_oracle(1, 1, 1, 1, 97, 64, causal=False, seed=6))
    _check(prefill_vs_oracle(1, 2, 1, 130, 31, 128, causal=False, seed=7))


def test_rows_without_visible_keys_are_zero():
    """q_pos0 < 0: the first rows see no key at all -> O = 0 (the l <= 0 guard of finalize_O)."""
    r = prefill_vs_oracle(1, 1, 1, 256, 256, 128, causal=True, q_pos0=-130, seed=8)
    _check(r)
    assert np.all(r["got"][0, 0, :130] == 0.0)


def test_v_scales_along_keys_reference_layout():
    _check(prefill_vs_oracle(1, 2, 1, 384, 384, 128, causal=True, v_axis=rk.V_SCALES_ALONG_KEYS, seed=9))
    _check(prefill_vs_oracle(1, 1, 1, 256, 200, 64, causal=False, v_axis=rk.V_SCALES_ALONG_KEYS, seed=10))


def test_e5m2_operands():
    _check(prefill_vs_oracle(1, 2, 1, 256, 256, 128, causal=True, fmt=rk.E5M2, seed=11))


def test_mxfp6_operands_e2m3_q_e3m2_kv():
    """MXFP6 variant: E2M3 queries, E3M2 keys and values (P stays E4M3), 6-bit codes packed for the tensor core."""
    import oracle
    for (B, H, Hkv, Sq, Skv, d, axis) in ((1, 2, 1, 256, 256, 128, rk.V_SCALES_ALONG_D), (1, 4, 2, 200, 333, 64, rk.V_SCALES_ALONG_KEYS),
                                          (1, 2, 1, 384, 384, 256, rk.V_SCALES_ALONG_D)):
        Q, K, V = randn_qkv(B, H, Hkv, Sq, Skv, d, seed=31, mul=0.5)
        qc, qs = rk.mx_quantize(Q, rk.E2M3)
        kc, ks = rk.mx_quantize(K, rk.E3M2)
        vc, vs = rk.mx_quantize(V, rk.E3M2) if axis == rk.V_SCALES_ALONG_D else rk.mx_quantize_keys(V, rk.E3M2)
        o = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, softcap=50.0 if d == 256 else 0.0, q_fmt=rk.E2M3, kv_fmt=rk.E3M2,
                            v_scale_axis=axis)
        torch.cuda.synchronize()
        assert rk.last_device_status() == 0
        ref = oracle.attn_prefill(np_(qc), np_(kc), np_(vc), np_(qs), np_(ks), np_(vs), causal=True, softmax_scale=d ** -0.5,
                                  softcap=50.0 if d == 256 else 0.0, q_fmt=rk.E2M3, kv_fmt=rk.E3M2, v_scale_axis=axis, block_n=128)
        ma, rl = errors(np_(o.float()), ref["o_f32"])
        assert ma <= MAX_ABS and rl <= REL_L2, (d, ma, rl)


def test_mxfp4_operands_e2m1():
    """FP4 variant (lib/golden/mx_fp_math.h:238-246; the reference studies it in
    kernels/flash_attention_mx_gqa/fp6_attn_relerr.py:31-36): E2M1 queries, keys and values under E8M0 block scales,
    P stays E4M3; the 4-bit codes cross the interface one per byte and are packed two per byte for the tensor core.
    Also E2M1 keys/values under E4M3 queries, the mix a 4-bit KV cache gives."""
    import oracle
    for (B, H, Hkv, Sq, Skv, d, axis, qf) in ((1, 2, 1, 256, 256, 128, rk.V_SCALES_ALONG_D, rk.E2M1),
                                              (1, 4, 2, 200, 333, 64, rk.V_SCALES_ALONG_KEYS, rk.E2M1),
                                              (1, 2, 1, 384, 384, 256, rk.V_SCALES_ALONG_D, rk.E2M1),
                                              (2, 4, 2, 512, 512, 128, rk.V_SCALES_ALONG_KEYS, rk.E4M3)):
        Q, K, V = randn_qkv(B, H, Hkv, Sq, Skv, d, seed=37, mul=0.5)
        qc, qs = rk.mx_quantize(Q, qf)
        kc, ks = rk.mx_quantize(K, rk.E2M1)
        vc, vs = rk.mx_quantize(V, rk.E2M1) if axis == rk.V_SCALES_ALONG_D else rk.mx_quantize_keys(V, rk.E2M1)
        assert int(qc.max()) < (16 if qf == rk.E2M1 else 256) and int(kc.max()) < 16 and int(vc.max()) < 16
        o = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, softcap=50.0 if d == 256 else 0.0, q_fmt=qf, kv_fmt=rk.E2M1,
                            v_scale_axis=axis)
        torch.cuda.synchronize()
        assert rk.last_device_status() == 0
        ref = oracle.attn_prefill(np_(qc), np_(kc), np_(vc), np_(qs), np_(ks), np_(vs), causal=True, softmax_scale=d ** -0.5,
                                  softcap=50.0 if d == 256 else 0.0, q_fmt=qf, kv_fmt=rk.E2M1, v_scale_axis=axis, block_n=128)
        ma, rl = errors(np_(o.float()), ref["o_f32"])
        assert ma <= MAX_ABS and rl <= REL_L2, (d, ma, rl)


def test_dense_sub_byte_operands_give_the_same_output():
    """Operands handed over in the dense 6- / 4-bit form (rk_mx_pack_rows, rk_mx_pack_vt) -- what a KV cache kept in
    those formats holds -- give bit for bit the output of the call that packs them itself, and with scale-factor
    atoms on top the same again."""
    for (B, H, Hkv, Sq, Skv, d, qf, kvf, cap) in ((1, 4, 2, 200, 333, 64, rk.E2M3, rk.E3M2, 0.0),
                                                    (2, 4, 2, 512, 512, 128, rk.E2M1, rk.E2M1, 0.0),
                                                    (1, 2, 1, 384, 384, 256, rk.E2M3, rk.E3M2, 50.0)):
        Q, K, V = randn_qkv(B, H, Hkv, Sq, Skv, d, seed=41, mul=0.5)
        qc, qs = rk.mx_quantize(Q, qf)
        kc, ks = rk.mx_quantize(K, kvf)
        vc, vs = rk.mx_quantize_keys(V, kvf)
        want = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, softcap=cap, q_fmt=qf, kv_fmt=kvf,
                               v_scale_axis=rk.V_SCALES_ALONG_KEYS)
        qp, kp, vtp = rk.mx_pack_rows(qc, qf), rk.mx_pack_rows(kc, kvf), rk.mx_pack_vt(vc, kvf)
        bits_q, bits_kv = (4 if qf == rk.E2M1 else 6), (4 if kvf == rk.E2M1 else 6)
        dp, sp = (d + 127) // 128 * 128, (Skv + 127) // 128 * 128
        assert qp.shape == (B, H, Sq, dp * bits_q // 8) and kp.shape == (B, Hkv, Skv, dp * bits_kv // 8)
        assert vtp.shape == (B, Hkv, d, sp * bits_kv // 8)
        kw = dict(S_q=Sq, S_kv=Skv, d=d, q_fmt=qf, kv_fmt=kvf, causal=True, softcap=cap)
        got = rk.attn_prefill_packed(qp, kp, vtp, qs, ks, vs, **kw)
        assert torch.equal(got, want)
        # the first codes of a row, unpacked by hand
        row = qp[0, 0, 0].cpu().numpy().astype(np.uint64)
        word = int(row[0]) | int(row[1]) << 8 | int(row[2]) << 16
        first = [(word >> (bits_q * i)) & ((1 << bits_q) - 1) for i in range(3)]
        assert first == [int(x) for x in qc[0, 0, 0, :3].cpu()]
        # prepared all the way: scale-factor atoms as well, so that the call is the attention kernel alone
        _, qa = rk.mx_quantize_ex(Q, qf, rk.SCALES_SF_ATOMS)
        _, ka = rk.mx_quantize_ex(K, kvf, rk.SCALES_SF_ATOMS)
        _, va = rk.mx_quantize_keys_ex(V, kvf, rk.SCALES_SF_ATOMS)
        got2 = rk.attn_prefill_packed(qp, kp, vtp, qa, ka, va, q_scale_layout=rk.SCALES_SF_ATOMS,
                                      k_scale_layout=rk.SCALES_SF_ATOMS, v_scale_layout=rk.SCALES_SF_ATOMS, **kw)
        assert torch.equal(got2, want)
        torch.cuda.synchronize()
        assert rk.last_device_status() == 0
    # 8-bit formats have no dense form (the front end stops it; the library would answer RK_ERR_BAD_FORMAT)
    with pytest.raises((rk.RkError, ValueError)):
        rk.attn_prefill_packed(qp, kp, vtp, qs, ks, vs, S_q=Sq, S_kv=Skv, d=d, q_fmt=rk.E4M3, kv_fmt=rk.E3M2, causal=True)


def test_lse_output():
    r = prefill_vs_oracle(1, 2, 1, 256, 256, 128, causal=True, want_lse=True, seed=12)
    _check(r)
    assert np.abs(r["lse"] - r["ref"]["lse"]).max() < 1e-3


def test_bit_identical_across_runs():
    """Race check borrowed from the reference ("bit-identical O across 13 runs",
    kernels/flash_attention_mx/kernel.cpp:158-160)."""
    Q, K, V = randn_qkv(2, 4, 2, 1024, 1024, 128, seed=13)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V)
    first = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
    for _ in range(5):
        again = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
        assert torch.equal(first, again)
    assert rk.last_device_status() == 0


def test_host_buffer_entry_point_matches_device_one():
    Q, K, V = randn_qkv(1, 4, 2, 512, 512, 128, seed=14)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V)
    dev = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
    host = rk.attn_prefill_host(*[t.cpu().pin_memory() for t in (qc, kc, vc, qs, ks, vs)], causal=True)
    assert torch.equal(dev.cpu(), host)


@pytest.mark.parametrize("B,H,Hkv,S,axis", [(3, 6, 3, 256, 1), (10, 2, 2, 128, 0), (2, 8, 8, 160, 1), (9, 4, 1, 128, 1)])
def test_host_entry_point_chunking(B, H, Hkv, S, axis):
    """The host entry point cuts the call into chunks of whole (batch, KV head) units (ranges of KV heads when
    the batch is small, groups of batches when it is large): every chunking gives the device call's bits, for O
    and for the log-sum-exp, with either V scale layout and a ragged sequence length."""
    Q, K, V = randn_qkv(B, H, Hkv, S, S, 128, seed=40 + B)
    qc, qs = rk.mx_quantize(Q); kc, ks = rk.mx_quantize(K)
    vc, vs = rk.mx_quantize(V) if axis == 1 else rk.mx_quantize_keys(V)
    lse = torch.empty(B, H, S, dtype=torch.float32, device="cuda")
    dev = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, v_scale_axis=axis, lse=lse)
    runner = rk.PrefillHostRunner(*[t.cpu().pin_memory() for t in (qc, kc, vc, qs, ks, vs)], causal=True,
                                  v_scale_axis=axis, want_lse=True)
    for _ in range(2):                      # twice: the shared copy streams and events are reused
        host = runner.run()
        assert torch.equal(dev.cpu(), host)
        assert torch.equal(lse.cpu(), runner.lse)
    assert rk.last_device_status() == 0


def test_full_size_head_slices_match_oracle():
    """B=8 H=16 S=4096 d=128 causal (the benchmark workload): the whole tensor runs on the GPU, two
    (batch, head) slices are checked against the oracle, and every row is checked for the size-independent
    property that O is a convex combination of V rows (|O| <= max|V| per column block)."""
    B, H, S, d = 8, 16, 4096, 128
    Q, K, V = randn_qkv(B, H, H, S, S, d, seed=15)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V)
    del Q, K
    o = rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
    torch.cuda.synchronize()
    assert rk.last_device_status() == 0
    assert torch.isfinite(o.float()).all()
    assert o.float().abs().max() <= V.abs().max() * 1.01
    for sl in (0, B * H - 1):
        b, h = divmod(sl, H)
        ref = oracle.attn_prefill(np_(qc[b:b + 1, h:h + 1]), np_(kc[b:b + 1, h:h + 1]), np_(vc[b:b + 1, h:h + 1]),
                                  np_(qs[b:b + 1, h:h + 1]), np_(ks[b:b + 1, h:h + 1]), np_(vs[b:b + 1, h:h + 1]),
                                  causal=True, softmax_scale=d ** -0.5, block_n=128)
        ma, rl = errors(np_(o[b, h].float()), ref["o_f32"][0, 0])
        assert ma <= MAX_ABS and rl <= REL_L2, (sl, ma, rl)


@pytest.mark.parametrize("d,qmul", [(128, 1.0), (128, 6.0), (64, 1.0)])
def test_stage_parity_s_and_requantized_p(d, qmul):
    """Stage-level parity on the first key tile of the last query tile (the kernels' debug dump): S = Q K^T within
    fp32 reassociation error, and the requantized P -- E4M3 codes and E8M0 block scales -- equal to the oracle's.
    A code may differ by one step where the fp32 p sits on a truncation boundary; such elements are counted and
    must stay below 0.05 %."""
    import ctypes as C
    Sq = Skv = 256
    Q, K, V = randn_qkv(1, 1, 1, Sq, Skv, d, seed=50, qmul=qmul)
    qc, qs, kc, ks, vc, vs = quantize_inputs(Q, K, V)
    dbg = torch.zeros(32768, dtype=torch.float32, device="cuda")
    rk.lib().rk_debug_set_prefill_dump(C.c_void_p(dbg.data_ptr()))
    try:
        rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True)
        torch.cuda.synchronize()
    finally:
        rk.lib().rk_debug_set_prefill_dump(None)
    assert rk.last_device_status() == 0
    scale = d ** -0.5
    r = oracle.attn_prefill(np_(qc), np_(kc), np_(vc), np_(qs), np_(ks), np_(vs), causal=True, softmax_scale=scale,
                            block_n=128, dump_slice=0)
    dd = np_(dbg)
    rows = slice(128, 256)                                    # the dump is the last query tile, key tile 0
    s_gpu = dd[:128 * 128].reshape(128, 128)
    s_ref = r["s"][rows, :128] / scale
    assert np.abs(s_gpu - s_ref).max() <= 1e-5 * np.abs(s_ref).max() + 1e-6
    pcodes = dd[128 * 128: 128 * 128 + 128 * 32].view(np.uint8).reshape(128, 128)
    pscale = dd[128 * 128 + 128 * 32: 128 * 128 + 128 * 32 + 128].view(np.uint8).reshape(128, 4)
    assert np.array_equal(pscale, r["p_scales"][rows, :4])
    diff = pcodes.astype(np.int32) - r["p_codes"][rows, :128].astype(np.int32)
    bad = np.count_nonzero(diff)
    assert np.abs(diff).max() <= 1 and bad <= 0.0005 * diff.size, (bad, int(np.abs(diff).max()))
    # running max and row sum after the tile's last key tile: m is kept in the log2 domain on the GPU
    ml = dd[128 * 128 + 128 * 32 + 128: 128 * 128 + 128 * 32 + 128 + 256].reshape(128, 2)
    m_gpu, l_gpu = ml[:, 0] * np.log(2.0), ml[:, 1]
    assert np.abs(m_gpu - r["m"][rows]).max() <= 4e-6 * np.abs(r["m"][rows]).max() + 1e-6
    assert np.abs(l_gpu / r["l"][rows] - 1.0).max() <= 1e-4
