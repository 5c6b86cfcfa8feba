#!/usr/bin/env python3
"""Regenerate the golden fixtures in this directory from the reference tree.

Run where the reference tree is checked out (its location: --ref, or the
environment variable RK_REFERENCE_DIR):

    python tests/golden/make_golden.py --ref <reference tree>

It never copies reference code into the repo; it runs / imports the reference's
own Python (lib/golden/golden.py, kernels/simt_quant/gen_quant.py) from a
scratch copy under a temp dir (the generator writes next to itself and the
reference tree is read-only) and stores only input/output vectors:

  simt_quant_kat.npz      the reference's own known-answer test for the MX block
                          quantizer: X_raw fp32 [64,512] and gold_all (8192
                          packed code words then 1024 E8M0 scale words), exactly
                          what kernels/simt_quant/kernel.cpp verifies on device.
  golden_py_vectors.npz   outputs of lib/golden/golden.py primitives on seeded
                          edge-case inputs chosen here: fp8_code_rshift (ties,
                          subnormals, saturation, signed zero, inf), block_exp /
                          pow2_neg_e, softcap (fp64 tanh reference).
  attn_fp32_ref_vectors.npz  the reference's own pure-fp32 attention references
                          (attention_reference_causal_gqa of kernels/flash_attention_mx_gqa/
                          flash_attention_model.py, attention_reference_gemma with soft-cap and
                          sliding window of kernels/flash_attention_mx_gemma/...), their mask
                          helpers and blocks_used, on seeded GQA inputs.  The model files import
                          fp8_matmul_model from a submodule that is absent; an empty stand-in
                          module satisfies that import, and only functions that never touch it
                          are called.
  rmsnorm_vectors.npz     lib/golden/golden.py rmsnorm (scalar fp32 accumulation order) on seeded inputs shaped
                          like kernels/rmsnorm_qkv_fused/gen_data.py (bf16-exact X and gamma, eps 1e-5) and on
                          plain fp32 inputs, row lengths 64 .. 1024: X, gamma, eps and the normalized output.
  mx_gemm_hw_vectors.npz  the reference's mx_golden program (lib/golden/mx_golden.cpp, built by `make -C oracle ref`)
                          run on operands drawn as kernels/gemm_mxgemmini/gen_mxgemm_data.py draws them (E4M3 codes
                          with |value| < 2, scale codes 0x7B..0x82, seed = sha256 of the shape): A, B, SA, SB and
                          the bf16 output for 64x64x64, 64x64x128, 128x128x256, and one overflowing case.
  rope_vectors.npz        lib/golden/golden.py rope_caches + rope_apply (HF Llama
                          rotate-half) on seeded inputs for head dims 64, 128, 256:
                          X, the half-width cos / sin caches and the rotated output.
"""
import argparse
import os
import importlib.util
import pathlib
import re
import shutil
import subprocess
import sys
import tempfile

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent


def load_golden(ref):
    spec = importlib.util.spec_from_file_location("ref_golden", ref / "lib" / "golden" / "golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def parse_c_array(text, name):
    m = re.search(name + r"\[\d+\]\s*=\s*\{(.*?)\};", text, re.S)
    return [t.strip() for t in m.group(1).replace("\n", " ").split(",") if t.strip()]


def make_simt_quant_kat(ref):
    with tempfile.TemporaryDirectory() as td:
        td = pathlib.Path(td)
        (td / "kernels" / "simt_quant").mkdir(parents=True)
        (td / "lib" / "golden").mkdir(parents=True)
        shutil.copy(ref / "kernels" / "simt_quant" / "gen_quant.py", td / "kernels" / "simt_quant")
        shutil.copy(ref / "lib" / "golden" / "golden.py", td / "lib" / "golden")
        subprocess.run([sys.executable, "gen_quant.py"], cwd=td / "kernels" / "simt_quant", check=True,
                       stdout=subprocess.DEVNULL)
        text = (td / "kernels" / "simt_quant" / "data").read_text()
    x = np.array([float(t.rstrip("f")) for t in parse_c_array(text, "X_raw")], dtype=np.float64).astype(np.float32)
    gold = np.array([int(t.rstrip("u"), 16) for t in parse_c_array(text, "gold_all")], dtype=np.uint32)
    assert x.size == 64 * 512 and gold.size == 8192 + 1024
    np.savez_compressed(HERE / "simt_quant_kat.npz", X_raw=x.reshape(64, 512), gold_all=gold)
    print("simt_quant_kat.npz:", x.shape, gold.shape, "scale range", gold[8192:].min(), gold[8192:].max())


def make_golden_py_vectors(ref):
    G = load_golden(ref)
    rng = np.random.default_rng(20240607)
    bits = []
    # every exponent around the E4M3 range with mantissas that sit on / next to
    # rounding ties of a 3-bit mantissa, both signs
    for e in range(127 - 14, 127 + 12):
        for m3 in range(8):
            for low in (0x00000, 0x7FFFF, 0x80000, 0x80001, 0xFFFFF, 0x40000, 0xC0000):
                for s in (0, 1):
                    bits.append((s << 31) | (e << 23) | (m3 << 20) | low)
    bits += [0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x43E00000, 0x43DFFFFF, 0x43E00001,
             0x43D00000, 0x43D80000, 0x00000001, 0x007FFFFF, 0x00800000]
    bits = np.array(bits, dtype=np.uint32)
    rnd = (rng.standard_normal(4096) * np.exp2(rng.integers(-12, 10, 4096))).astype(np.float32)
    xin = np.concatenate([bits.view(np.float32), rnd])
    codes = np.array([G.fp8_code_rshift(float(v)) for v in xin], dtype=np.uint8)

    amax_bits = np.concatenate([
        np.array([(e << 23) | m for e in range(1, 255, 3) for m in (0, 1, 0x5FFFFF, 0x600000, 0x600001, 0x7FFFFF)],
                 dtype=np.uint32),
        rng.integers(0x00800000, 0x7F000000, 512, dtype=np.uint32)])
    bexp = np.array([G.block_exp(int(b)) for b in amax_bits], dtype=np.int32)
    ok = (bexp > -127) & (bexp < 128)
    p2 = np.array([G.pow2_neg_e(int(e)) if o else 0.0 for e, o in zip(bexp, ok)], dtype=np.float32)

    cap_x = (rng.standard_normal(2048) * 60).astype(np.float32)
    cap_y = G.softcap(cap_x, 50.0)
    np.savez_compressed(HERE / "golden_py_vectors.npz", enc_in=xin, enc_codes=codes,
                        amax_bits=amax_bits, block_exp=bexp, pow2_ok=ok, pow2_neg_e=p2,
                        cap_x=cap_x, cap_y=cap_y)
    print("golden_py_vectors.npz:", xin.size, "encode cases,", amax_bits.size, "block_exp cases")


def run_mx_golden(exe, A, B, SA, SB, tmp):
    M, K = A.shape
    N = B.shape[1]
    names = {}
    for n, arr in (("A", A), ("B", B), ("SA", SA), ("SB", SB)):
        names[n] = os.path.join(tmp, n + ".bin")
        np.ascontiguousarray(arr).tofile(names[n])
    out = os.path.join(tmp, "C.bin")
    env = {k: v for k, v in os.environ.items() if not k.startswith("MX_")}
    subprocess.run([exe, str(M), str(N), str(K), names["A"], names["B"], names["SA"], names["SB"], out], check=True, env=env)
    return np.fromfile(out, np.uint16).reshape(M, N)


def make_mx_gemm_hw_vectors(ref):
    import hashlib
    G = load_golden(ref)
    exe = HERE.parent.parent / "oracle" / "_ref" / "mx_golden"
    if not exe.exists():
        subprocess.run(["make", "-C", str(HERE.parent.parent / "oracle"), "ref", "REF=" + str(ref)], check=True)
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for i, (M, N, K, full_range) in enumerate(((64, 64, 64, False), (64, 64, 128, False), (128, 128, 256, False), (32, 32, 64, True))):
            seed = int.from_bytes(hashlib.sha256(f"fp8_{M}_{N}_{K}".encode()).digest()[:4], "little")     # gen_mxgemm_data.py:35-39
            rng = np.random.default_rng(seed)
            A = G.rand_fp8(rng, M * K).reshape(M, K)
            B = G.rand_fp8(rng, K * N).reshape(K, N)
            if full_range:      # exponent fields up to 14: products overflow the 4-bit-exponent stages to inf / NaN
                A = (A | (rng.integers(0, 2, A.shape).astype(np.uint8) << 6)).astype(np.uint8)
                A[(A & 0x7F) == 0x7F] = 0x7E
            SA = rng.integers(0x7B, 0x83, size=(K // 32, M), dtype=np.uint8)
            SB = rng.integers(0x7B, 0x83, size=(K // 32, N), dtype=np.uint8)
            out[f"a{i}"] = A; out[f"b{i}"] = B; out[f"sa{i}"] = SA; out[f"sb{i}"] = SB
            out[f"c{i}"] = run_mx_golden(str(exe), A, B, SA, SB, tmp)
    np.savez_compressed(HERE / "mx_gemm_hw_vectors.npz", **out)
    print("mx_gemm_hw_vectors.npz:", {k: v.shape for k, v in out.items() if k.startswith("c")})


def make_rmsnorm_vectors(ref):
    G = load_golden(ref)
    rng = np.random.default_rng(0x5A17)
    out = {}
    for i, (M, K, bf16_exact, eps) in enumerate(((16, 256, True, 1e-5), (8, 64, False, 1e-6), (6, 1024, False, 1e-5), (5, 96, True, 1e-3))):
        X = (rng.standard_normal((M, K)) * np.exp2(rng.integers(-4, 5, (M, 1)))).astype(np.float32)
        gamma = (0.75 + 0.5 * rng.random(K)).astype(np.float32)
        if bf16_exact:
            X, gamma = G.bf16_trunc(X), G.bf16_trunc(gamma)
        Y = G.rmsnorm(X, gamma, eps)
        out[f"x{i}"] = X; out[f"g{i}"] = gamma; out[f"eps{i}"] = np.float32(eps); out[f"y{i}"] = Y.astype(np.float32)
    np.savez_compressed(HERE / "rmsnorm_vectors.npz", **out)
    print("rmsnorm_vectors.npz:", {k: v.shape for k, v in out.items() if k.startswith("y")})


def make_rope_vectors(ref):
    G = load_golden(ref)
    rng = np.random.default_rng(777)
    out = {}
    for d in (64, 128, 256):
        M = 40
        X = (rng.standard_normal((M, d)) * np.exp2(rng.integers(-3, 4, (M, 1)))).astype(np.float32)
        cos_h, sin_h, _, _ = G.rope_caches(M, d)
        Y = G.rope_apply(X, cos_h, sin_h)
        out[f"x{d}"] = X; out[f"cos{d}"] = cos_h; out[f"sin{d}"] = sin_h; out[f"y{d}"] = Y.astype(np.float32)
    np.savez_compressed(HERE / "rope_vectors.npz", **out)
    print("rope_vectors.npz:", {k: v.shape for k, v in out.items() if k.startswith("y")})


def load_attention_model(path):
    """Import a flash_attention_model.py of the reference; `fp8_matmul_model` (absent submodule) becomes a stand-in
    that only carries the three constants the module reads at import time."""
    import types
    stub = types.ModuleType("fp8_matmul_model")
    stub.GROUP, stub.INPUT_SPEC, stub.TILE = 32, "fp8:e4m3", 16
    sys.modules["fp8_matmul_model"] = stub
    try:
        spec = importlib.util.spec_from_file_location("ref_attn_model_" + path.parent.name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        del sys.modules["fp8_matmul_model"]
    return mod


def make_attn_fp32_ref_vectors(ref):
    import torch
    gqa = load_attention_model(ref / "kernels" / "flash_attention_mx_gqa" / "flash_attention_model.py")
    gem = load_attention_model(ref / "kernels" / "flash_attention_mx_gemma" / "flash_attention_model.py")
    out = {}
    # causal GQA, query block offset into the keys (the reference's own generator and head layout)
    n_q, n_kv, Sq, Sk, d, q_pos0 = 4, 2, 24, 64, 32, 36
    Q, K, V = gqa.make_inputs_gqa(Sq, Sk, d, n_q, n_kv, seed=3)
    scale = d ** -0.5
    out["gqa_q"], out["gqa_k"], out["gqa_v"] = Q.numpy(), K.numpy(), V.numpy()
    out["gqa_o"] = gqa.attention_reference_causal_gqa(Q, K, V, scale, q_pos0).numpy()
    out["gqa_meta"] = np.array([q_pos0], np.int32)
    out["gqa_mask"] = gqa.causal_bool_mask(Sq, Sk, q_pos0).numpy()
    out["blocks_used"] = np.array([[sq, sk, qp, bn, gqa.blocks_used(sq, sk, qp, bn)]
                                   for sq in (64, 128) for sk in (128, 512) for qp in (0, 64, 300) for bn in (64, 128)],
                                  np.int32)
    # Gemma: soft-cap (Q scaled up so that it bites, as the reference's generator does) and sliding window
    n_q, n_kv, Sq, Sk, d, q_pos0, cap, window = 4, 2, 24, 64, 32, 40, 50.0, 20
    Q, K, V = gem.make_inputs_gqa(Sq, Sk, d, n_q, n_kv, seed=5)
    Q = Q * 20.0
    out["gem_q"], out["gem_k"], out["gem_v"] = Q.numpy(), K.numpy(), V.numpy()
    out["gem_o_cap_win"] = gem.attention_reference_gemma(Q, K, V, scale, q_pos0, attn_softcap=cap, window=window).numpy()
    out["gem_o_cap"] = gem.attention_reference_gemma(Q, K, V, scale, q_pos0, attn_softcap=cap, window=None).numpy()
    out["gem_meta"] = np.array([q_pos0, window], np.int32)
    out["gem_cap"] = np.array([cap], np.float32)
    out["gem_mask"] = gem.gemma_bool_mask(Sq, Sk, q_pos0, window).numpy()
    np.savez_compressed(HERE / "attn_fp32_ref_vectors.npz", **out)
    print("attn_fp32_ref_vectors.npz:", out["gqa_o"].shape, out["gem_o_cap_win"].shape, out["blocks_used"].shape)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("RK_REFERENCE_DIR") or str(HERE.parents[2] / "reference"),
                    help="the reference's source tree (default: $RK_REFERENCE_DIR, else ../reference beside this checkout)")
    ref = pathlib.Path(ap.parse_args().ref)
    make_simt_quant_kat(ref)
    make_golden_py_vectors(ref)
    make_rope_vectors(ref)
    make_rmsnorm_vectors(ref)
    make_mx_gemm_hw_vectors(ref)
    make_attn_fp32_ref_vectors(ref)
