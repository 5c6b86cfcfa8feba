"""RMSNorm fused with the MX quantizer (the QKV-projection prologue of kernels/rmsnorm_qkv_fused) on the GPU: codes and
scales bit-exact with the reference's rmsnorm golden followed by the block quantizer."""
import os

import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import np_

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _expect(x, gamma, eps, fmt, unit):
    y = oracle.rmsnorm(x, gamma, eps)
    if unit:
        L = oracle.lib()
        codes = np.array([L.rko_encode_elem_rne(float(v), fmt) for v in y.ravel()], np.uint8).reshape(y.shape)
        return codes, np.full((y.shape[0], y.shape[1] // 32), 0x7F, np.uint8)
    return oracle.quantize(y, fmt)


def test_reference_golden_inputs_bit_exact():
    """The inputs of the committed rmsnorm fixture (made by importing lib/golden/golden.py): normalized values that
    equal the reference's bit for bit go through the same block rule, so codes and scales must match exactly."""
    z = np.load(os.path.join(GOLDEN, "rmsnorm_vectors.npz"))
    for i in range(4):
        x, g, eps = z[f"x{i}"], z[f"g{i}"], float(z[f"eps{i}"])
        if x.shape[1] % 32:
            continue
        want_c, want_s = oracle.quantize(z[f"y{i}"])
        c, s = rk.rmsnorm_mx_quantize(torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda(), eps)
        assert np.array_equal(np_(c), want_c) and np.array_equal(np_(s), want_s), i


@pytest.mark.parametrize("rows,K,fmt,unit,bf16", [(64, 256, 0, True, True), (100, 4096, 0, False, False), (33, 128, 3, False, False),
                                                  (257, 1024, 1, False, True), (1, 32, 0, False, False), (70, 2048, 2, False, False),
                                                  (48, 512, 4, False, False), (96, 256, 4, False, True)])
def test_rmsnorm_quantize_matches_oracle(rows, K, fmt, unit, bf16):
    rng = np.random.default_rng(rows * 7 + K)
    x = (rng.standard_normal((rows, K)) * np.exp2(rng.integers(-6, 7, (rows, 1)))).astype(np.float32)
    gamma = (0.75 + 0.5 * rng.random(K)).astype(np.float32)
    xt = torch.from_numpy(x).cuda()
    if bf16:
        xt = xt.bfloat16()
        x = np_(xt.float())
    eps = 1e-5
    want_c, want_s = _expect(x, gamma, eps, fmt, unit)
    c, s = rk.rmsnorm_mx_quantize(xt, torch.from_numpy(gamma).cuda(), eps, fmt=fmt, unit_scale=unit)
    torch.cuda.synchronize()
    assert np.array_equal(np_(s), want_s)
    assert np.array_equal(np_(c), want_c)


def test_zero_rows_and_huge_rows():
    """An all-zero row normalizes to zeros (rms = 1/sqrt(eps)); a row of large values stays finite."""
    x = np.zeros((3, 64), np.float32)
    x[1] = 3.0e18
    x[2, 5] = -1.0e-30
    gamma = np.ones(64, np.float32)
    want_c, want_s = oracle.quantize(oracle.rmsnorm(x, gamma, 1e-6))
    c, s = rk.rmsnorm_mx_quantize(torch.from_numpy(x).cuda(), torch.from_numpy(gamma).cuda(), 1e-6)
    assert np.array_equal(np_(c), want_c) and np.array_equal(np_(s), want_s)
