"""MX matmul in the mesh's hardware-accumulate semantics on the GPU: bit-exact with the output of the reference's own
mx_golden program (committed fixture, made by running it on operands drawn as its GEMM data generator draws them)
and with the CPU oracle on larger shapes, overflow to inf / NaN included."""
import os

import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import np_

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gpu(A, B, SA, SB):
    c = rk.mx_gemm_hw(*[torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (A, B, SA, SB)])
    torch.cuda.synchronize()
    return np_(c.view(torch.uint16))


def test_reference_program_outputs_bit_exact():
    z = np.load(os.path.join(GOLDEN, "mx_gemm_hw_vectors.npz"))
    for i in range(4):
        got = _gpu(z[f"a{i}"], z[f"b{i}"], z[f"sa{i}"], z[f"sb{i}"])
        assert np.array_equal(got, z[f"c{i}"]), (i, int((got != z[f"c{i}"]).sum()))


@pytest.mark.parametrize("M,N,K,expmax", [(128, 128, 512, 7), (128, 256, 2048, 7), (16, 48, 96, 14), (128, 64, 5632, 6)])
def test_matches_oracle_on_projection_shapes(M, N, K, expmax):
    """The batched-decode projection shape (M = 128 rows of activations) and deep K, operands bounded as the reference
    bounds them (exponent field <= 7) or unbounded (products overflow the 4-bit-exponent stages)."""
    rng = np.random.default_rng(M + N + K)
    code = lambda shape: ((rng.integers(0, 2, shape) << 7) | (rng.integers(0, expmax + 1, shape) << 3) | rng.integers(0, 8, shape)).astype(np.uint8)
    A, B = code((M, K)), code((K, N))
    SA = rng.integers(0x70, 0x90, (K // 32, M)).astype(np.uint8)
    SB = rng.integers(0x70, 0x90, (K // 32, N)).astype(np.uint8)
    want = oracle.mx_gemm_hw(A, B, SA, SB)
    got = _gpu(A, B, SA, SB)
    assert np.array_equal(got, want), int((got != want).sum())
