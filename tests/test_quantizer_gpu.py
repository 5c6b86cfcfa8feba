"""MX block quantizer on the GPU: bit-exact against the oracle, the reference's known-answer test and
golden.py vectors, through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle
import radiance_kernels_b200 as rk
from helpers import np_

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def test_simt_quant_known_answer_on_gpu():
    kat = np.load(os.path.join(G, "simt_quant_kat.npz"))
    x = torch.from_numpy(kat["X_raw"]).cuda()
    codes, scales = rk.mx_quantize(x)
    packed = np_(codes).reshape(-1, 4).astype(np.uint32)
    words = packed[:, 0] | (packed[:, 1] << 8) | (packed[:, 2] << 16) | (packed[:, 3] << 24)
    assert np.array_equal(words, kat["gold_all"][:8192])
    assert np.array_equal(np_(scales).reshape(-1).astype(np.uint32), kat["gold_all"][8192:])


def test_golden_py_encode_vectors_on_gpu():
    """Each golden.py fp8_code_rshift vector becomes element 0 of a block whose amax is exactly 448*2^0 wide,
    so the block scale is 2^0 and the code must equal the vector's code."""
    v = np.load(os.path.join(G, "golden_py_vectors.npz"))
    xin = v["enc_in"]
    keep = np.isfinite(xin) & (np.abs(xin) <= 448.0)
    xin, want = xin[keep], v["enc_codes"][keep]
    x = np.zeros((xin.size, 32), np.float32)
    x[:, 0] = xin
    x[:, 1] = 448.0          # pins e = 0
    codes, scales = rk.mx_quantize(torch.from_numpy(x).cuda())
    assert np.all(np_(scales) == 127)
    assert np.array_equal(np_(codes)[:, 0], want)


@pytest.mark.parametrize("fmt", [rk.E4M3, rk.E5M2, rk.E2M3, rk.E3M2])
def test_hardware_converter_equals_reference_encoder_on_every_fp32(fmt):
    """All 2^32 fp32 bit patterns (NaNs aside, which the kernels route to the integer encoder): the hardware
    converter used in the hot loops gives the code of the reference's round-shift encoder
    (kernels/simt_quant/kernel.cpp:56-81)."""
    import ctypes as C
    count = torch.zeros(1, dtype=torch.int64, device="cuda")
    first = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rc = rk.lib().rk_debug_verify_encoder(fmt, C.c_void_p(count.data_ptr()), C.c_void_p(first.data_ptr()), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(count.item()) == 0, f"{int(count.item())} mismatches, first at bits {int(first.item()) & 0xFFFFFFFF:#010x}"


@pytest.mark.parametrize("fmt", [rk.E4M3, rk.E5M2, rk.E2M3, rk.E3M2, rk.E2M1])
def test_quantize_rows_bit_exact(fmt):
    g = torch.Generator(device="cuda").manual_seed(11 + fmt)
    x = torch.randn(512, 1024, generator=g, device="cuda")
    x = x * torch.exp2(torch.randint(-20, 20, (512, 32), generator=g, device="cuda").float()).repeat_interleave(32, 1)
    x[3, 64:96] = 0.0                       # all-zero block
    x[4, 0:32] = -0.0
    x[5, 7] = float("inf")
    x[6, 9] = 3e38
    x[7, 0:32] = 1e-41                      # denormal amax
    x[8, 3] = float("nan")
    x[9, 40] = float("-inf")
    codes, scales = rk.mx_quantize(x, fmt)
    oc, os_ = oracle.quantize(np_(x), fmt)
    assert np.array_equal(np_(codes), oc)
    assert np.array_equal(np_(scales), os_)


def test_quantize_exhaustive_bf16_inputs():
    """Every finite bf16 pattern as an input element (the reference validates its fp6 encoder the same way,
    kernels/flash_attention_mx_fp6/README.md:14-18), in blocks whose scale is pinned to 2^0."""
    bits = np.arange(65536, dtype=np.uint32)
    vals = (bits << 16).view(np.float32)
    keep = np.isfinite(vals) & (np.abs(vals) <= 448.0)
    vals = vals[keep]
    x = np.zeros((vals.size, 32), np.float32)
    x[:, 0] = vals
    x[:, 1] = 448.0
    codes, scales = rk.mx_quantize(torch.from_numpy(x).cuda())
    oc, os_ = oracle.quantize(x)
    assert np.array_equal(np_(codes), oc) and np.array_equal(np_(scales), os_)


@pytest.mark.parametrize("fmt", [rk.E5M2, rk.E3M2, rk.E2M1])
def test_quantize_keys_other_formats_bit_exact(fmt):
    """Blocks of 32 along the keys (the V layout the attention kernels take as it lies) in the non-default formats,
    the 4-bit one included, ragged row count."""
    g = torch.Generator(device="cuda").manual_seed(50 + fmt)
    x = torch.randn(2, 150, 128, generator=g, device="cuda") * 2.0
    ck, sk = rk.mx_quantize_keys(x, fmt)
    for b in range(2):
        oc, os_ = oracle.quantize(np_(x[b]), fmt, axis=0)
        assert np.array_equal(np_(ck[b]), oc) and np.array_equal(np_(sk[b]), os_)


def test_quantize_keys_and_rebase_bit_exact():
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(3, 200, 128, generator=g, device="cuda") * 3.0       # ragged: 200 rows = 6 blocks + 8
    ck, sk = rk.mx_quantize_keys(x)
    for b in range(3):
        oc, os_ = oracle.quantize(np_(x[b]), axis=0)
        assert np.array_equal(np_(ck[b]), oc) and np.array_equal(np_(sk[b]), os_)
    c, s = rk.mx_quantize(x)
    rc, rs = rk.mx_rebase_v(c, s)
    for b in range(3):
        oc, os_ = oracle.rebase_v(np_(c[b]), np_(s[b]))
        assert np.array_equal(np_(rc[b]), oc) and np.array_equal(np_(rs[b]), os_)


@pytest.mark.parametrize("fmt", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("S,d", [(32 * 7 + 5, 256), (96, 64), (40, 128), (32, 32)])
def test_rebase_bit_exact_on_adversarial_codes(S, d, fmt):
    """Every branch of the integer re-blocking, for all five element formats: random raw codes (zeros, subnormals,
    both signs; the E4M3 NaN encodings replaced) under scale codes that vary row to row by up to 2^24, extreme
    scale codes that must take the generic path, all-zero columns, ragged tails, and widths where a warp spans
    several key blocks."""
    rng = np.random.default_rng(11 + fmt)
    nb = d // 32
    nbits = 8 if fmt < 2 else 6
    sign, mant_bits = 1 << (nbits - 1), (3 if fmt in (0, 2) else 2)
    codes = rng.integers(0, 1 << nbits, size=(4, S, d), dtype=np.uint8)
    if fmt == 0:
        codes[(codes & 0x7F) == 0x7F] = 0x7E
    codes[0, :, 0:4] = 0                                   # all-zero columns
    codes[0, :, 4:8] = sign                                # all negative zero
    codes[0, :, 9] = 0                                     # a zero column beside ordinary ones
    codes[1, :, :] &= sign | ((1 << mant_bits) - 1)        # a slice of subnormals and zeros only
    scales = rng.integers(115, 140, size=(4, S, nb), dtype=np.uint8)
    scales[2] = rng.integers(100, 124, size=(S, nb), dtype=np.uint8)
    scales[3, :, 0] = rng.integers(0, 256, size=S, dtype=np.uint8)       # extreme scale codes: generic path
    if nb > 2:
        scales[3, :, 1] = rng.integers(236, 246, size=S, dtype=np.uint8)
        scales[3, :, 2] = rng.integers(4, 40, size=S, dtype=np.uint8)
    scales[3][scales[3] == 255] = 254
    c = torch.from_numpy(codes).cuda()
    s = torch.from_numpy(scales).cuda()
    rc, rs = rk.mx_rebase_v(c, s, fmt)
    for b in range(4):
        oc, os_ = oracle.rebase_v(codes[b], scales[b], fmt)
        assert np.array_equal(np_(rs[b]), os_), f"scales differ in slice {b}"
        assert np.array_equal(np_(rc[b]), oc), f"codes differ in slice {b}"


def test_rebase_is_nearly_lossless():
    """Re-blocking V along the keys changes the decoded values only where an element sits more than 2^14 below
    its new block's amax."""
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(1, 4096, 128, generator=g, device="cuda")
    c, s = rk.mx_quantize(x)
    rc, rs = rk.mx_rebase_v(c, s)
    a = oracle.dequant(np_(c[0]), np_(s[0]))
    b = oracle.dequant(np_(rc[0]), np_(rs[0]), axis=0)
    assert np.linalg.norm(a - b) / np.linalg.norm(a) < 1e-5


def test_quantize_full_size_idempotent():
    """At the benchmark's tensor size: dequant(quantize(dequant(quantize(x)))) == dequant(quantize(x)) -- every
    decoded value is exactly representable again (a size-independent property checked without the CPU oracle).
    Codes may differ: a block whose amax rounded down can pick a smaller scale the second time."""
    n_rows, d = 8 * 16 * 4096 // 8, 128          # one eighth of the B8 H16 S4096 d128 tensor
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(n_rows, d, generator=g, device="cuda")
    lut = torch.tensor([oracle.lib().rko_decode_elem(i, 0) for i in range(256)], device="cuda")

    def deq(c, s):
        return lut[c.long()] * torch.exp2(s.float() - 127.0).repeat_interleave(32, 1)

    c1, s1 = rk.mx_quantize(x)
    d1 = deq(c1, s1)
    c2, s2 = rk.mx_quantize(d1)
    assert torch.equal(d1, deq(c2, s2))
    assert (s2 <= s1).all()


@pytest.mark.parametrize("fmt", [0, 1, 2, 3, 4])
def test_rope_quantize_bit_exact_against_reference_rope_golden(fmt):
    """The fused RoPE + quantizer: codes and scales equal oracle.quantize of the reference's own rope_apply output
    (tests/golden/rope_vectors.npz, made by lib/golden/golden.py), for head dims 64 / 128 / 256 and every format."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_vectors.npz"))
    for d in (64, 128, 256):
        x, c, s, y = z[f"x{d}"], z[f"cos{d}"], z[f"sin{d}"], z[f"y{d}"]
        codes, scales = rk.rope_mx_quantize(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), torch.from_numpy(s).cuda(), fmt=fmt)
        oc, os_ = oracle.quantize(y, fmt=fmt)
        assert np.array_equal(np_(codes), oc) and np.array_equal(np_(scales), os_), (fmt, d)


def test_rope_quantize_positions_and_layouts():
    """[batch][head][S][d] input with an offset into the caches, and an explicit per-row position list; compared
    with the oracle's rope + quantize.  Includes a row of zeros, a NaN and an inf (integer encoder path)."""
    rng = np.random.default_rng(5)
    B, H, S, d, npos = 2, 3, 50, 128, 80
    x = rng.standard_normal((B, H, S, d)).astype(np.float32)
    x[0, 0, 3] = 0.0
    x[1, 2, 7, 5] = np.nan
    x[1, 1, 9, 100] = np.inf
    ang = np.arange(npos)[:, None] * (10000.0 ** (-(np.arange(d // 2) * 2.0 / d)))[None, :]
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    xt, ct, st = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), torch.from_numpy(s).cuda()
    codes, scales = rk.rope_mx_quantize(xt, ct, st, pos0=11)
    pos = np.tile(np.arange(11, 11 + S, dtype=np.int32), B * H)
    y = oracle.rope(x.reshape(-1, d), pos, c, s)
    oc, os_ = oracle.quantize(y)
    assert np.array_equal(np_(codes).reshape(-1, d), oc) and np.array_equal(np_(scales).reshape(-1, d // 32), os_)
    pos2 = rng.integers(0, npos, size=B * H * S).astype(np.int32)
    codes, scales = rk.rope_mx_quantize(xt, ct, st, pos=torch.from_numpy(pos2).cuda())
    y = oracle.rope(x.reshape(-1, d), pos2, c, s)
    oc, os_ = oracle.quantize(y)
    assert np.array_equal(np_(codes).reshape(-1, d), oc) and np.array_equal(np_(scales).reshape(-1, d // 32), os_)


@pytest.mark.parametrize("fmt", [0, 1, 2, 3])
def test_bf16_input_quantizer_equals_fp32_path(fmt):
    """A bf16 tensor quantizes to exactly what its fp32 widening does (and to what the oracle says)."""
    g = torch.Generator(device="cuda").manual_seed(70 + fmt)
    x = (torch.randn(333, 256, generator=g, device="cuda") * torch.exp2(torch.randint(-20, 20, (333, 1), generator=g, device="cuda").float())).bfloat16()
    x[5] = 0
    x[7, 3] = float("inf")
    cb, sb = rk.mx_quantize(x, fmt)
    cf, sf = rk.mx_quantize(x.float(), fmt)
    assert torch.equal(cb, cf) and torch.equal(sb, sf)
    oc, os_ = oracle.quantize(np_(x.float()), fmt=fmt)
    assert np.array_equal(np_(cb), oc) and np.array_equal(np_(sb), os_)
