"""The CPU oracle against every frozen value the reference's tests hold for the encode path."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.golden import reference_goldens as G


def _bits(a):
    return [int(v) for v in np.asarray(a, dtype=np.float32).view(np.uint32).ravel()]


def test_rotation_golden_dim8():
    x = np.array([i - 3.5 for i in range(8)], dtype=np.float32)
    assert _bits(O.rotate_rows(x)) == G.ROTATION_DIM8


def test_rotation_golden_dim24():
    x = np.array([((i * 7) % 11) - 5.0 for i in range(24)], dtype=np.float32)
    assert _bits(O.rotate_rows(x)) == G.ROTATION_DIM24


def test_rotation_golden_dim64():
    x = np.array([((i * 13) % 29) - 14.0 for i in range(64)], dtype=np.float32)
    assert _bits(O.rotate_rows(x)) == G.ROTATION_DIM64


def test_rotation_golden_dim128_fold():
    e = np.zeros(128, dtype=np.float32)
    e[0] = 1.0
    bits = _bits(O.rotate_rows(e))
    fold = 0
    for b in bits:
        fold = (((fold << 1) & 0xFFFFFFFF) | (fold >> 31)) ^ b
    assert (fold, *bits[:4]) == G.ROTATION_DIM128_FOLD


def test_block_sizes():
    # turbovec/src/rotation.rs:1045-1053
    import ctypes
    lib = O._lib()
    for dim, want in [(8, 8), (200, 8), (1000, 8), (768, 256), (1536, 512), (3072, 1024), (1024, 1024), (16384, 16384)]:
        assert lib.tvo_block_size(ctypes.c_int(dim)) == want


@pytest.mark.parametrize("row", G.ENCODE_FINGERPRINT, ids=lambda r: f"d{r[0]}b{r[1]}")
def test_encode_fingerprint(row):
    dim, bits, g_bnd, g_cent, g_cal, g_codes, g_scales, _g_file = row
    bnd, cent = O.codebook(bits, dim)
    assert O.fnv1a(bnd) == g_bnd
    assert O.fnv1a(cent) == g_cent
    x = O.lcg_vectors(2000, dim, G.cell_seed(dim, bits))
    shift, scale = O.fit_calibration(x, bits)
    assert O.fnv1a(np.concatenate([shift, scale])) == g_cal
    enc = O.encode(x, bits, shift, scale)
    assert O.fnv1a(enc["packed"]) == g_codes
    assert O.fnv1a(enc["scales"]) == g_scales


def test_codebook_midpoints_and_order():
    # turbovec/src/codebook.rs:174-207
    for bits in (2, 3, 4):
        for dim in (8, 128, 200, 768, 1000, 1024, 1536, 3072):
            bnd, cent = O.codebook(bits, dim)
            assert np.array_equal(bnd, (cent[:-1] + cent[1:]) * np.float32(0.5))
            assert np.all(np.diff(bnd) > 0) and np.all(np.diff(cent) > 0)


def test_beta_cdf_matches_scipy():
    from scipy.special import betainc
    for a in (3.5, 99.5, 383.5, 767.5, 1535.5, 8191.5):
        for x in (0.01, 0.3, 0.45, 0.49, 0.5, 0.51, 0.55, 0.7, 0.99):
            want = float(betainc(a, a, x))
            got = O.beta_cdf(a, a, x)
            assert got == pytest.approx(want, rel=1e-10, abs=1e-300)


def test_norm_chain_order():
    # turbovec/src/encode.rs:1798-1814: the 8-chain order is observable in f32.
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(1536) * 10 ** rng.uniform(-3, 3, 1536)).astype(np.float32)
    c = np.zeros(8, dtype=np.float32)
    for j, v in enumerate(x):
        c[j % 8] = np.float32(c[j % 8] + np.float32(v * v))
    want = np.sqrt(np.float32(np.float32(np.float32(c[0] + c[1]) + np.float32(c[2] + c[3]))
                              + np.float32(np.float32(c[4] + c[5]) + np.float32(c[6] + c[7]))))
    assert O.norm(x) == want


def test_blocked_layout_fixture():
    # turbovec/src/pack.rs:964-1008: 33 vectors, dim 64, 4-bit; byte (block, g, lane) holds
    # coordinate 2g in the high nibble and 2g+1 in the low nibble; padding lanes are zero.
    n, dim, bits = 33, 64, 4
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 16, size=(n, dim), dtype=np.uint8)
    packed = np.zeros((n, bits * dim // 8), dtype=np.uint8)
    for v in range(n):
        for j in range(dim):
            for p in range(bits):
                packed[v, p * (dim // 8) + j // 8] |= ((codes[v, j] >> p) & 1) << (7 - j % 8)
    blocked = O.packed_to_blocked(packed, bits, dim)
    ng = dim // 2
    assert blocked.size == 2 * ng * 32
    for v in range(n):
        b, lane = divmod(v, 32)
        for g in range(ng):
            assert blocked[(b * ng + g) * 32 + lane] == (codes[v, 2 * g] << 4) | codes[v, 2 * g + 1]
    for lane in range(1, 32):
        assert not blocked[ng * 32 + lane::32][: ng].any()
    assert np.array_equal(O.blocked_to_packed(blocked, n, bits, dim), packed)


@pytest.mark.parametrize("bits,dim", [(2, 200), (3, 600), (4, 1000)])
def test_layout_roundtrip(bits, dim):
    x = O.lcg_vectors(70, dim, 99)
    enc = O.encode(x, bits, want_codes=True)
    blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    assert np.array_equal(O.blocked_to_packed(blocked, 70, bits, dim), enc["packed"])
    # group byte vs per-coordinate codes
    cpb = 8 // bits
    field = 4 if bits == 3 else bits
    ng = dim // cpb
    v = 37
    for g in range(ng):
        byte = 0
        for kk in range(cpb):
            byte |= int(enc["codes"][v, g * cpb + kk]) << ((cpb - 1 - kk) * field)
        assert blocked[((v // 32) * ng + g) * 32 + v % 32] == byte


def test_zero_norm_row_scale_zero():
    # turbovec/tests/input_validation.rs:367-389
    x = np.zeros((3, 64), dtype=np.float32)
    x[1] = 1e-23
    x[2, 0] = 1.0
    enc = O.encode(x, 4)
    assert enc["scales"][0] == 0.0 and enc["scales"][1] == 0.0 and enc["scales"][2] > 0


def test_first_invalid():
    x = np.ones((4, 8), dtype=np.float32)
    assert O.first_invalid(x) == -1
    x[2, 3] = np.nan
    x[3, 0] = np.inf
    assert O.first_invalid(x) == 2 * 8 + 3
    x[0, 7] = 1e16
    assert O.first_invalid(x) == 7
