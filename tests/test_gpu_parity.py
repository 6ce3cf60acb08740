"""CUDA path vs the CPU oracle through the C ABI (via the ctypes classes): bit-exact codes, scales and
rotation; scores and id lists identical under the oracle's own arithmetic."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.golden import reference_goldens as G
from tests.util import anisotropic, assert_topk_equal, clustered

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    import turbovec_b200
    return turbovec_b200


# ---------------------------------------------------------------- rotation
@pytest.mark.parametrize("dim", [8, 16, 24, 64, 128, 200, 256, 768, 1000, 1536, 2048, 3072, 4096, 6144])
def test_rotation_bit_exact(T, dim):
    rng = np.random.default_rng(dim)
    x = (rng.standard_normal((5, dim)) * 10 ** rng.uniform(-2, 2, (5, 1))).astype(np.float32)
    idx = T.TurboQuantIndex(dim, 4)
    idx.prepare()
    got = idx.rotate(x)
    want = O.rotate_rows(x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_rotation_goldens_on_device(T):
    for dim, inp, gold in [(8, [i - 3.5 for i in range(8)], G.ROTATION_DIM8),
                           (24, [((i * 7) % 11) - 5.0 for i in range(24)], G.ROTATION_DIM24),
                           (64, [((i * 13) % 29) - 14.0 for i in range(64)], G.ROTATION_DIM64)]:
        idx = T.TurboQuantIndex(dim, 2)
        idx.prepare()
        out = idx.rotate(np.array([inp], dtype=np.float32))
        assert [int(v) for v in out.view(np.uint32)[0]] == gold


# ---------------------------------------------------------------- ingest
@pytest.mark.parametrize("row", G.ENCODE_FINGERPRINT, ids=lambda r: f"d{r[0]}b{r[1]}")
def test_encode_fingerprint_on_device(T, row):
    """The reference's frozen encode fingerprint reproduced by the ingest kernel (calibrated encode)."""
    dim, bits, g_bnd, g_cent, _g_cal, g_codes, g_scales, _ = row
    x = O.lcg_vectors(2000, dim, G.cell_seed(dim, bits))
    shift, scale = O.fit_calibration(x, bits)      # the fit itself is host-side and checked in the oracle tests
    idx = T.TurboQuantIndex(dim, bits)
    idx.set_calibration(shift, scale)
    idx.add(x)
    bnd, cent = idx.codebook()
    assert O.fnv1a(bnd) == g_bnd and O.fnv1a(cent) == g_cent
    assert O.fnv1a(idx.packed_codes()) == g_codes
    assert O.fnv1a(idx.scales()) == g_scales


@pytest.mark.parametrize("dim,bits", [(1536, 4), (1536, 2), (3072, 2), (200, 4), (200, 2), (600, 3), (64, 4), (4096, 4)])
def test_ingest_matches_oracle(T, dim, bits):
    n = 1000 + 37
    x = anisotropic(n, dim, seed=dim + bits) if dim != 200 else clustered(n, dim, seed=3)
    enc = O.encode(x, bits)
    want_blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    idx = T.TurboQuantIndex(dim, bits)
    # ragged batches: partial head blocks, single rows, block-aligned runs
    cuts = [0, 1, 5, 32, 33, 100, 517, 1000, n]
    for a, b in zip(cuts[:-1], cuts[1:]):
        idx.add(x[a:b])
    assert len(idx) == n
    got = idx.codes_blocked_seq()
    mism = int((got != want_blocked).sum())
    assert mism == 0, f"{mism} code bytes differ"
    assert np.array_equal(idx.scales().view(np.uint32), enc["scales"].view(np.uint32))
    assert np.array_equal(idx.packed_codes(), enc["packed"])


def test_ingest_zero_and_tiny_rows(T):
    x = anisotropic(40, 256, seed=1)
    x[3] = 0.0
    x[17] = 1e-23
    enc = O.encode(x, 4)
    idx = T.TurboQuantIndex(256, 4)
    idx.add(x)
    s = idx.scales()
    assert s[3] == 0.0 and s[17] == 0.0
    assert np.array_equal(s.view(np.uint32), enc["scales"].view(np.uint32))
    assert np.array_equal(idx.packed_codes(), enc["packed"])


@pytest.mark.parametrize("dim,bits", [(128, 4), (256, 2), (384, 3), (512, 4), (768, 4), (1024, 2), (1536, 3), (1536, 4),
                                      (2048, 4), (2048, 2), (3072, 2), (3072, 4)])
def test_pipelined_ingest_matches_oracle_and_block_kernel(T, dim, bits):
    """Whole code blocks go through the pipelined kernel, a partial head block through the block-at-a-time
    one; both must produce the oracle's bytes and scales, and so must the block-at-a-time kernel alone and
    the pipelined kernel with its certified parallel sum switched off."""
    n = 1500 + 13
    x = anisotropic(n, dim, seed=7 * dim + bits)
    x[5] = 0.0
    x[700] = 1e-23
    enc = O.encode(x, bits)
    want_blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    a = T.TurboQuantIndex(dim, bits)
    assert a.get_option(T.OPT_INGEST_PIPELINE) == 1
    a.add(x[:3])            # leaves a partly filled block
    a.add(x[3:1000])        # head rows complete it, the rest are whole blocks plus a ragged tail
    a.add(x[1000:])
    b = T.TurboQuantIndex(dim, bits)
    b.set_option(T.OPT_INGEST_PIPELINE, 0)
    b.add(x)
    c = T.TurboQuantIndex(dim, bits)
    c.set_option(T.OPT_INGEST_PIPELINE, 2)      # every reconstruction sum walks the sequential chains
    c.add(x)
    for idx in (a, b, c):
        assert np.array_equal(idx.codes_blocked_seq(), want_blocked)
        assert np.array_equal(idx.scales().view(np.uint32), enc["scales"].view(np.uint32))
        assert np.array_equal(idx.packed_codes(), enc["packed"])


@pytest.mark.parametrize("dim,bits", [(256, 4), (768, 2), (1024, 3), (1536, 4), (3072, 2)])
def test_pipelined_ingest_with_calibration(T, dim, bits):
    """A committed TQ+ pair: the pipelined kernel (with its certified sum and with the sequential chains
    forced) and the block-at-a-time kernel all produce the oracle's calibrated codes and scales."""
    n = 1200 + 9
    x = anisotropic(n, dim, seed=5 * dim + bits) * np.float32(2.0)
    x[:, ::9] *= np.float32(3.0)
    sh, sc = O.fit_calibration(x[:700], bits)
    enc = O.encode(x, bits, sh, sc)
    want_blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    for mode in (1, 0, 2):
        idx = T.TurboQuantIndex(dim, bits)
        idx.set_option(T.OPT_INGEST_PIPELINE, mode)
        idx.calibrate(x[:700])
        idx.add(x[:3])
        idx.add(x[3:])
        assert np.array_equal(idx.codes_blocked_seq(), want_blocked), mode
        assert np.array_equal(idx.scales().view(np.uint32), enc["scales"].view(np.uint32)), mode


def test_pipelined_ingest_reports_first_invalid_coordinate(T):
    x = anisotropic(400, 256, seed=12)
    idx = T.TurboQuantIndex(256, 4)
    bad = x.copy()
    bad[333, 200] = -np.inf
    bad[150, 9] = 2e16
    bad[150, 77] = np.nan
    with pytest.raises(ValueError, match="vector 150 coordinate 9"):
        idx.add(bad)
    assert len(idx) == 0
    idx.add(x)
    enc = O.encode(x, 4)
    assert np.array_equal(idx.codes_blocked_seq(), O.packed_to_blocked(enc["packed"], 4, 256))
    assert np.array_equal(idx.scales().view(np.uint32), enc["scales"].view(np.uint32))


def test_add_rejects_invalid_and_leaves_index_unchanged(T):
    x = anisotropic(70, 128, seed=2)
    idx = T.TurboQuantIndex(128, 4)
    idx.add(x[:40])
    before_codes, before_scales = idx.codes_blocked_seq(), idx.scales()
    bad = x[40:].copy()
    bad[7, 5] = np.nan
    bad[9, 0] = np.inf
    with pytest.raises(ValueError, match="vector 7 coordinate 5"):
        idx.add(bad)
    assert len(idx) == 40
    assert np.array_equal(idx.codes_blocked_seq(), before_codes)
    assert np.array_equal(idx.scales(), before_scales)
    idx.add(x[40:])
    enc = O.encode(x, 4)
    assert np.array_equal(idx.codes_blocked_seq(), O.packed_to_blocked(enc["packed"], 4, 128))


@pytest.mark.parametrize("row", G.ENCODE_FINGERPRINT, ids=lambda r: f"d{r[0]}b{r[1]}")
def test_calibrate_then_add_reproduces_the_frozen_fingerprint(T, row):
    """calibrate(sample) + add(sample), the reference's own fixture: calibration, codes and scales hashes."""
    dim, bits, _b, _c, g_cal, g_codes, g_scales, _ = row
    x = O.lcg_vectors(2000, dim, G.cell_seed(dim, bits))
    idx = T.TurboQuantIndex(dim, bits)
    assert idx.calibration_state == "uncalibrated"
    idx.calibrate(x)
    assert idx.calibration_state == "calibrated"
    shift, scale = idx.calibration()
    assert O.fnv1a(np.concatenate([shift, scale])) == g_cal
    idx.add(x)
    assert O.fnv1a(idx.packed_codes()) == g_codes
    assert O.fnv1a(idx.scales()) == g_scales


def test_calibrated_search_matches_oracle(T):
    dim, bits, n = 512, 4, 3000
    x = anisotropic(n, dim, seed=51) * np.float32(3.0)
    x[:, ::7] *= np.float32(2.5)                       # heavy coordinates so the fit is far from identity
    q = anisotropic(9, dim, seed=51, offset=3)
    shift, scale = O.fit_calibration(x, bits)
    for mode_bits in (4, 2):
        sh, sc = O.fit_calibration(x, mode_bits)
        idx = T.TurboQuantIndex(dim, mode_bits)
        idx.calibrate(x)
        idx.add(x)
        enc = O.encode(x, mode_bits, sh, sc)
        blocked = O.packed_to_blocked(enc["packed"], mode_bits, dim)
        assert np.array_equal(idx.codes_blocked_seq(), blocked)
        s, i = idx.search(q, 10)
        rs, ri = O.search(q, blocked, enc["scales"], n, dim, mode_bits, 10, shift=sh, scale=sc)
        assert np.array_equal(i, ri) and np.array_equal(s, rs)


@pytest.mark.parametrize("dim,bits", [(512, 4), (256, 2), (384, 3), (1536, 4)])
def test_calibrate_on_populated_index_reencodes_stored_rows(T, dim, bits):
    """calibrate() on an index that already holds rows re-encodes every stored row from its own codes under
    the new pair (the reference's refit): first from the identity pair, then from a committed pair."""
    n = 1000 + 21
    x = anisotropic(n, dim, seed=57) * np.float32(2.0)
    x[:, ::5] *= np.float32(3.0)
    x[11] = 0.0                                          # a degenerate row stays degenerate
    idx = T.TurboQuantIndex(dim, bits)
    idx.add(x)
    enc = O.encode(x, bits, want_codes=True)
    sample1 = x[:600]
    sh1, sc1 = O.fit_calibration(sample1, bits)
    idx.calibrate(sample1)
    got_sh, got_sc = idx.calibration()
    assert np.array_equal(got_sh, sh1) and np.array_equal(got_sc, sc1)
    codes1, scales1 = O.reencode(enc["codes"], enc["scales"], bits, None, None, sh1, sc1)
    want1 = O.packed_to_blocked(_pack_bitplanes(codes1, bits), bits, dim)
    assert np.array_equal(idx.codes_blocked_seq(), want1)
    assert np.array_equal(idx.scales().view(np.uint32), scales1.view(np.uint32))
    assert idx.scales()[11] == 0.0
    # second refit, now from a committed pair
    sample2 = x[300:] * np.float32(1.5)
    sh2, sc2 = O.fit_calibration(sample2, bits)
    idx.calibrate(sample2)
    codes2, scales2 = O.reencode(codes1, scales1, bits, sh1, sc1, sh2, sc2)
    assert np.array_equal(idx.codes_blocked_seq(), O.packed_to_blocked(_pack_bitplanes(codes2, bits), bits, dim))
    assert np.array_equal(idx.scales().view(np.uint32), scales2.view(np.uint32))
    # rows added afterwards are encoded under the new pair, and searches see one consistent index
    y = anisotropic(100, dim, seed=58)
    idx.add(y)
    enc_y = O.encode(y, bits, sh2, sc2, want_codes=True)
    all_codes = np.concatenate([codes2, enc_y["codes"]])
    all_scales = np.concatenate([scales2, enc_y["scales"]])
    blocked = O.packed_to_blocked(_pack_bitplanes(all_codes, bits), bits, dim)
    assert np.array_equal(idx.codes_blocked_seq(), blocked)
    q = anisotropic(6, dim, seed=59)
    s, i = idx.search(q, 10)
    rs, ri = O.search(q, blocked, all_scales, n + 100, dim, bits, 10, shift=sh2, scale=sc2)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)


def test_refit_under_the_committed_pair_keeps_the_codes(T):
    """The property the reference states for its refit (lib.rs:2776-2782): re-quantising an exact centroid
    value lands in its own cell, so calibrating again with the sample that produced the committed pair
    reproduces every stored code."""
    dim, bits, n = 768, 4, 700
    x = anisotropic(n, dim, seed=63) * np.float32(2.0)
    idx = T.TurboQuantIndex(dim, bits)
    idx.calibrate(x)
    idx.add(x)
    before = idx.codes_blocked_seq()
    idx.calibrate(x)
    assert np.array_equal(idx.codes_blocked_seq(), before)
    assert np.allclose(idx.scales(), O.encode(x, bits, *O.fit_calibration(x, bits))["scales"], rtol=1e-5)


def _pack_bitplanes(codes, bits):
    """[n, dim] codes -> the reference's bit-plane rows (encode.rs:1464-1470)."""
    n, dim = codes.shape
    out = np.zeros((n, bits * dim // 8), dtype=np.uint8)
    c = codes.reshape(n, dim // 8, 8)
    for p in range(bits):
        plane = np.zeros((n, dim // 8), dtype=np.uint8)
        for k in range(8):
            plane |= (((c[:, :, k] >> p) & 1) << (7 - k)).astype(np.uint8)
        out[:, p * (dim // 8):(p + 1) * (dim // 8)] = plane
    return out


# ---------------------------------------------------------------- search
def _build(T, x, bits, kind="pos", ids=None):
    dim = x.shape[1]
    if kind == "pos":
        idx = T.TurboQuantIndex(dim, bits)
        idx.add(x)
    else:
        idx = T.IdMapIndex(dim, bits)
        idx.add_with_ids(x, ids)
    return idx


def _oracle_search(x, q, bits, k, mask=None, mode=O.MODE_AUTO):
    n, dim = x.shape
    enc = O.encode(x, bits)
    blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    words = None if mask is None else O.pack_mask(mask)
    return O.search(q, blocked, enc["scales"], n, dim, bits, k, mask_words=words, mode=mode)


@pytest.mark.parametrize("dim,bits,n,nq", [
    (1536, 4, 3000, 1), (1536, 4, 3000, 7), (1536, 4, 5003, 70), (256, 4, 4100, 33), (200, 4, 2000, 5),
    (1536, 2, 3000, 1), (1536, 2, 3000, 9), (3072, 2, 1500, 6), (200, 2, 2500, 6), (600, 3, 2000, 5), (1024, 3, 1500, 3),
])
def test_search_matches_oracle(T, dim, bits, n, nq):
    x = anisotropic(n, dim, seed=11)
    q = anisotropic(nq, dim, seed=11, offset=1000)
    idx = _build(T, x, bits)
    for k in (1, 10, 100):
        s, i = idx.search(q, k)
        rs, ri = _oracle_search(x, q, bits, k)
        assert s.shape == (nq, min(k, n))
        assert np.array_equal(i, ri), f"k={k}: id lists differ"
        assert np.array_equal(s, rs), f"k={k}: scores differ"


@pytest.mark.parametrize("dim,bits,n,nq", [(1536, 4, 5003, 70), (256, 4, 4100, 50), (1536, 2, 3000, 9), (1024, 3, 1500, 12)])
def test_search_without_tensor_memory_path_matches_oracle(T, dim, bits, n, nq):
    """The tensor-memory scan switched off: every batch size runs on the mma.sync / CUDA-core scans (passes of
    up to 64 and 4 queries), which the default switch points would only use for small batches."""
    x = anisotropic(n, dim, seed=13)
    q = anisotropic(nq, dim, seed=13, offset=1000)
    idx = _build(T, x, bits)
    assert idx.get_option(T.OPT_MMA_MIN_BATCH) == -1
    idx.set_option(T.OPT_MMA_MIN_BATCH, 0)
    for k in (1, 10):
        s, i = idx.search(q, k)
        rs, ri = _oracle_search(x, q, bits, k)
        assert np.array_equal(i, ri), f"k={k}: id lists differ"
        assert np.array_equal(s, rs), f"k={k}: scores differ"


def test_search_large_n_chunk_schedule(T):
    """Enough vectors for several growing chunks, and the bounded recovery schedule gives the same answer."""
    n, dim, nq = 200_000, 64, 12
    x = anisotropic(n, dim, seed=5)
    q = anisotropic(nq, dim, seed=5, offset=9)
    idx = _build(T, x, 4)
    s, i = idx.search(q, 10)
    rs, ri = _oracle_search(x, q, 4, 10)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)
    idx.set_option(T.OPT_FORCE_CAREFUL, 1)
    s2, i2 = idx.search(q, 10)
    assert np.array_equal(i2, ri) and np.array_equal(s2, rs)


def test_search_adversarial_order_overflows_and_recovers(T):
    """Rows sorted by increasing similarity to the query overflow the candidate buffer of the growing
    schedule; the bounded schedule must then return the exact answer."""
    n, dim = 150_000, 64
    x = anisotropic(n, dim, seed=8)
    q = anisotropic(1, dim, seed=8, offset=3)
    order = np.argsort(x @ q[0])
    x = np.ascontiguousarray(x[order])
    idx = _build(T, x, 4)
    s, i = idx.search(q, 10)
    rs, ri = _oracle_search(x, q, 4, 10)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)


@pytest.mark.parametrize("bits", [4, 2])
def test_filtered_search(T, bits):
    n, dim, nq = 6000, 256, 9
    x = anisotropic(n, dim, seed=21)
    q = anisotropic(nq, dim, seed=21, offset=5)
    idx = _build(T, x, bits)
    rng = np.random.default_rng(0)
    for sel in (0.001, 0.01, 0.1, 0.5, 1.0):
        mask = rng.random(n) < sel
        if not mask.any():
            mask[123] = True
        for k in (10, 100):
            s, i = idx.search(q, k, mask=mask)
            rs, ri = _oracle_search(x, q, bits, k, mask=mask)
            assert s.shape == (nq, min(k, int(mask.sum())))
            assert np.array_equal(i, ri) and np.array_equal(s, rs)
            assert mask[i].all()
            # the packed-word entry point agrees
            s2, i2 = idx.search_mask_words(q, k, O.pack_mask(mask))
            assert np.array_equal(i2, ri) and np.array_equal(s2, rs)
    # contiguous range and all-false
    mask = np.zeros(n, bool)
    mask[1000:1007] = True
    s, i = idx.search(q, 10, mask=mask)
    assert s.shape == (nq, 7) and set(i[0]) == set(range(1000, 1007))
    s, i = idx.search(q, 10, mask=np.zeros(n, bool))
    assert s.shape == (nq, 0) and i.shape == (nq, 0)


def test_search_edge_cases(T):
    dim = 128
    x = anisotropic(100, dim, seed=4)
    idx = T.TurboQuantIndex(dim, 4)
    q = anisotropic(3, dim, seed=4, offset=2)
    s, i = idx.search(q, 5)                       # empty index
    assert s.shape == (3, 0)
    idx.add(x)
    s, i = idx.search(q, 1000)                    # k clamps to n
    assert s.shape == (3, 100)
    assert np.all(np.diff(s, axis=1) <= 0)
    s, i = idx.search(np.zeros((0, dim), np.float32), 5)
    assert s.shape == (0, 5)
    # zero query: all scores tie, slots 0..k-1 by the tie rule
    s, i = idx.search(np.zeros((1, dim), np.float32), 7)
    assert list(i[0]) == list(range(7)) and np.all(np.isfinite(s))
    with pytest.raises(ValueError):
        idx.search(np.full((1, dim), np.nan, np.float32), 3)
    with pytest.raises(ValueError):
        idx.search(q[:, :64].copy(), 3)
    with pytest.raises(ValueError):
        idx.search(q, 3, mask=np.ones(99, bool))
    lazy = T.TurboQuantIndex(None, 4)
    s, i = lazy.search(q, 3)
    assert s.shape == (3, 0)


def test_duplicate_vectors_tie_by_slot(T):
    dim = 128
    base = anisotropic(10, dim, seed=6)
    x = np.ascontiguousarray(np.tile(base, (20, 1)))   # every vector 20 times
    idx = _build(T, x, 4)
    q = base[:2].copy()
    s, i = idx.search(q, 25)
    rs, ri = _oracle_search(x, q, 4, 25)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)


def test_batch_equals_single(T):
    dim, n = 512, 3000
    x = anisotropic(n, dim, seed=9)
    q = anisotropic(19, dim, seed=9, offset=1)
    idx = _build(T, x, 4)
    s, i = idx.search(q, 10)
    for j in range(19):
        s1, i1 = idx.search(q[j:j + 1], 10)
        assert np.array_equal(i1[0], i[j]) and np.array_equal(s1[0], s[j])


# ---------------------------------------------------------------- mutation and ids
def test_swap_remove(T):
    dim, n = 128, 70
    x = anisotropic(n, dim, seed=12)
    idx = _build(T, x, 4)
    keep = list(range(n))
    for victim in (5, 68, 0, 31, 32):
        moved = idx.swap_remove(victim)
        assert moved == len(keep) - 1
        keep[victim] = keep[-1]
        keep.pop()
        enc = O.encode(x[keep], 4)
        assert np.array_equal(idx.codes_blocked_seq(), O.packed_to_blocked(enc["packed"], 4, dim))
        assert np.array_equal(idx.scales(), enc["scales"])
    with pytest.raises(IndexError):
        idx.swap_remove(len(keep))


def test_idmap_semantics(T):
    dim, n = 128, 500
    x = anisotropic(n, dim, seed=14)
    ids = (np.random.default_rng(1).permutation(n) + 10**9).astype(np.uint64)
    idx = _build(T, x, 4, "idmap", ids)
    q = anisotropic(4, dim, seed=14, offset=8)
    s, got = idx.search(q, 10)
    rs, ri = _oracle_search(x, q, 4, 10)
    assert np.array_equal(got, ids[ri]) and np.array_equal(s, rs)
    allow = ids[::7].copy()
    mask = np.zeros(n, bool)
    mask[::7] = True
    s, got = idx.search(q, 10, allowlist=allow)
    rs, ri = _oracle_search(x, q, 4, 10, mask=mask)
    assert np.array_equal(got, ids[ri]) and np.array_equal(s, rs)
    # n_allowed < k
    s, got = idx.search(q, 10, allowlist=ids[:3].copy())
    assert s.shape == (4, 3) and set(got[0]) == set(ids[:3])
    with pytest.raises(KeyError):
        idx.search(q, 10, allowlist=np.array([5], np.uint64))
    with pytest.raises(ValueError):
        idx.search(q, 10, allowlist=np.array([], np.uint64))
    with pytest.raises(ValueError, match="already present"):
        idx.add_with_ids(x[:1], ids[:1].copy())
    with pytest.raises(ValueError, match="twice"):
        idx.add_with_ids(x[:2], np.array([1, 1], np.uint64))
    assert len(idx) == n
    # removal moves the last row into the hole
    assert idx.remove(int(ids[10])) is True
    assert idx.remove(int(ids[10])) is False
    assert int(ids[10]) not in idx and int(ids[-1]) in idx
    cur = list(ids)
    cur[10] = cur[-1]
    cur.pop()
    assert list(idx.ids()) == cur
    xs = x.copy()
    xs[10] = xs[-1]
    xs = xs[:-1]
    s, got = idx.search(q, 10)
    rs, ri = _oracle_search(xs, q, 4, 10)
    assert np.array_equal(got, np.array(cur, np.uint64)[ri]) and np.array_equal(s, rs)


def test_from_parts_roundtrip(T):
    dim, n = 256, 333
    x = anisotropic(n, dim, seed=15)
    a = _build(T, x, 2)
    b = T.TurboQuantIndex.from_parts(dim, 2, a.packed_codes(), a.scales())
    assert np.array_equal(a.codes_blocked_seq(), b.codes_blocked_seq())
    q = anisotropic(3, dim, seed=15, offset=1)
    sa, ia = a.search(q, 10)
    sb, ib = b.search(q, 10)
    assert np.array_equal(ia, ib) and np.array_equal(sa, sb)


def test_recall_at_10_matches_reference_floor(T):
    """recall@10 against exact fp32 inner products equals the oracle's (same codes, same arithmetic) and
    clears the floors of turbovec/tests/recall_sanity.rs:97-118 on clustered data."""
    n, dim, nq = 2000, 1536, 50
    x = clustered(n, dim, seed=77, n_clusters=50)
    q = clustered(nq, dim, seed=77, n_clusters=50, offset=4)
    truth = np.argsort(-(q @ x.T), axis=1)[:, :10]
    for bits, floor in ((4, 0.70), (3, 0.58), (2, 0.40)):
        idx = _build(T, x, bits)
        _, i = idx.search(q, 10)
        _, ri = _oracle_search(x, q, bits, 10)
        rec = np.mean([len(set(i[j]) & set(truth[j])) / 10 for j in range(nq)])
        rec_ref = np.mean([len(set(ri[j]) & set(truth[j])) / 10 for j in range(nq)])
        assert abs(rec - rec_ref) <= 0.002
        assert rec >= floor


# ---------------------------------------------------------------- tcgen05 / TMEM scan
@pytest.mark.parametrize("dim,n,nq", [(1536, 3000, 1), (1536, 5003, 70), (1536, 4100, 300), (256, 4100, 257), (200, 2000, 5),
                                      (64, 70000, 600)])
@pytest.mark.parametrize("tiles", [1, 2])
def test_tensor_memory_scan_matches_oracle(T, dim, n, nq, tiles):
    """The tcgen05 path (forced for every batch size, both work-item shapes) returns exactly what the oracle returns."""
    x = anisotropic(n, dim, seed=41)
    q = anisotropic(nq, dim, seed=41, offset=77)
    idx = _build(T, x, 4)
    idx.set_option(T.OPT_MMA_MIN_BATCH, 1)
    idx.set_option(T.OPT_TC_TILES, tiles)
    for k in (1, 10, 100):
        s, i = idx.search(q, k)
        rs, ri = _oracle_search(x, q, 4, k)
        assert np.array_equal(i, ri), f"k={k}: id lists differ"
        assert np.array_equal(s, rs), f"k={k}: scores differ"
    mask = np.random.default_rng(3).random(n) < 0.05
    s, i = idx.search(q, 10, mask=mask)
    rs, ri = _oracle_search(x, q, 4, 10, mask=mask)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)


@pytest.mark.parametrize("dim,bits,n,nq", [(1536, 2, 3000, 9), (3072, 2, 1500, 300), (1024, 3, 1500, 70), (256, 4, 4100, 33),
                                           (64, 2, 40000, 513)])
def test_tensor_memory_lut_scan_matches_oracle(T, dim, bits, n, nq):
    """The u8-LUT scan as a one-hot int8 contraction on tcgen05 returns exactly the oracle's LUT results."""
    x = anisotropic(n, dim, seed=43)
    q = anisotropic(nq, dim, seed=43, offset=7)
    idx = _build(T, x, bits)
    idx.set_option(T.OPT_SCORE_MODE, T.SCORE_LUT_MULADD)
    idx.set_option(T.OPT_MMA_MIN_BATCH, 1)
    for k in (1, 10, 100):
        s, i = idx.search(q, k)
        rs, ri = _oracle_search(x, q, bits, k, mode=O.MODE_LUT_MULADD)
        assert np.array_equal(i, ri), f"k={k}: id lists differ"
        assert np.array_equal(s, rs), f"k={k}: scores differ"
    mask = np.random.default_rng(5).random(n) < 0.05
    s, i = idx.search(q, 10, mask=mask)
    rs, ri = _oracle_search(x, q, bits, 10, mask=mask, mode=O.MODE_LUT_MULADD)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)


def test_sharded_index_single_rank_on_device(T):
    """The slot-sharded wrapper around a real device index (one rank): same answers as the plain index."""
    from turbovec_b200.sharded import ShardedIndex
    dim, n = 128, 5000
    x = anisotropic(n, dim, seed=71)
    q = anisotropic(6, dim, seed=71, offset=2)
    sh = ShardedIndex(dim, 4, chunk_blocks=16)
    for a, b in ((0, 700), (700, 701), (701, n)):
        sh.add(x[a:b])
    ref = _build(T, x, 4)
    s, i = sh.search(q, 10)
    rs, ri = ref.search(q, 10)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)
    mask = np.random.default_rng(1).random(n) < 0.01
    s, i = sh.search(q, 10, mask=mask)
    rs, ri = ref.search(q, 10, mask=mask)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)
    assert sh.swap_remove(17) == ref.swap_remove(17)
    s, i = sh.search(q, 10)
    rs, ri = ref.search(q, 10)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)
    codes, scale = ref.get_row(17)
    ref.set_row(3, codes, scale)
    c2, s2 = ref.get_row(3)
    assert np.array_equal(c2, codes) and s2 == scale


@pytest.mark.parametrize("nq,k", [(5, 10), (70, 100), (3, 1200)])
def test_keyed_shard_search_and_device_merge_equal_the_whole_index(T, nq, k):
    """Two shards searched with result keys and global slot offsets, merged on the device, give exactly the
    scores and slots of one index holding all vectors (a vector's score does not depend on its neighbours)."""
    import torch
    n, dim = 2000, 256
    x = anisotropic(n, dim, seed=21)
    q = anisotropic(nq, dim, seed=21, offset=500)
    whole = T.TurboQuantIndex(dim, 4)
    whole.add(x)
    want_s, want_i = whole.search(q, k)
    cut = 1120
    shards = [T.TurboQuantIndex(dim, 4), T.TurboQuantIndex(dim, 4)]
    shards[0].add(x[:cut])
    shards[1].add(x[cut:])
    qd = torch.from_numpy(q).cuda()
    keys = torch.empty((2, nq, k), dtype=torch.int64, device="cuda")
    for r, (idx, off) in enumerate(zip(shards, (0, cut))):
        ke = idx.search_device_keys(qd.data_ptr(), nq, k, keys[r].data_ptr(), off)
        assert ke == min(k, len(idx))
    s = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    i = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    T.merge_keys_device(keys.data_ptr(), 2, nq, k, s.data_ptr(), i.data_ptr(), device=0,
                        stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ke = want_s.shape[1]
    assert np.array_equal(i.cpu().numpy()[:, :ke], want_i)
    assert np.array_equal(s.cpu().numpy()[:, :ke], want_s)
    if ke < k:                                      # places past the number of vectors: (-inf, 0) padding
        assert np.all(np.isneginf(s.cpu().numpy()[:, ke:])) and np.all(i.cpu().numpy()[:, ke:] == 0)


def test_large_allowlist_resolved_by_host_threads(T):
    """Allowlists of 65,536 ids and more are resolved by several host threads; the result and the unknown id
    that is reported (the first one in list order) are those of a sequential walk."""
    n, dim = 140_000, 64
    rng = np.random.default_rng(3)
    x = anisotropic(n, dim, seed=31)
    ids = (rng.permutation(n).astype(np.uint64) + np.uint64(10 ** 9))
    idx = T.IdMapIndex(dim, 4)
    idx.add_with_ids(x, ids)
    q = anisotropic(4, dim, seed=31, offset=77)
    allow = ids[rng.permutation(n)[:100_000]].copy()
    s, got = idx.search(q, 10, allowlist=allow)
    mask = np.isin(ids, allow)
    rs, ri = _oracle_search(x, q, 4, 10, mask=mask)
    assert np.array_equal(got, ids[ri]) and np.array_equal(s, rs)
    bad = allow.copy()
    bad[70_000] = np.uint64(5)
    bad[90_001] = np.uint64(6)
    with pytest.raises(KeyError, match="5"):
        idx.search(q, 10, allowlist=bad)


def test_host_add_through_several_staging_chunks(T):
    """A host-memory add larger than the staging buffers (64 MB each, two of them in rotation): every chunk but
    the first starts in the middle of a code block; codes and scales must still be the oracle's."""
    n, dim = 35_017, 1536
    x = anisotropic(n, dim, seed=51)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x[:7])
    idx.add(x[7:])
    enc = O.encode(x, 4)
    assert np.array_equal(idx.codes_blocked_seq(), O.packed_to_blocked(enc["packed"], 4, dim))
    assert np.array_equal(idx.scales().view(np.uint32), enc["scales"].view(np.uint32))
    bad = x.copy()
    bad[30_123, 77] = np.inf                      # in the fourth chunk
    idx2 = T.TurboQuantIndex(dim, 4)
    with pytest.raises(ValueError, match="vector 30123 coordinate 77"):
        idx2.add(bad)
    assert len(idx2) == 0


def test_pipelined_ingest_block_and_wave_boundaries(T):
    """Batch sizes around the boundaries of the pipelined kernel: fewer blocks than CTAs, a single wave,
    one block per CTA exactly, a ragged last block, adds that start on and off a block boundary."""
    dim = 128
    x = anisotropic(9_600, dim, seed=61)
    enc = O.encode(x, 4)
    want_blocked = O.packed_to_blocked(enc["packed"], 4, dim)
    for n in (1, 7, 8, 9, 31, 32, 33, 63, 64, 65, 255, 256, 257, 4_735, 4_736, 4_737, 9_473):
        for first in (0, 5, 32):
            if first >= n:
                continue
            idx = T.TurboQuantIndex(dim, 4)
            if first:
                idx.add(x[:first])
            idx.add(x[first:n])
            sub = O.encode(x[:n], 4)
            assert np.array_equal(idx.packed_codes(), sub["packed"]), (n, first)
            assert np.array_equal(idx.scales().view(np.uint32), sub["scales"].view(np.uint32)), (n, first)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    assert np.array_equal(idx.codes_blocked_seq(), want_blocked)


@pytest.mark.parametrize("n", [1, 31, 33, 4095, 4096, 4097, 4129, 12_000, 110_000])
def test_tensor_memory_scan_chunk_boundaries(T, n):
    """Index sizes around the first chunk (written in place, 4,096 or 8,192 vectors) and the growth steps of
    the tensor-memory path's chunk schedule, for k below and above the 512 that doubles the list capacity."""
    dim, nq = 64, 40
    x = anisotropic(n, dim, seed=71)
    q = anisotropic(nq, dim, seed=71, offset=3)
    idx = _build(T, x, 4)
    for k in (1, 10, 600):
        s, i = idx.search(q, k)
        rs, ri = _oracle_search(x, q, 4, k)
        assert s.shape == (nq, min(k, n))
        assert np.array_equal(i, ri), f"n={n} k={k}: id lists differ"
        assert np.array_equal(s, rs), f"n={n} k={k}: scores differ"


def test_chunk_size_keyword_gives_the_unsliced_results(T):
    """search / add / add_with_ids accept the reference binding's chunk_size= keyword; slicing changes nothing."""
    dim, n = 64, 3000
    x = anisotropic(n, dim, seed=81)
    q = anisotropic(70, dim, seed=81, offset=9)
    a, b = T.TurboQuantIndex(dim, 4), T.TurboQuantIndex(dim, 4)
    a.add(x)
    b.add(x, chunk_size=999)
    assert np.array_equal(a.codes_blocked_seq(), b.codes_blocked_seq()) and np.array_equal(a.scales(), b.scales())
    s0, i0 = a.search(q, 10)
    for cs in (1, 7, 64, 0, -3, 1000):
        s1, i1 = a.search(q, 10, chunk_size=cs)
        assert np.array_equal(s0, s1) and np.array_equal(i0, i1)
    bad = x.copy()
    bad[2500, 3] = np.nan
    c = T.TurboQuantIndex(dim, 4)
    with pytest.raises(ValueError, match="vector 2500 coordinate 3"):
        c.add(bad, chunk_size=100)
    assert len(c) == 0                                   # rejected whole: no slice was committed
    ids = np.arange(n, dtype=np.uint64) + np.uint64(10)
    m = T.IdMapIndex(dim, 4)
    m.add_with_ids(x, ids, chunk_size=512)
    s2, g2 = m.search(q, 10, chunk_size=16, allowlist=ids[::3].copy())
    s3, g3 = m.search(q, 10, allowlist=ids[::3].copy())
    assert np.array_equal(s2, s3) and np.array_equal(g2, g3)
    with pytest.raises(ValueError, match="already present"):
        m.add_with_ids(x[:600], ids[:600].copy(), chunk_size=100)
    assert len(m) == n


def test_concurrent_searches_from_host_threads(T):
    """`search(&self)` is concurrent-safe in the reference (lib.rs:22-52, tests/concurrent_search.rs): searches
    issued from several host threads on one handle return what the same searches return one after another."""
    import threading
    dim, n = 256, 20_000
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(anisotropic(n, dim, seed=71))
    batches = [anisotropic(b, dim, seed=72, offset=100 * j) for j, b in enumerate([1, 7, 40, 300, 3, 64, 1, 130])]
    want = [idx.search(q, 10) for q in batches]
    got = [None] * len(batches)
    errors = []

    def work(j):
        try:
            for _ in range(5):
                got[j] = idx.search(batches[j], 10)
        except Exception as e:            # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(j,)) for j in range(len(batches))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    for (s0, i0), (s1, i1) in zip(want, got):
        assert np.array_equal(i0, i1) and np.array_equal(s0, s1)


def test_add_with_ids_from_device_memory(T):
    """Rows that already live on the GPU enter an id-mapped index exactly as host rows do."""
    import torch
    dim, n = 384, 5000
    x = anisotropic(n, dim, seed=81)
    ids = (np.arange(n, dtype=np.uint64) * 5 + 77)
    a, b = T.IdMapIndex(dim, 4), T.IdMapIndex(dim, 4)
    a.add_with_ids(x, ids)
    xd = torch.from_numpy(x).cuda()
    b.add_with_ids_device(xd.data_ptr(), 3000, dim, ids[:3000])
    b.add_with_ids_device(xd[3000:].contiguous().data_ptr(), n - 3000, dim, ids[3000:])
    assert a.to_bytes() == b.to_bytes()
    with pytest.raises(ValueError, match="already present"):
        b.add_with_ids_device(xd.data_ptr(), 1, dim, ids[:1])
    assert len(b) == n


@pytest.mark.parametrize("nq", [1, 5, 16, 17, 32])
def test_split_and_merged_level_lookups_agree_with_the_oracle(T, nq):
    """The small-batch permute-dot scan looks levels up in two half-tables (two exact contractions, subtracted) or
    in one merged table (`TV_OPT_PD_SPLIT`); both must reproduce the oracle bit for bit, masked or not."""
    dim, n, k = 512, 9000, 10
    x = anisotropic(n, dim, seed=91)
    q = anisotropic(nq, dim, seed=91, offset=7)
    enc = O.encode(x, 4)
    blocked = O.packed_to_blocked(enc["packed"], 4, dim)
    mask = np.random.default_rng(3).random(n) < 0.3
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    idx.set_option(T.OPT_TC_EXPANDED, 0)            # 17 and 32 queries stay on the mma.sync scan
    for m in (None, mask):
        words = None if m is None else O.pack_mask(m)
        want_s, want_i = O.search(q, blocked, enc["scales"], n, dim, 4, k, mask_words=words)
        for split in (1, 0):
            idx.set_option(T.OPT_PD_SPLIT, split)
            assert idx.get_option(T.OPT_PD_SPLIT) == split
            s, i = idx.search(q, k, mask=m)
            assert np.array_equal(i, want_i) and np.array_equal(s.view(np.uint32), want_s.view(np.uint32))


@pytest.mark.parametrize("n,dim,ties", [(40_000, 256, False), (3000, 200, True), (2, 64, False), (777, 1536, True)])
def test_device_quantile_fit_equals_the_oracle(T, n, dim, ties):
    """The two order statistics per coordinate of the TQ+ fit are selected on the device (radix select over the rotated
    sample); shift and scale must equal the oracle's, which sorts on the host -- also with many equal values (rows
    repeated, coordinates quantised to a few levels) and at the smallest sample."""
    x = anisotropic(n, dim, seed=91)
    if ties:
        x = np.round(x * 3.0) / 3.0 + 1e-3                       # few distinct values per coordinate, no zero rows
        x[n // 2:] = x[: n - n // 2]                              # and every row twice
        x = np.ascontiguousarray(x, np.float32)
    idx = T.TurboQuantIndex(dim, 4)
    idx.calibrate(x)
    shift, scale = idx.calibration()
    o_shift, o_scale = O.fit_calibration(x, 4)
    assert np.array_equal(shift.view(np.uint32), o_shift.view(np.uint32))
    assert np.array_equal(scale.view(np.uint32), o_scale.view(np.uint32))
