"""The reference's search property tests, replayed against the CPU oracle (no GPU).

The reference freezes no score or id list for a search, so the oracle's search half cannot be pinned on
golden vectors.  What the reference does hold is a set of behavioural properties that every one of its
kernels must satisfy; this file replays them against `oracle/tv_oracle.c`, in every score mode the property
applies to, on seeded Gaussian rows of the same shapes:

  turbovec/tests/kernel_correctness.rs:72-132   self-match at block-tail sizes (4-bit top-1, 2-bit top-3)
  turbovec/tests/kernel_correctness.rs:135-180  scores finite and sorted descending (2/3/4-bit)
  turbovec/tests/kernel_correctness.rs:184-245  k > len clamps to len, distinct in-range slots
  turbovec/tests/kernel_correctness.rs:268-320, tests/batch_matches_single.rs:58-85   batch == single query
  turbovec/tests/kernel_correctness.rs:409-457  more than 256 byte-groups (flush cadence of the LUT family)
  turbovec/tests/filtering.rs:87-165            masked == post-filtered, all-true == none, effective k, all-false
  turbovec/tests/filtering.rs:175-229           multi-query batch under a mask; 1e-4 cross-kernel score tolerance
  turbovec/tests/filtering.rs:609-622           n_allowed < k on a large index
  turbovec/tests/filtering.rs:685-720           every k is a prefix of the full ranking, bit for bit
  turbovec/tests/query_scale_invariance.rs:201-284   power-of-two rescale is exact, linear scaling, zero query
"""
import numpy as np
import pytest

from oracle import oracle as O

TAIL_SIZES = [32, 33, 63, 64, 65, 96, 127, 128, 129, 160, 191, 192, 193, 256, 257, 500]
SEAM_NQS = [1, 7, 8, 9, 23, 50]


def unit_rows(n, dim, seed):
    x = np.random.default_rng(seed).standard_normal((n, dim)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return np.ascontiguousarray(x)


class Index:
    """The oracle's encode output in the form its search takes."""

    def __init__(self, x, bits):
        self.n, self.dim, self.bits = x.shape[0], x.shape[1], bits
        enc = O.encode(x, bits)
        self.blocked = O.packed_to_blocked(enc["packed"], bits, self.dim)
        self.scales = enc["scales"]

    def search(self, q, k, mask=None, mode=O.MODE_AUTO):
        words = None if mask is None else O.pack_mask(mask)
        return O.search(q, self.blocked, self.scales, self.n, self.dim, self.bits, k, mask_words=words, mode=mode)


def modes_for(bits, dim):
    """Every score mode the oracle implements for this geometry (search.rs:2975-2980, pack.rs:1260-1263)."""
    ng = O.ngroups(dim, bits)
    modes = [O.MODE_LUT_FLUSH, O.MODE_LUT_SCALAR]
    if ng % 4 == 0:
        modes.append(O.MODE_LUT_MULADD)
        if bits == 4:
            modes.append(O.MODE_PD)
    return modes


@pytest.mark.parametrize("n", TAIL_SIZES)
def test_self_query_returns_self(n):
    dim = 512
    x4, x2 = unit_rows(n, dim, 0x5EED ^ n), unit_rows(n, dim, 0xC0FF ^ n)
    i4, i2 = Index(x4, 4), Index(x2, 2)
    nq = min(n, 8)
    for mode in modes_for(4, dim):
        _, slots = i4.search(x4[:nq], 1, mode=mode)
        assert np.array_equal(slots[:, 0], np.arange(nq)), f"4-bit self-match, n={n} mode={mode}"
    for mode in modes_for(2, dim):
        _, slots = i2.search(x2[:nq], min(3, n), mode=mode)
        assert all(q in slots[q] for q in range(nq)), f"2-bit self-match in top 3, n={n} mode={mode}"


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_scores_finite_and_sorted_descending(bits):
    dim = 256
    for n in [64, 100, 128, 200, 256, 500]:
        x = unit_rows(n, dim, 0xA11CE ^ n ^ bits)
        idx = Index(x, bits)
        for mode in modes_for(bits, dim):
            scores, slots = idx.search(x[:4], min(10, n), mode=mode)
            assert np.all(np.isfinite(scores))
            assert np.all(scores[:, :-1] >= scores[:, 1:])
            # ties resolve to the lower slot (search.rs:236-252)
            tie = scores[:, :-1] == scores[:, 1:]
            assert np.all(slots[:, :-1][tie] < slots[:, 1:][tie])


def test_k_exceeding_len_clamps_to_len():
    dim, n, k, nq = 512, 3, 10, 2
    idx = Index(unit_rows(n, dim, 0xEFFEC7), 4)
    scores, slots = idx.search(unit_rows(nq, dim, 0xEFFEC8), k)
    assert scores.shape == (nq, n) and slots.shape == (nq, n)
    for q in range(nq):
        assert sorted(slots[q]) == list(range(n))
        assert np.all(np.isfinite(scores[q])) and np.all(scores[q][:-1] >= scores[q][1:])


@pytest.mark.parametrize("bits,dim", [(4, 64), (2, 64), (3, 64), (4, 256)])
def test_batch_results_match_single_query_results(bits, dim):
    n, k = 9000, 10
    idx = Index(unit_rows(n, dim, 0xBA7C4 + bits), bits)
    queries = unit_rows(50, dim, 0xBA7C5)
    for mode in modes_for(bits, dim):
        for nq in SEAM_NQS:
            bs, bi = idx.search(queries[:nq], k, mode=mode)
            assert bs.shape == (nq, k)
            for q in range(nq):
                ss, si = idx.search(queries[q:q + 1], k, mode=mode)
                assert np.array_equal(bi[q], si[0])
                assert np.array_equal(bs[q].view(np.uint32), ss[0].view(np.uint32))


@pytest.mark.parametrize("dim", [1024, 2048])
def test_flush_cadence_beyond_256_byte_groups(dim):
    """dim/2 > 256 byte-groups: the per-256-group fma of the flush family runs more than once."""
    for n in [64, 100]:
        x = unit_rows(n, dim, 0xF1054000 ^ dim ^ n)
        idx = Index(x, 4)
        for mode in modes_for(4, dim):
            for nq in [1, 4, 8]:
                scores, slots = idx.search(x[:nq], 5, mode=mode)
                assert np.array_equal(slots[:, 0], np.arange(nq))
                assert np.all(np.isfinite(scores))
                assert np.all(np.abs(scores[:, 0] - 1.0) < 0.25), "self-score off scale: wrapped or missed flush"


def post_filter(idx, q, mask, k, mode):
    scores, slots = idx.search(q, idx.n, mode=mode)
    keep = mask[slots[0]]
    return scores[0][keep][:k], slots[0][keep][:k]


@pytest.mark.parametrize("bits", [2, 4])
def test_mask_matches_post_hoc_filter(bits):
    dim, n = 128, 256
    idx = Index(unit_rows(n, dim, 0xF11D0001), bits)
    q = unit_rows(1, dim, 0xF11D0002)
    mask = np.arange(n) % 2 == 0
    for mode in modes_for(bits, dim):
        scores, slots = idx.search(q, 10, mask=mask, mode=mode)
        ref_s, ref_i = post_filter(idx, q, mask, 10, mode)
        assert scores.shape == (1, 10)
        assert np.array_equal(slots[0], ref_i) and np.array_equal(scores[0].view(np.uint32), ref_s.view(np.uint32))
        assert np.all(mask[slots[0]])


def test_mask_none_equals_mask_all_true():
    dim, n = 64, 200
    idx = Index(unit_rows(n, dim, 0xF11D0003), 4)
    q = unit_rows(1, dim, 0xF11D0004)
    for mode in modes_for(4, dim):
        a = idx.search(q, 20, mode=mode)
        b = idx.search(q, 20, mask=np.ones(n, bool), mode=mode)
        assert np.array_equal(a[1], b[1]) and np.array_equal(a[0].view(np.uint32), b[0].view(np.uint32))


def test_effective_k_and_all_false_mask():
    dim, n = 64, 100
    idx = Index(unit_rows(n, dim, 0xF11D0005), 4)
    q = unit_rows(1, dim, 0xF11D0006)
    mask = np.zeros(n, bool)
    mask[[3, 42, 77]] = True
    scores, slots = idx.search(q, 10, mask=mask)
    assert scores.shape == (1, 3) and sorted(slots[0]) == [3, 42, 77]
    scores, slots = idx.search(q, 5, mask=np.zeros(n, bool))
    assert scores.shape[1] == 0 and slots.shape[1] == 0


def test_multi_query_batch_respects_mask():
    dim, n, nq = 128, 256, 7
    idx = Index(unit_rows(n, dim, 0xF11D000B), 4)
    queries = unit_rows(nq, dim, 0xF11D000C)
    mask = np.arange(n) % 3 == 0
    for mode in modes_for(4, dim):
        scores, slots = idx.search(queries, 8, mask=mask, mode=mode)
        assert scores.shape == (nq, 8)
        assert np.all(mask[slots]) and np.all(scores[:, :-1] >= scores[:, 1:])
        for q in range(nq):
            ref_s, ref_i = post_filter(idx, queries[q:q + 1], mask, 8, mode)
            assert np.array_equal(slots[q], ref_i)
            assert np.array_equal(scores[q].view(np.uint32), ref_s.view(np.uint32))


@pytest.mark.parametrize("bits,dim", [(4, 128), (4, 1536), (2, 512), (3, 256)])
def test_cross_kernel_score_tolerance(bits, dim):
    """The reference's kernel families order the two or three float operations after the exact integer sum
    differently; its own tests hold them to 1e-4 relative (filtering.rs:217-229).  The oracle's LUT float
    variants must agree to that tolerance on every vector, and the id order may differ only inside it."""
    n = 300
    idx = Index(unit_rows(n, dim, 0x70C ^ dim), bits)
    q = unit_rows(3, dim, 0x70D ^ dim)
    lut_modes = [m for m in modes_for(bits, dim) if m != O.MODE_PD]
    base_s, base_i = idx.search(q, n, mode=lut_modes[0])
    by_slot = np.empty_like(base_s)
    np.put_along_axis(by_slot, base_i, base_s, axis=1)
    for mode in lut_modes[1:]:
        s, i = idx.search(q, n, mode=mode)
        other = np.empty_like(s)
        np.put_along_axis(other, i, s, axis=1)
        tol = 1e-4 * np.maximum(np.maximum(np.abs(by_slot), np.abs(other)), 1.0)
        assert np.all(np.abs(by_slot - other) <= tol)


def test_n_allowed_below_k_on_a_large_index():
    dim, n = 64, 10000
    idx = Index(unit_rows(n, dim, 0xF11D2008), 4)
    q = unit_rows(1, dim, 0xF11D2009)
    mask = np.zeros(n, bool)
    mask[[3, 4000, 9500]] = True
    scores, slots = idx.search(q, 10, mask=mask)
    assert scores.shape == (1, 3) and np.all(mask[slots[0]])


@pytest.mark.parametrize("seed", [0xBEEF0001, 0xBEEF0002])
def test_every_k_is_a_prefix_of_the_full_ranking(seed):
    dim, n = 64, 10000
    idx = Index(unit_rows(n, dim, seed), 4)
    q = unit_rows(1, dim, seed ^ 0xABCD)
    for mode in modes_for(4, dim):
        full_s, full_i = idx.search(q, n, mode=mode)
        for k in [1, 10, 64, 100]:
            s, i = idx.search(q, k, mode=mode)
            assert np.array_equal(i[0], full_i[0][:k])
            assert np.array_equal(s[0].view(np.uint32), full_s[0][:k].view(np.uint32))


@pytest.mark.parametrize("mode", [O.MODE_PD, O.MODE_LUT_MULADD, O.MODE_LUT_FLUSH])
def test_power_of_two_query_scaling_is_bit_exact(mode):
    dim, n, nq, k = 768, 1000, 32, 10
    idx = Index(unit_rows(n, dim, 0x5EED), 4)
    q = unit_rows(nq, dim, 0x1234)
    base_s, base_i = idx.search(q, k, mode=mode)
    base_t = O.query_tables(q, dim, 4, mode=mode)
    for c in [1024.0, 65536.0, 1.0 / 1024.0, 2.0 ** -60]:
        qc = (q * np.float32(c)).astype(np.float32)
        t = O.query_tables(qc, dim, 4, mode=mode)
        # the integer tables do not move; the scale carries the factor exactly
        assert np.array_equal(t["luts"], base_t["luts"]) and np.array_equal(t["weights"], base_t["weights"])
        assert np.array_equal(t["scale"], base_t["scale"] * np.float32(c))
        s, i = idx.search(qc, k, mode=mode)
        assert np.array_equal(i, base_i)
        assert np.array_equal(s, base_s * np.float32(c))


def test_scores_scale_linearly_and_ids_survive_rescaling():
    dim, n, nq, k = 768, 1000, 32, 10
    idx = Index(unit_rows(n, dim, 0x5EED), 4)
    q = unit_rows(nq, dim, 0x1234)
    for mode in [O.MODE_PD, O.MODE_LUT_MULADD]:
        base_s, base_i = idx.search(q, k, mode=mode)
        for c in [1e6, 1e3, 1e-3, 1e-6]:
            s, i = idx.search((q * np.float32(c)).astype(np.float32), k, mode=mode)
            want = base_s * np.float32(c)
            assert np.all(np.abs(s - want) / np.maximum(np.abs(want), np.finfo(np.float32).tiny) < 2e-2)
            # the ranking may move only between near-tied neighbours: the id sets stay almost the same
            overlap = np.mean([len(set(i[j]) & set(base_i[j])) / k for j in range(nq)])
            assert overlap >= 0.95


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_zero_query_is_well_formed(bits):
    dim = 256
    idx = Index(unit_rows(500, dim, 0xABCD), bits)
    for mode in modes_for(bits, dim):
        scores, slots = idx.search(np.zeros((1, dim), np.float32), 10, mode=mode)
        assert np.all(np.isfinite(scores))
        # every score ties, so the lower slots win (search.rs:236-252)
        assert np.array_equal(slots[0], np.arange(10))
