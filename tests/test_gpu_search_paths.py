"""Search paths beyond the defaults, each through the C ABI and against the CPU oracle on the same inputs:
every variant of the stream-shaped small-batch scan, paged top-k for k above one selection pass, u8-LUT
geometries whose tables crowd shared memory, prepared masks, searches that overlap on one handle, two devices
in one process, and the all-or-nothing contract under an injected allocation / upload failure."""
import threading

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import anisotropic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    import turbovec_b200
    return turbovec_b200


def oracle_index(x, bits):
    enc = O.encode(x, bits)
    return O.packed_to_blocked(enc["packed"], bits, x.shape[1]), enc["scales"]


def oracle_search(x, q, bits, k, mask=None, mode=O.MODE_AUTO, pre=None):
    blocked, scales = pre if pre is not None else oracle_index(x, bits)
    words = None if mask is None else O.pack_mask(mask)
    return O.search(q, blocked, scales, x.shape[0], x.shape[1], bits, k, mask_words=words, mode=mode)


# ------------------------------------------------------------------ stream-shaped small-batch scan
@pytest.mark.parametrize("dim,n", [(1536, 9000), (200, 5000), (64, 4500), (4096, 1200), (1000, 3000)])
def test_small_scan_variants_match_oracle(T, dim, n):
    """All ring depths, plain and swizzled stage fills, 1..16 queries, with and without a mask: bit-identical to
    the oracle.  dim 200 has a 36-row tail chunk, dim 64 a single half-filled chunk, dim 1000 an 8-point rotation."""
    x = anisotropic(n, dim, seed=41)
    pre = oracle_index(x, 4)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    mask = np.random.default_rng(3).random(n) < 0.3
    for nq in (1, 3, 8, 9, 16):
        q = anisotropic(nq, dim, seed=41, offset=700 + nq)
        want = oracle_search(x, q, 4, 10, pre=pre)
        want_m = oracle_search(x, q, 4, 10, mask=mask, pre=pre)
        for variant in (-1, 0, 1, 2, 4, 5, 6):
            idx.set_option(T.OPT_SMALL_SCAN, variant)
            s, i = idx.search(q, 10)
            assert np.array_equal(i, want[1]) and np.array_equal(s, want[0]), f"variant {variant}, {nq} queries"
            s, i = idx.search(q, 10, mask=mask)
            assert np.array_equal(i, want_m[1]) and np.array_equal(s, want_m[0]), f"variant {variant}, {nq} queries, masked"


def test_small_scan_many_chunks_and_recovery(T):
    n, dim = 150_000, 128
    x = anisotropic(n, dim, seed=8)
    q = anisotropic(4, dim, seed=8, offset=3)
    order = np.argsort(x @ q[0])                       # adversarial order for query 0: overflows, then recovers
    x = np.ascontiguousarray(x[order])
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    want = oracle_search(x, q, 4, 10)
    for variant in (0, 6):
        idx.set_option(T.OPT_SMALL_SCAN, variant)
        s, i = idx.search(q, 10)
        assert np.array_equal(i, want[1]) and np.array_equal(s, want[0])


# ------------------------------------------------------------------ the forms of the tensor-memory scan
@pytest.mark.parametrize("dim,n,nq", [(1536, 5003, 70), (1536, 4100, 300), (256, 4100, 257), (200, 9000, 1024), (1536, 40_000, 129), (512, 7000, 17),
                                      (64, 300_000, 65), (256, 20_000, 513), (128, 9000, 770)])
@pytest.mark.parametrize("form", ["dense", "dense1", "wide", "narrow"])
def test_tensor_scan_forms_match_oracle(T, dim, n, nq, form):
    """The forms of the tensor-memory scan: over the int8 copy of the index (both operands by TMA) on CTA pairs (the
    default) and on single CTAs ("dense1"), and over the codes with two query groups per expanded slab ("wide": batches
    above 256 queries; 513 and 770 queries end in an item of one group) or with one group per item ("narrow").  Odd numbers of 128-vector tiles, several chunks, partial query groups, masks."""
    x = anisotropic(n, dim, seed=57)
    q = anisotropic(nq, dim, seed=57, offset=31)
    pre = oracle_index(x, 4)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    idx.set_option(T.OPT_TC_EXPANDED, 2 if form.startswith("dense") else 0)
    idx.set_option(T.OPT_DENSE_PAIR, 1 if form == "dense" else 0)
    idx.set_option(T.OPT_TC_WIDE, 1 if form == "wide" else 0)
    mask = np.random.default_rng(6).random(n) < 0.2
    for k in (10, 100):
        s, i = idx.search(q, k)
        rs, ri = oracle_search(x, q, 4, k, pre=pre)
        assert np.array_equal(i, ri) and np.array_equal(s, rs), f"k={k}"
    s, i = idx.search(q, 10, mask=mask)
    rs, ri = oracle_search(x, q, 4, 10, mask=mask, pre=pre)
    assert np.array_equal(i, ri) and np.array_equal(s, rs), "masked"
    assert (idx.get_option(T.OPT_EXPANDED_BYTES) > 0) == form.startswith("dense")


def test_int8_copy_follows_every_change_of_the_index(T):
    """The int8 copy behind large permute-dot batches is brought up to date lazily: after appends (also into a
    partly filled block and past a growth of the code array), removals, rewritten rows, a re-fit that re-encodes
    every row and a load, a search over it must equal the search over the codes (copy switched off)."""
    dim, nq = 256, 40
    rng = np.random.default_rng(77)
    x = anisotropic(30_000, dim, seed=77)
    q = anisotropic(nq, dim, seed=77, offset=9)
    idx = T.TurboQuantIndex(dim, 4)
    idx.set_option(T.OPT_TC_EXPANDED, 2)

    def check(tag):
        got = idx.search(q, 10)
        idx.set_option(T.OPT_TC_EXPANDED, 0)
        assert idx.get_option(T.OPT_EXPANDED_BYTES) == 0
        want = idx.search(q, 10)
        idx.set_option(T.OPT_TC_EXPANDED, 2)
        assert np.array_equal(got[1], want[1]) and np.array_equal(got[0], want[0]), tag

    def check_kept(tag):                                          # without dropping the copy in between
        got = idx.search(q, 10)
        ref = T.TurboQuantIndex.from_bytes(idx.to_bytes())
        ref.set_option(T.OPT_TC_EXPANDED, 0)
        want = ref.search(q, 10)
        assert np.array_equal(got[1], want[1]) and np.array_equal(got[0], want[0]), tag

    idx.add(x[:1000])
    check_kept("first build")
    idx.add(x[1000:1013])                                         # ends inside a block
    check_kept("append into a block")
    idx.add(x[1013:1020])
    check_kept("append into a partly filled block")
    idx.add(x[1020:20_000])                                       # the code array grows: the copy is rebuilt
    check_kept("growth")
    for victim in rng.integers(0, 15_000, 50):
        idx.swap_remove(int(victim))
    check_kept("removals")
    groups, scale = idx.get_row(5)
    idx.set_row(77, groups, scale)
    idx.set_row(19_000, groups, 0.5 * scale)
    check_kept("rewritten rows")
    for victim in rng.integers(0, 10_000, 5000):                  # more changed blocks than the list holds
        idx.swap_remove(int(victim))
    check_kept("many removals")
    idx.add(x[20_000:])
    check_kept("append after removals")
    idx.calibrate(x[:4000])                                       # re-encodes every stored row
    check_kept("re-fit")
    check("copy dropped and rebuilt")


# ------------------------------------------------------------------ u8-LUT flush family on tensor memory
@pytest.mark.parametrize("dim,n,nq", [(200, 6000, 9), (200, 6000, 300), (1000, 3000, 40), (1016, 2500, 600), (1032, 2000, 12), (40, 5000, 70)])
def test_flush_family_scan_matches_oracle(T, dim, n, nq):
    """2-bit geometries whose byte-group count is not a multiple of 4 (the reference's per-256-group fma family,
    search.rs:516, 577).  Up to 256 groups the batch runs on the tensor-memory scan with K padded to whole slabs;
    dim 1032 (258 groups) needs the partial sums and stays on the CUDA-core scan."""
    x = anisotropic(n, dim, seed=63)
    q = anisotropic(nq, dim, seed=63, offset=17)
    pre = oracle_index(x, 2)
    idx = T.TurboQuantIndex(dim, 2)
    idx.add(x)
    assert idx.get_option(T.OPT_SCORE_MODE) == T.SCORE_LUT_FLUSH
    mask = np.random.default_rng(8).random(n) < 0.3
    for k in (10, 100):
        s, i = idx.search(q, k)
        rs, ri = oracle_search(x, q, 2, k, pre=pre)
        assert np.array_equal(i, ri) and np.array_equal(s, rs), f"k={k}"
    s, i = idx.search(q, 10, mask=mask)
    rs, ri = oracle_search(x, q, 2, 10, mask=mask, pre=pre)
    assert np.array_equal(i, ri) and np.array_equal(s, rs), "masked"
    idx.set_option(T.OPT_MMA_MIN_BATCH, 0)                  # the CUDA-core scan gives the same bits
    s, i = idx.search(q, 10)
    rs, ri = oracle_search(x, q, 2, 10, pre=pre)
    assert np.array_equal(i, ri) and np.array_equal(s, rs), "CUDA-core scan"


# ------------------------------------------------------------------ k above one selection pass
@pytest.mark.parametrize("bits,dim", [(4, 64), (2, 64)])
def test_paged_topk_beyond_4096(T, bits, dim):
    n = 21_000
    x = anisotropic(n, dim, seed=51)
    q = anisotropic(3, dim, seed=51, offset=9)
    idx = T.TurboQuantIndex(dim, bits)
    idx.add(x)
    pre = oracle_index(x, bits)
    for k in (4097, 9000, n, n + 5):
        s, i = idx.search(q, k)
        rs, ri = oracle_search(x, q, bits, k, pre=pre)
        assert s.shape == (3, min(k, n))
        assert np.array_equal(i, ri) and np.array_equal(s, rs), f"k={k}"
    mask = np.random.default_rng(5).random(n) < 0.5
    s, i = idx.search(q, 6000, mask=mask)
    rs, ri = oracle_search(x, q, bits, 6000, mask=mask, pre=pre)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)


# ------------------------------------------------------------------ u8-LUT tables against the shared-memory limit
@pytest.mark.parametrize("dim,bits", [(4096, 3), (8192, 2), (16384, 2), (16384, 3)])
def test_lut_scan_with_large_tables(T, dim, bits):
    n = 700
    x = anisotropic(n, dim, seed=61)
    idx = T.TurboQuantIndex(dim, bits)
    idx.add(x)
    pre = oracle_index(x, bits)
    for nq in (1, 3, 7):
        q = anisotropic(nq, dim, seed=61, offset=40 + nq)
        s, i = idx.search(q, 10)
        rs, ri = oracle_search(x, q, bits, 10, pre=pre)
        assert np.array_equal(i, ri) and np.array_equal(s, rs), f"{nq} queries"


def test_lut_flush_mode_without_room_for_one_table_is_refused(T):
    dim = 16384
    idx = T.TurboQuantIndex(dim, 3)
    idx.add(anisotropic(64, dim, seed=1))
    idx.set_option(T.OPT_SCORE_MODE, T.SCORE_LUT_FLUSH)
    with pytest.raises(RuntimeError, match="exceed shared memory"):
        idx.search(anisotropic(1, dim, seed=1, offset=5), 5)


# ------------------------------------------------------------------ prepared masks
def test_prepared_mask_equals_mask_per_call(T):
    import torch
    n, dim, nq = 50_000, 256, 5
    x = anisotropic(n, dim, seed=71)
    q = anisotropic(nq, dim, seed=71, offset=11)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    mask = np.random.default_rng(2).random(n) < 0.02
    want = idx.search(q, 20, mask=mask)
    rs, ri = oracle_search(x, q, 4, 20, mask=mask)
    assert np.array_equal(want[1], ri) and np.array_equal(want[0], rs)
    words = O.pack_mask(mask)
    idx.prepare_mask_words(words)
    for _ in range(2):
        s, i = idx.search_prepared(q, 20)
        assert np.array_equal(i, ri) and np.array_equal(s, rs)
    d_words = torch.from_numpy(words.view(np.int64)).cuda()
    idx.prepare_mask_device(d_words.data_ptr())
    qd = torch.from_numpy(q).cuda()
    out_s = torch.empty((nq, 20), dtype=torch.float32, device="cuda")
    out_i = torch.empty((nq, 20), dtype=torch.int64, device="cuda")
    ke = idx.search_device_prepared(qd.data_ptr(), nq, 20, out_s.data_ptr(), out_i.data_ptr())
    assert ke == 20 and np.array_equal(out_i.cpu().numpy(), ri) and np.array_equal(out_s.cpu().numpy(), rs)
    # a change of the index drops the prepared mask
    idx.swap_remove(3)
    with pytest.raises(RuntimeError, match="no prepared mask"):
        idx.search_prepared(q, 20)


def test_prepared_allowlist_on_idmap(T):
    n, dim = 4000, 128
    x = anisotropic(n, dim, seed=72)
    ids = (np.random.default_rng(4).permutation(n) + 10**9).astype(np.uint64)
    idx = T.IdMapIndex(dim, 4)
    idx.add_with_ids(x, ids)
    allow = np.ascontiguousarray(ids[::7])
    q = anisotropic(3, dim, seed=72, offset=2)
    want = idx.search(q, 50, allowlist=allow)
    idx.prepare_allowlist(allow)
    got = idx.search_prepared(q, 50)
    assert np.array_equal(got[1], want[1]) and np.array_equal(got[0], want[0])
    with pytest.raises(KeyError):
        idx.prepare_allowlist(np.array([5], np.uint64))


def test_long_allowlists_resolved_by_the_device_id_table(T):
    """Allowlists of 32768 ids and more are turned into mask bits by a hash table on the device; the result must be
    the one the same set gives as a packed slot mask (no id table involved), through adds, removals and rebuilds."""
    n, dim = 120_000, 64
    rng = np.random.default_rng(101)
    x = anisotropic(n, dim, seed=101)
    ids = rng.permutation(n).astype(np.uint64) * np.uint64(0x9E3779B1) + np.uint64(7)
    idx = T.IdMapIndex(dim, 4)
    idx.add_with_ids(x[:100_000], ids[:100_000])
    q = anisotropic(6, dim, seed=101, offset=5)

    def check(k=20):
        live = idx.ids()                                                 # slot order
        pick = rng.random(live.size) < 0.4
        allow = np.concatenate([live[pick], live[pick][:500]])         # duplicates are fine
        assert allow.size >= 32768
        rng.shuffle(allow)
        got = idx.search(q, k, allowlist=np.ascontiguousarray(allow))
        bits = np.zeros(((live.size + 63) // 64) * 64, np.uint8)
        bits[: live.size] = pick
        idx.prepare_mask_words(np.packbits(bits, bitorder="little").view(np.uint64))
        want = idx.search_prepared(q, k)
        assert np.array_equal(got[1], want[1]) and np.array_equal(got[0], want[0])
        return allow

    allow = check()                                                      # first use: the table is built
    bad = np.ascontiguousarray(np.concatenate([allow[:40_000], np.array([3], np.uint64), allow[:10]]))
    with pytest.raises(KeyError, match="allowlist id 3 "):
        idx.search(q, 5, allowlist=bad)
    victims = [int(v) for v in rng.choice(idx.ids(), 300, replace=False)]
    for victim in victims:                                               # swap-removes: updates of the table
        assert idx.remove(victim)
    idx.add_with_ids(x[100_000:100_500], ids[100_000:100_500])
    check()
    gone = np.ascontiguousarray(np.concatenate([idx.ids()[:40_000], np.array([victims[0]], np.uint64)]))
    with pytest.raises(KeyError):
        idx.search(q, 5, allowlist=gone)
    idx.add_with_ids(x[100_500:], ids[100_500:])                        # a larger update in one go
    check(k=64)
    idx = T.IdMapIndex.from_bytes(idx.to_bytes())                        # a loaded index builds its table afresh
    check(k=64)
    half = np.ascontiguousarray(idx.ids()[::2])
    want = idx.search(q, 10, allowlist=half)
    idx.prepare_allowlist(half)                                          # prepared masks use the same table
    got = idx.search_prepared(q, 10)
    assert np.array_equal(got[1], want[1]) and np.array_equal(got[0], want[0])
    with pytest.raises(KeyError):
        idx.prepare_allowlist(np.ascontiguousarray(np.concatenate([half, np.array([5], np.uint64)])))


# ------------------------------------------------------------------ overlapping searches on one handle
def test_searches_from_several_threads_overlap_and_agree(T):
    n, dim = 60_000, 256
    x = anisotropic(n, dim, seed=81)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    queries = [anisotropic(nq, dim, seed=81, offset=100 + t) for t, nq in enumerate([1, 5, 40, 3, 70, 2])]
    want = [idx.search(q, 10) for q in queries]
    errors = []

    def worker(t):
        try:
            for _ in range(8):
                s, i = idx.search(queries[t], 10)
                assert np.array_equal(i, want[t][1]) and np.array_equal(s, want[t][0])
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(len(queries))]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors


# ------------------------------------------------------------------ two devices in one process
def test_indexes_on_two_devices_in_one_process(T):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n, dim = 5000, 256
    x = anisotropic(n, dim, seed=91)
    pre = oracle_index(x, 4)
    for nq, k in [(3, 10), (70, 10), (2, 600)]:
        q = anisotropic(nq, dim, seed=91, offset=nq)
        want = oracle_search(x, q, 4, k, pre=pre)
        for dev in (0, 1):
            idx = T.TurboQuantIndex(dim, 4, device=dev)
            idx.add(x)
            s, i = idx.search(q, k)
            assert np.array_equal(i, want[1]) and np.array_equal(s, want[0]), f"device {dev}"


# ------------------------------------------------------------------ failure before / between launches
def test_injected_failure_leaves_the_index_unchanged(T):
    """The reference's unwind guards restore the pre-call state when an encode step fails
    (turbovec/src/lib.rs:889-930, exercised by its FORCE_ENCODE_PANIC tests).  Here the failure is injected on the
    host: the n-th guarded allocation or upload of the call reports out-of-memory instead of running."""
    dim, n0 = 1536, 5000
    x0 = anisotropic(n0, dim, seed=95)
    ids0 = np.arange(n0, dtype=np.uint64) + 7
    idx = T.IdMapIndex(dim, 4)
    idx.add_with_ids(x0, ids0)
    codes, scales = idx.codes_blocked_seq(), idx.scales()
    more = anisotropic(25_000, dim, seed=96)              # 154 MB: three staging chunks from host memory
    more_ids = np.arange(25_000, dtype=np.uint64) + 10**6
    for nth in (1, 2, 3):                                  # capacity growth, first upload, second upload
        idx.set_option(T.OPT_FAIL_NEXT, nth)
        with pytest.raises(RuntimeError):
            idx.add_with_ids(more, more_ids)
        assert idx.get_option(T.OPT_FAIL_NEXT) == 0
        assert len(idx) == n0 and np.array_equal(idx.ids(), ids0) and not idx.contains(10**6)
        assert np.array_equal(idx.codes_blocked_seq(), codes) and np.array_equal(idx.scales(), scales)
    q = anisotropic(2, dim, seed=95, offset=1)
    want = idx.search(q, 5)
    idx.set_option(T.OPT_FAIL_NEXT, 1)
    with pytest.raises(RuntimeError):
        idx.search(q, 5)
    got = idx.search(q, 5)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    # and the add goes through once nothing fails
    idx.add_with_ids(more, more_ids)
    assert len(idx) == n0 + 25_000 and idx.contains(10**6)
    full = (n0 // 32) * 32 * (dim // 2)                    # the complete blocks of the first add
    assert np.array_equal(idx.codes_blocked_seq()[:full], codes[:full])


# ------------------------------------------------------------------ the reference's CPU-runnable workload at its stated size
def test_reference_workload_config1_full_size(T):
    """100,000 x 1536 4-bit, 1,000 queries, k = 10, single queries and one batch of 1,000: ids and scores against the
    multithreaded CPU restatement of the reference's permute-dot kernel on every query, and against the scalar
    oracle on a sample of them."""
    n, dim, nq, k = 100_000, 1536, 1000, 10
    x = anisotropic(n, dim, seed=1)
    q = anisotropic(nq, dim, seed=1, offset=10_000_000)
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(x)
    enc = O.encode(x, 4)
    blocked = O.packed_to_blocked(enc["packed"], 4, dim)
    assert np.array_equal(idx.codes_blocked_seq(), blocked)
    assert np.array_equal(idx.scales().view(np.uint32), enc["scales"].view(np.uint32))
    bs, bi = idx.search(q, k)                                   # one batch of 1,000: the tensor-memory scan
    singles = [idx.search(q[j:j + 1], k) for j in range(0, nq, 25)]   # single queries: the stream-shaped scan
    for j, (s, i) in zip(range(0, nq, 25), singles):
        assert np.array_equal(i[0], bi[j]) and np.array_equal(s[0], bs[j])
    if O.simd_available():
        vm = O.to_vector_major(blocked, n, dim)
        rs, ri = O.search_simd(q, vm, enc["scales"], n, dim, k)
        assert np.array_equal(bi, ri) and np.array_equal(bs, rs)
    sample = np.arange(0, nq, 50)
    rs, ri = O.search(q[sample], blocked, enc["scales"], n, dim, 4, k)
    assert np.array_equal(bi[sample], ri) and np.array_equal(bs[sample], rs)
    truth = np.argsort(-(q[:100] @ x.T), axis=1)[:, :k]
    recall = np.mean([len(set(bi[j]) & set(truth[j])) / k for j in range(100)])
    assert recall >= 0.70                                       # the reference's 4-bit floor (tests/recall_sanity.rs:97-118)
