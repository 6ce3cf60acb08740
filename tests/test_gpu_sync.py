"""Incremental `sync` (lib.rs:1737, io_v7.rs plan_incremental / run_sync / cursor_state): after every sync the file,
read by an independent restatement of the reference's loader, holds exactly the live index; commits alternate
header slots; removals ride the header as redo ops and are written into place by a later sync; a torn commit
falls back to the previous one; foreign files are refused."""
import os

import numpy as np
import pytest

from tests import v7_reader as R
from tests.util import anisotropic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    import turbovec_b200
    return turbovec_b200


def live_state(idx):
    n = len(idx)
    codes = np.asarray(idx.codes_blocked_seq())
    rb = codes.size // (max(1, -(-n // 32)) * 32) if n else 0
    return codes.reshape(-1, rb, 32) if n else codes.reshape(0, 0, 32), np.asarray(idx.scales())


def check_file(T, idx, path, kind):
    lib = T._native.load()
    img = R.read(lib, path.read_bytes())
    codes, scales = live_state(idx)
    assert img["n"] == len(idx)
    assert np.array_equal(img["codes"], codes)
    assert np.array_equal(img["scales"].view(np.uint32), scales.view(np.uint32))
    if kind == 1:
        assert np.array_equal(img["ids"], idx.ids())
    # and the library's own loader (pinned on the reference's frozen file hashes) agrees
    cls = T.IdMapIndex if kind == 1 else T.TurboQuantIndex
    back = cls.load(str(path))
    assert back.to_bytes() == idx.to_bytes()
    return img, back


def test_sync_appends_and_alternates_slots(T, tmp_path):
    dim, bits = 256, 4
    path = tmp_path / "a.tv"
    idx = T.TurboQuantIndex(dim, bits)
    idx.add(anisotropic(70, dim, seed=1))
    idx.sync(str(path))
    img, _ = check_file(T, idx, path, 0)
    assert img["gen"] == 0 and img["nonce"] != 0 and idx._sync_state()[:2] == (True, 0)
    first_nonce, size0 = img["nonce"], path.stat().st_size
    assert size0 == img["geo"].unit_at(70 // 32)
    for step, rows in enumerate([5, 20, 1, 64, 31], start=1):
        idx.add(anisotropic(rows, dim, seed=10 + step))
        before = path.read_bytes()
        idx.sync(str(path))
        img, _ = check_file(T, idx, path, 0)
        assert img["gen"] == step and img["slot"] == step % 2 and img["nonce"] == first_nonce
        assert img["pending"] == [] and img["mat"] == []
        after = path.read_bytes()
        # the previous commit's header slot and every unit it covered are untouched
        geo = img["geo"]
        prev = geo.hdr_at((step - 1) % 2)
        assert after[prev: prev + geo.hdr_len] == before[prev: prev + geo.hdr_len]
        assert after[geo.unit_at(0): geo.unit_at(img["app"][0])] == before[geo.unit_at(0): geo.unit_at(img["app"][0])]
        assert len(after) == geo.unit_at(len(idx) // 32)
    # an idle sync is a commit with an empty delta
    idx.sync(str(path))
    img, _ = check_file(T, idx, path, 0)
    assert img["gen"] == 6 and img["app"][0] == img["app"][1]


def test_sync_removals_ride_the_header_then_materialise(T, tmp_path):
    dim, bits = 128, 2
    path = tmp_path / "ids.tvim"
    n = 200
    idx = T.IdMapIndex(dim, bits)
    ids = (np.arange(n) * 7 + 1_000_000).astype(np.uint64)
    idx.add_with_ids(anisotropic(n, dim, seed=2), ids)
    idx.sync(str(path))
    units_before = path.read_bytes()
    geo = R.read(T._native.load(), units_before)["geo"]
    # remove rows of blocks 0 and 3: the holes take the bytes of the last rows
    for victim in (ids[5], ids[100], ids[7]):
        assert idx.remove(int(victim))
    assert idx._sync_state()[3] > 0
    idx.sync(str(path))
    img, _ = check_file(T, idx, path, 1)
    assert img["gen"] == 1 and img["mat"] == []
    assert set(img["pending"]) >= {5, 7, 100} and all(s < (len(idx) // 32) * 32 for s in img["pending"])
    after = path.read_bytes()
    # committed units are not touched by the sync that commits the removal
    live_units = min(n // 32, len(idx) // 32)
    assert after[geo.unit_at(0): geo.unit_at(live_units)] == units_before[geo.unit_at(0): geo.unit_at(live_units)]
    assert idx._sync_state()[2] == len(img["pending"])
    # the next sync writes the ops into their units
    idx.sync(str(path))
    img2, back = check_file(T, idx, path, 1)
    assert img2["gen"] == 2 and img2["pending"] == [] and img2["mat"] == sorted({s // 32 for s in img["pending"]})
    assert back._sync_state()[0]                       # loaded from a claimed file: bound
    # a unit dirtied again before it is materialised keeps all its ops in the header
    assert idx.remove(int(idx.ids()[3]))
    idx.sync(str(path))
    assert idx.remove(int(idx.ids()[4]))               # same unit, dirtied again
    idx.sync(str(path))
    img3, _ = check_file(T, idx, path, 1)
    assert img3["mat"] == [] and {3, 4} <= set(img3["pending"])


def test_loaded_index_keeps_syncing_forward(T, tmp_path):
    dim, bits = 256, 4
    path = tmp_path / "b.tv"
    a = T.TurboQuantIndex(dim, bits)
    a.add(anisotropic(100, dim, seed=3))
    a.sync(str(path))
    a.swap_remove(10)
    a.sync(str(path))                                   # generation 1 with a pending op
    b = T.TurboQuantIndex.load(str(path))
    assert b._sync_state() == (True, 1, 1, 0)
    b.add(anisotropic(40, dim, seed=4))
    b.sync(str(path))
    img, _ = check_file(T, b, path, 0)
    assert img["gen"] == 2 and img["mat"] == [0] and img["pending"] == []
    # the first writer's cursor now points at a commit that is no longer the newest: refused
    a.add(anisotropic(1, dim, seed=5))
    with pytest.raises(OSError, match="another writer"):
        a.sync(str(path))
    # a snapshot is loaded unbound; the first sync to it rewrites and claims it
    snap = tmp_path / "snap.tv"
    b.write(str(snap))
    c = T.TurboQuantIndex.load(str(snap))
    assert c._sync_state()[0] is False
    c.sync(str(snap))
    assert R.read(T._native.load(), snap.read_bytes())["nonce"] != 0 and c._sync_state()[:2] == (True, 0)


def test_full_rewrite_cases(T, tmp_path):
    dim, bits = 128, 4
    path = tmp_path / "c.tv"
    lib = T._native.load()
    idx = T.TurboQuantIndex(dim, bits)
    x = anisotropic(40_000, dim, seed=6)
    idx.add(x)
    idx.sync(str(path))
    nonce0 = R.read(lib, path.read_bytes())["nonce"]
    # more dirtied committed slots than one header carries: rewritten whole under a new identity
    for s in range(0, 33_000, 31):
        idx.swap_remove(s)
    assert idx._sync_state()[3] > 1024
    idx.sync(str(path))
    img, _ = check_file(T, idx, path, 0)
    assert img["gen"] == 0 and img["nonce"] not in (0, nonce0) and idx._sync_state() == (True, 0, 0, 0)
    # a refit rewrites every stored code: the next sync compacts
    idx.add(x[:10])
    idx.sync(str(path))
    assert R.read(lib, path.read_bytes())["gen"] == 1
    idx.calibrate(x[:5000])
    idx.sync(str(path))
    img, _ = check_file(T, idx, path, 0)
    assert img["gen"] == 0 and img["shift"].size == dim
    # another path: full write there, and the binding moves
    other = tmp_path / "d.tv"
    idx.sync(str(other))
    check_file(T, idx, other, 0)
    idx.add(x[:3])
    idx.sync(str(other))
    assert R.read(lib, other.read_bytes())["gen"] == 1
    # the file was deleted: written again whole
    os.remove(other)
    idx.sync(str(other))
    assert R.read(lib, other.read_bytes())["gen"] == 0
    with pytest.raises(OSError):
        T.TurboQuantIndex(bit_width=4).sync(str(tmp_path / "lazy.tv"))


def test_torn_commit_falls_back_and_is_repaired(T, tmp_path):
    dim, bits = 128, 4
    path = tmp_path / "e.tv"
    lib = T._native.load()
    idx = T.TurboQuantIndex(dim, bits)
    idx.add(anisotropic(64, dim, seed=7))
    idx.sync(str(path))
    idx.add(anisotropic(10, dim, seed=8))
    idx.sync(str(path))                                 # generation 1 in slot 1
    good = path.read_bytes()
    idx.add(anisotropic(40, dim, seed=9))
    state_before = idx.to_bytes()
    idx.sync(str(path))                                 # generation 2 in slot 0, appends unit 2
    done = path.read_bytes()
    geo = R.read(lib, done)["geo"]
    # (a) the header landed, its data did not: the delta check refuses the commit
    torn = bytearray(done)
    torn[geo.unit_at(2): geo.unit_at(3)] = bytes(geo.unit_len)
    img = R.read(lib, bytes(torn))
    assert img["gen"] == 1 and img["newest"] == 2 and img["n"] == 74
    path.write_bytes(bytes(torn))
    back = T.TurboQuantIndex.load(str(path))
    assert len(back) == 74 and back._sync_state()[:2] == (True, 1)
    # the recovered index syncs generation 2 again, into the slot that still holds the rejected header: the
    # plan opens with the repair barrier, and the result is a clean generation 2
    back.add(anisotropic(40, dim, seed=9))
    assert back.to_bytes() == state_before
    back.sync(str(path))
    img = R.read(lib, path.read_bytes())
    assert img["gen"] == 2 and img["newest"] == 2 and img["n"] == 114
    check_file(T, back, path, 0)
    # (b) a header torn in the middle fails its checksum: the other slot wins
    torn = bytearray(done)
    at = geo.hdr_at(0)
    torn[at + 20] ^= 0xFF
    assert R.read(lib, bytes(torn))["gen"] == 1
    path.write_bytes(bytes(torn))
    assert len(T.TurboQuantIndex.load(str(path))) == 74
    # (c) the untouched previous image still loads as it was
    assert R.read(lib, good)["n"] == 74


def test_sync_keeps_search_results(T, tmp_path):
    dim, bits = 256, 4
    path = tmp_path / "f.tvim"
    idx = T.IdMapIndex(dim, bits)
    n = 3000
    ids = np.random.default_rng(1).permutation(np.arange(10_000, 10_000 + n)).astype(np.uint64)
    idx.add_with_ids(anisotropic(n, dim, seed=11), ids)
    idx.sync(str(path))
    rng = np.random.default_rng(2)
    for round_ in range(4):
        for victim in rng.choice(idx.ids(), 40, replace=False):
            idx.remove(int(victim))
        fresh = (np.arange(25) + 100_000 + 100 * round_).astype(np.uint64)
        idx.add_with_ids(anisotropic(25, dim, seed=20 + round_), fresh)
        idx.sync(str(path))
        _, back = check_file(T, idx, path, 1)
        q = anisotropic(8, dim, seed=11, offset=50)
        s0, i0 = idx.search(q, 10)
        s1, i1 = back.search(q, 10)
        assert np.array_equal(i0, i1) and np.array_equal(s0, s1)


# ---- the scenarios of the reference's own tests/sync_v7.rs, replayed through the same calls ----

DIM = 128


def fresh_index(T, bits=4, calib_seed=30, kind=0):
    idx = (T.IdMapIndex if kind else T.TurboQuantIndex)(DIM, bits)
    idx.calibrate(anisotropic(1024, DIM, seed=calib_seed))
    return idx


def same_as_loaded(T, idx, path, queries_seed=999, k=10):
    loaded = type(idx).load(str(path))
    assert loaded.to_bytes() == idx.to_bytes()
    q = anisotropic(8, DIM, seed=queries_seed)
    a, b = idx.search(q, min(k, len(idx))), loaded.search(q, min(k, len(idx)))
    assert np.array_equal(a[1], b[1]) and np.array_equal(a[0], b[0])
    return loaded


def test_remove_then_readd_across_a_block_boundary_between_syncs(T, tmp_path):
    """sync_v7.rs:69: a shrink below a block boundary and a re-add into the dipped region between two syncs."""
    path = tmp_path / "gap1.tv"
    idx = fresh_index(T)
    idx.add(anisotropic(64, DIM, seed=31))
    idx.sync(str(path))
    while len(idx) > 24:
        idx.swap_remove(0)
    idx.add(anisotropic(8, DIM, seed=32))
    idx.sync(str(path))
    same_as_loaded(T, idx, path)
    path2 = tmp_path / "gap1b.tv"
    idx = fresh_index(T, calib_seed=33)
    idx.add(anisotropic(64, DIM, seed=34))
    idx.sync(str(path2))
    idx.swap_remove(10)
    idx.add(anisotropic(1, DIM, seed=35))
    idx.sync(str(path2))
    same_as_loaded(T, idx, path2)


def test_interleaved_lifecycle_and_sync_cost(T, tmp_path):
    """sync_v7.rs:102 and :231: syncs stay proportional to the change, also after a reload."""
    path = tmp_path / "life.tv"
    idx = fresh_index(T, calib_seed=1)
    idx.add(anisotropic(100, DIM, seed=2))
    idx.sync(str(path))
    full = path.stat().st_size
    idx.add(anisotropic(37, DIM, seed=3))
    idx.swap_remove(5)
    idx.swap_remove(len(idx) - 1)
    idx.swap_remove(70)
    before = path.stat().st_size
    idx.sync(str(path))
    assert path.stat().st_size - before < full // 2
    idx = same_as_loaded(T, idx, path)
    idx.add(anisotropic(64, DIM, seed=4))
    idx.swap_remove(0)
    before = path.stat().st_size
    idx.sync(str(path))
    assert path.stat().st_size - before < before // 2
    same_as_loaded(T, idx, path)
    # a 32-row sync appends one unit; a single removal appends nothing
    idx = fresh_index(T, calib_seed=20)
    path = tmp_path / "cost.tv"
    idx.add(anisotropic(512, DIM, seed=21))
    idx.sync(str(path))
    idx.add(anisotropic(32, DIM, seed=22))
    before = path.stat().st_size
    idx.sync(str(path))
    assert path.stat().st_size - before < 2500
    idx.swap_remove(3)
    before = path.stat().st_size
    idx.sync(str(path))
    assert path.stat().st_size == before
    same_as_loaded(T, idx, path)


def test_shrink_below_the_watermark_then_regrow(T, tmp_path):
    """sync_v7.rs:154"""
    path = tmp_path / "shrink.tv"
    idx = fresh_index(T, calib_seed=5)
    idx.add(anisotropic(200, DIM, seed=6))
    idx.sync(str(path))
    while len(idx) > 40:
        idx.swap_remove(len(idx) // 2)
    idx.sync(str(path))
    assert len(same_as_loaded(T, idx, path, k=5)) == 40
    idx.add(anisotropic(100, DIM, seed=7))
    idx.sync(str(path))
    assert len(same_as_loaded(T, idx, path)) == 140


def test_write_over_a_synced_file_and_foreign_writers(T, tmp_path):
    """sync_v7.rs:267, :284, :421, :310"""
    path = tmp_path / "swsync.tv"
    idx = fresh_index(T)
    idx.add(anisotropic(50, DIM, seed=31))
    idx.sync(str(path))
    idx.write(str(path))                          # a snapshot replaces the synced file: the cursor is stale
    idx.add(anisotropic(10, DIM, seed=32))
    idx.sync(str(path))                           # detected, written whole again
    assert idx._sync_state()[:2] == (True, 0)
    same_as_loaded(T, idx, path)
    # two independent writers, both at generation 0: the file identity tells them apart
    path = tmp_path / "noncegen.tv"
    a = fresh_index(T, calib_seed=90)
    a.add(anisotropic(40, DIM, seed=91))
    a.sync(str(path))
    b = fresh_index(T, calib_seed=92)
    b.add(anisotropic(20, DIM, seed=93))
    b.sync(str(path))
    a.add(anisotropic(1, DIM, seed=94))
    with pytest.raises(OSError, match="another writer"):
        a.sync(str(path))
    assert T.TurboQuantIndex.load(str(path)).to_bytes() == b.to_bytes()
    # trailing garbage of a torn writer does not disturb a matching cursor
    path = tmp_path / "shed.tv"
    idx = fresh_index(T, calib_seed=37)
    idx.add(anisotropic(40, DIM, seed=38))
    idx.sync(str(path))
    with open(path, "ab") as f:
        f.write(b"SEG1garbage-from-a-torn-sync\x00\x00\x00")
    idx.add(anisotropic(12, DIM, seed=39))
    idx.sync(str(path))
    assert idx._sync_state()[1] == 1
    same_as_loaded(T, idx, path)


def test_a_failed_first_sync_cleans_up_its_temp(T, tmp_path):
    """sync_v7.rs:335"""
    path = tmp_path / "cleanup"
    path.mkdir()
    (path / "occupied").write_bytes(b"x")
    idx = fresh_index(T, calib_seed=40)
    idx.add(anisotropic(40, DIM, seed=41))
    with pytest.raises(OSError):
        idx.sync(str(path))
    assert not [p for p in os.listdir(tmp_path) if ".tmp." in p]
    good = tmp_path / "good.tv"
    idx.sync(str(good))
    same_as_loaded(T, idx, good)


def test_churn_does_not_grow_the_file(T, tmp_path):
    """sync_v7.rs:364"""
    path = tmp_path / "churn.tv"
    idx = fresh_index(T, calib_seed=42)
    idx.add(anisotropic(64, DIM, seed=43))
    idx.sync(str(path))
    full, peak = path.stat().st_size, 0
    for i in range(120):
        idx.add(anisotropic(1, DIM, seed=100 + i))
        idx.swap_remove(len(idx) - 2)
        idx.sync(str(path))
        peak = max(peak, path.stat().st_size)
    assert peak < full + full // 4
    same_as_loaded(T, idx, path)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("n", [50, 64])
@pytest.mark.parametrize("kind", [0, 1])
def test_every_bit_width_round_trips(T, tmp_path, bits, n, kind):
    """sync_v7.rs:392 and sync_v7_idmap.rs, both index kinds"""
    path = tmp_path / "bw.tv"
    idx = fresh_index(T, bits=bits, calib_seed=80, kind=kind)
    x = anisotropic(n, DIM, seed=81)
    if kind:
        idx.add_with_ids(x, np.arange(n, dtype=np.uint64) + 500)
    else:
        idx.add(x)
    idx.sync(str(path))
    same_as_loaded(T, idx, path, k=5)
    more = anisotropic(3, DIM, seed=82)
    if kind:
        idx.remove(505)
        idx.add_with_ids(more, np.arange(3, dtype=np.uint64) + 9000)
    else:
        idx.swap_remove(5)
        idx.add(more)
    idx.sync(str(path))
    same_as_loaded(T, idx, path, k=5)


def _sync_writes(lib, before: bytes, after: bytes):
    """The positioned writes of the sync that turned `before` into `after`, in the order the plan issues them:
    materialised units, appended units, then the commit header's used prefix (io_v7.rs:738-762)."""
    img = R.read(lib, after)
    geo = img["geo"]
    writes = [(geo.unit_at(u), after[geo.unit_at(u): geo.unit_at(u + 1)]) for u in img["mat"] + list(range(*img["app"]))]
    at = geo.hdr_at(img["slot"])
    writes.append((at, after[at: at + img["used"]]))
    # nothing else changed
    rebuilt = bytearray(before.ljust(len(after), b"\0"))
    for off, data in writes:
        rebuilt[off: off + len(data)] = data
    assert bytes(rebuilt) == after
    return writes


def test_every_sampled_tear_recovers_the_old_or_the_new_commit(T, tmp_path):
    """The reference's torn-write harness (lib.rs:3446-4620) applies every prefix of every planned write; here the
    writes are cut at every write boundary, around it, and at random bytes, and the file must load as exactly
    the previous commit or exactly the new one - with the library's loader and with the independent reader."""
    lib = T._native.load()
    path = tmp_path / "tear.tvim"
    dim, bits = 64, 2
    idx = T.IdMapIndex(dim, bits)
    idx.add_with_ids(anisotropic(150, dim, seed=1), np.arange(150, dtype=np.uint64) + 10)
    idx.sync(str(path))
    rng = np.random.default_rng(3)
    next_id = 1000
    for step in range(4):
        before = path.read_bytes()
        old = R.read(lib, before)
        for victim in rng.choice(idx.ids()[:96], 3, replace=False):   # holes inside committed units
            idx.remove(int(victim))
        rows = int(rng.integers(20, 70))
        idx.add_with_ids(anisotropic(rows, dim, seed=50 + step), np.arange(rows, dtype=np.uint64) + next_id)
        next_id += rows
        idx.sync(str(path))
        after = path.read_bytes()
        new = R.read(lib, after)
        assert new["gen"] == old["gen"] + 1
        writes = _sync_writes(lib, before, after)
        total = sum(len(d) for _, d in writes)
        cuts, acc = {0, total}, 0
        for _, d in writes:
            cuts.update(c for c in (acc - 1, acc + 1, acc + 7, acc + 8, acc + 9, acc + len(d) // 2) if 0 <= c <= total)
            acc += len(d)
            cuts.update({acc - 5, acc - 4, acc - 1})
        cuts.update(int(c) for c in rng.integers(0, total, 40))
        torn_path = tmp_path / "torn.tvim"
        for n_cut, cut in enumerate(sorted(cuts)):
            img = bytearray(before.ljust(len(after), b"\0")) if cut else bytearray(before)
            left = cut
            for off, data in writes:
                take = min(left, len(data))
                img[off: off + take] = data[:take]
                left -= take
                if not left:
                    break
            got = R.read(lib, bytes(img))
            want = new if got["gen"] == new["gen"] else old
            assert got["gen"] in (old["gen"], new["gen"])
            assert got["n"] == want["n"] and np.array_equal(got["codes"], want["codes"])
            assert np.array_equal(got["scales"], want["scales"]) and np.array_equal(got["ids"], want["ids"])
            if cut == total:
                assert got["gen"] == new["gen"]
            if n_cut % 9 == 0 or cut == total:                        # the library's loader on a subset
                torn_path.write_bytes(bytes(img))
                back = T.IdMapIndex.load(str(torn_path))
                assert len(back) == want["n"] and np.array_equal(back.ids(), want["ids"])
                assert np.array_equal(np.asarray(back.scales()), want["scales"])


def test_sync_errors_name_the_path(T, tmp_path):
    """turbovec-python/tests/test_sync.py:67-80"""
    idx = fresh_index(T, calib_seed=10)
    idx.add(anisotropic(8, DIM, seed=11))
    missing = str(tmp_path / "no-such-dir" / "index.tv")
    with pytest.raises(OSError) as exc:
        idx.sync(missing)
    assert "no-such-dir" in str(exc.value)
    assert idx._sync_state()[0] is False
    with pytest.raises(OSError):
        T.TurboQuantIndex(bit_width=4).sync(str(tmp_path / "never-written.tv"))
