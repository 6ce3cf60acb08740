"""Incremental `sync` (lib.rs:1737, io_v7.rs plan_incremental / run_sync / cursor_state): after every sync the file,
read by an independent restatement of the reference's loader, holds exactly the live index; commits alternate
header slots; removals ride the header as redo ops and are written into place by a later sync; a torn commit
falls back to the previous one; foreign files are refused."""
import os
import struct

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
