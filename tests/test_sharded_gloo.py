"""Host-side logic of the slot-sharded index, run as two gloo ranks on CPU: slot arithmetic, add routing,
the all-gather + merge, cross-rank swap_remove.  The per-rank index is a numpy stand-in with the same
interface as TurboQuantIndex (exact inner products), so no GPU is needed."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from turbovec_b200.sharded import IdTable, ShardedIdMapIndex, ShardedIndex, SlotMap, merge_topk, pack_mask_words


def test_slot_map_roundtrip_and_balance():
    for world in (1, 2, 4, 8):
        m = SlotMap(world, chunk_blocks=4)          # 128 slots per chunk
        slots = np.arange(5000)
        owner, local = m.owner(slots), m.to_local(slots)
        for r in range(world):
            mine = slots[owner == r]
            assert np.array_equal(m.to_global(r, local[owner == r]), mine)
            assert np.array_equal(np.sort(local[owner == r]), np.arange(mine.size))   # dense local numbering
            for n in (0, 1, 127, 128, 129, 1000, 5000):
                assert m.local_len(r, n) == int((owner[:n] == r).sum())
        runs = m.runs(100, 700)
        assert sum(r[2] for r in runs) == 700 and runs[0][1] == 0
        for o, off, ln in runs:
            assert np.all(owner[100 + off: 100 + off + ln] == o)


def test_merge_orders_by_score_then_slot():
    s = torch.tensor([[1.0, 3.0, 3.0, -float("inf"), 2.0, 3.0]])
    i = torch.tensor([[7, 9, 4, np.iinfo(np.int64).max, 1, 6]])
    ms, mi = merge_topk(torch, s, i, 4)
    assert mi.tolist() == [[4, 6, 9, 1]] and ms.tolist() == [[3.0, 3.0, 3.0, 2.0]]


class FakeLocal:
    """Same interface as TurboQuantIndex, exact fp32 inner products, rows kept in numpy."""

    def __init__(self, dim, bits):
        self.dim, self.x = dim, np.empty((0, dim), np.float32)

    def __len__(self):
        return self.x.shape[0]

    def add(self, v):
        self.x = np.concatenate([self.x, v])

    def search(self, q, k, mask=None):
        sc = q @ self.x.T
        if mask is not None:
            sc = np.where(mask[None, :], sc, -np.inf)
        ke = min(k, len(self) if mask is None else int(mask.sum()))
        order = np.lexsort((np.broadcast_to(np.arange(len(self)), sc.shape), -sc), axis=1)[:, :ke]
        return np.take_along_axis(sc, order, 1).astype(np.float32), order.astype(np.int64)

    def swap_remove(self, idx):
        last = len(self) - 1
        self.x[idx] = self.x[last]
        self.x = self.x[:last]
        return last

    def row_bytes(self):
        return self.dim * 4

    def get_row(self, slot):
        return np.frombuffer(self.x[slot].tobytes(), np.uint8).copy(), 1.0

    def set_row(self, slot, groups, scale):
        self.x[slot] = np.frombuffer(groups.tobytes(), np.float32)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dim, n = 16, 700
        rng = np.random.default_rng(0)
        x = rng.standard_normal((n, dim)).astype(np.float32)
        q = rng.standard_normal((5, dim)).astype(np.float32)
        idx = ShardedIndex(dim, 4, device=torch.device("cpu"), chunk_blocks=2, local_factory=FakeLocal)
        for a, b in ((0, 1), (1, 100), (100, 333), (333, 700)):     # ragged appends crossing chunk borders
            idx.add(x[a:b])
        ref = FakeLocal(dim, 4)
        ref.add(x)
        out = {}
        s, i = idx.search(q, 10)
        rs, ri = ref.search(q, 10)
        out["plain"] = bool(np.array_equal(i, ri) and np.allclose(s, rs))
        mask = rng.random(n) < 0.02
        s, i = idx.search(q, 10, mask=mask)
        rs, ri = ref.search(q, 10, mask=mask)
        out["masked"] = bool(np.array_equal(i, ri) and s.shape == (5, min(10, int(mask.sum()))))
        ok = True
        for victim in (5, 650, 64, 0, 300):                           # same-rank and cross-rank moves
            moved = idx.swap_remove(victim)
            ok &= moved == ref.swap_remove(victim)
            s, i = idx.search(q, 7)
            rs, ri = ref.search(q, 7)
            ok &= bool(np.array_equal(i, ri) and np.allclose(s, rs))
        out["remove"] = bool(ok) and len(idx) == len(ref)

        # id-mapped: replicated id tables, allowlists, removal by id (same-rank and cross-rank moves)
        ids = (rng.permutation(n) + 10**9).astype(np.uint64)
        im = ShardedIdMapIndex(dim, 4, device=torch.device("cpu"), chunk_blocks=2, local_factory=FakeLocal)
        for a, b in ((0, 130), (130, 131), (131, 700)):
            im.add_with_ids(x[a:b], ids[a:b])
        ref2, ref_ids = FakeLocal(dim, 4), list(ids)
        ref2.add(x)
        ok = True
        s, got = im.search(q, 10)
        rs, ri = ref2.search(q, 10)
        ok &= bool(np.array_equal(got, np.array(ref_ids, np.uint64)[ri]) and np.allclose(s, rs))
        allow = np.ascontiguousarray(ids[::9])
        s, got = im.search(q, 100, allowlist=allow)
        amask = np.isin(np.array(ref_ids, np.uint64), allow)
        rs, ri = ref2.search(q, 100, mask=amask)
        ok &= bool(s.shape == (5, min(100, allow.size)) and np.array_equal(got, np.array(ref_ids, np.uint64)[ri]))
        for victim in (int(ids[3]), int(ids[690]), int(ids[64]), int(ids[699])):
            ok &= im.remove(victim) and not im.contains(victim) and not im.remove(victim)
            slot = ref_ids.index(victim)
            last = ref2.swap_remove(slot)
            ref_ids[slot] = ref_ids[last]
            ref_ids.pop()
            s, got = im.search(q, 7)
            rs, ri = ref2.search(q, 7)
            ok &= bool(np.array_equal(got, np.array(ref_ids, np.uint64)[ri]) and np.allclose(s, rs))
        ok &= bool(np.array_equal(im.ids(), np.array(ref_ids, np.uint64)))
        try:
            im.add_with_ids(x[:2], np.array([ref_ids[0], 5], np.uint64))     # already present: nothing changes
            ok = False
        except ValueError:
            ok &= len(im) == len(ref_ids) and not im.contains(5)
        try:
            im.search(q, 3, allowlist=np.array([12345], np.uint64))
            ok = False
        except KeyError:
            pass
        out["idmap"] = bool(ok)
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_sharded_index_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert len(results) == 2
    for rank in (0, 1):
        assert results[rank] == {"plain": True, "masked": True, "remove": True, "idmap": True}, results[rank]


def test_id_table_semantics():
    t = IdTable()
    t.add(np.array([10, 11, 12, 13], np.uint64))
    assert len(t) == 4 and t.contains(12) and not t.contains(9)
    with pytest.raises(ValueError, match="already present"):
        t.add(np.array([20, 11], np.uint64))
    with pytest.raises(ValueError, match="twice in the batch"):
        t.add(np.array([20, 20], np.uint64))
    assert len(t) == 4 and not t.contains(20)
    assert t.remove(11) == (True, 1, 3)                    # the last slot's id moves into slot 1
    assert np.array_equal(t.ids(), np.array([10, 13, 12], np.uint64))
    assert t.remove(11) == (False, 0, 0)
    assert np.array_equal(t.resolve(np.array([12, 10, 12], np.uint64)), np.array([2, 0, 2], np.uint64))
    with pytest.raises(KeyError, match="11"):
        t.resolve(np.array([10, 11, 99], np.uint64))       # the first unknown id in list order
    with pytest.raises(ValueError, match="empty"):
        t.resolve(np.array([], np.uint64))
    assert np.array_equal(t.ids_of(np.array([[2, 0]], np.int64)), np.array([[12, 10]], np.uint64))
    t.truncate(1)
    assert np.array_equal(t.ids(), np.array([10], np.uint64)) and not t.contains(13)


def test_local_mask_words_gather():
    for world in (1, 2, 3):
        m = SlotMap(world, chunk_blocks=2)                  # 64 slots per chunk: one word
        for n in (1, 63, 64, 65, 200, 64 * world * 3, 64 * world * 3 + 5):
            mask = np.random.default_rng(n).random(n) < 0.4
            flags = torch.zeros(((n + 63) // 64) * 64, dtype=torch.uint8)
            flags[:n] = torch.from_numpy(mask.view(np.uint8))
            words = pack_mask_words(torch, flags)
            for r in range(world):
                n_local = m.local_len(r, n)
                got = m.local_mask_words(torch, words, r, n)
                want = np.zeros(((n_local + 63) // 64) * 64, bool)
                want[:n_local] = mask[m.to_global(r, np.arange(n_local))]
                want_words = pack_mask_words(torch, torch.from_numpy(want.view(np.uint8)))
                assert torch.equal(got, want_words)
