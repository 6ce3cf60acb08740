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

from turbovec_b200.sharded import ShardedIndex, SlotMap, merge_topk


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
        assert results[rank] == {"plain": True, "masked": True, "remove": True}, results[rank]
