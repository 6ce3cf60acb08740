"""Slot-sharded index over several GPUs: one process per GPU, `torch.distributed` for the exchange.

The reference scans block ranges on different cores and merges per-range candidates by
(score descending, slot ascending) (turbovec/src/search.rs:3455-3499, 4285-4298).  Here the ranges live on
different GPUs.  Global slot numbering is kept (it carries the tie-break, the masks and swap_remove's
semantics); ownership is arithmetic:

    global block b = slot // 32,  chunk = b // C,  owner = chunk % G,
    local block    = (chunk // G) * C + b % C                       (C = chunk_blocks, G = world size)

so appends stay balanced at any length.  Every rank makes the same calls with the same arguments (SPMD).
A search is: local scan on every rank -> one all-gather of the per-rank top-k (score, global slot) -> the same
merge on every rank.  Removal moves the globally last row into the hole; when the two rows live on different
ranks the row (ngroups code bytes + one scale) is broadcast from its owner.
"""
from __future__ import annotations

import numpy as np

BLOCK = 32


class SlotMap:
    """Pure arithmetic between global slots and (rank, local slot)."""

    def __init__(self, world: int, chunk_blocks: int = 1024):
        self.world, self.cb = int(world), int(chunk_blocks)
        self.chunk_slots = self.cb * BLOCK

    def owner(self, slot):
        return (np.asarray(slot) // self.chunk_slots) % self.world

    def to_local(self, slot):
        slot = np.asarray(slot)
        chunk = slot // self.chunk_slots
        return (chunk // self.world) * self.chunk_slots + slot % self.chunk_slots

    def to_global(self, rank: int, local):
        local = np.asarray(local)
        lchunk = local // self.chunk_slots
        return (lchunk * self.world + rank) * self.chunk_slots + local % self.chunk_slots

    def local_len(self, rank: int, n_total: int) -> int:
        """Number of global slots < n_total owned by `rank`."""
        full_rounds, rem = divmod(n_total, self.chunk_slots * self.world)
        extra = min(max(rem - rank * self.chunk_slots, 0), self.chunk_slots)
        return full_rounds * self.chunk_slots + extra

    def runs(self, start: int, count: int):
        """Splits global slots [start, start+count) into (owner, offset_in_batch, length) runs."""
        out, pos, end = [], start, start + count
        while pos < end:
            nxt = min(end, (pos // self.chunk_slots + 1) * self.chunk_slots)
            out.append((int(self.owner(pos)), pos - start, nxt - pos))
            pos = nxt
        return out


def merge_topk(torch, scores, slots, k: int):
    """[nq, m] candidates -> best k under (score desc, slot asc).  Padding entries carry score -inf and the
    largest slot, so they sort last."""
    order = torch.argsort(slots, dim=1, stable=True)
    s, i = torch.gather(scores, 1, order), torch.gather(slots, 1, order)
    order = torch.argsort(s, dim=1, descending=True, stable=True)
    return torch.gather(s, 1, order)[:, :k].contiguous(), torch.gather(i, 1, order)[:, :k].contiguous()


_PAD_SLOT = np.iinfo(np.int64).max


class ShardedIndex:
    """Positional index sharded over the ranks of a process group.  Mirrors TurboQuantIndex's add / search /
    swap_remove / __len__ with global slot numbers.  `local_factory(dim, bit_width)` builds the per-rank index
    (default: turbovec_b200.TurboQuantIndex on this rank's GPU)."""

    def __init__(self, dim: int, bit_width: int = 4, *, group=None, device=None, chunk_blocks: int = 1024,
                 local_factory=None):
        import torch
        import torch.distributed as dist
        self._torch, self._dist, self._group = torch, dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.map = SlotMap(self.world, chunk_blocks)
        self.dim, self.bit_width, self.n_total = dim, bit_width, 0
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = device
        if local_factory is None:
            from . import TurboQuantIndex
            local_factory = lambda d, b: TurboQuantIndex(d, b, device=device.index or 0)  # noqa: E731
        self.local = local_factory(dim, bit_width)

    def __len__(self) -> int:
        return self.n_total

    # ---- ingest: each rank encodes the rows whose global slot it owns; no exchange ----
    def add(self, vectors: np.ndarray) -> None:
        n = vectors.shape[0]
        mine = [vectors[off:off + ln] for owner, off, ln in self.map.runs(self.n_total, n) if owner == self.rank]
        if mine:
            self.local.add(np.ascontiguousarray(np.concatenate(mine) if len(mine) > 1 else mine[0]))
        self.n_total += n
        assert len(self.local) == self.map.local_len(self.rank, self.n_total)

    # ---- search: local scan, one all-gather, identical merge everywhere ----
    def search(self, queries: np.ndarray, k: int, *, mask=None):
        torch, dist = self._torch, self._dist
        nq = queries.shape[0]
        n_local = len(self.local)
        local_mask = None
        if mask is not None:
            if mask.size != self.n_total:
                raise ValueError(f"mask length {mask.size} does not match index size {self.n_total}")
            local_mask = np.ascontiguousarray(mask[self.map.to_global(self.rank, np.arange(n_local))]) if n_local else None
        if n_local and (local_mask is None or local_mask.any()):
            s, i = self.local.search(queries, k, mask=local_mask) if local_mask is not None else self.local.search(queries, k)
            gi = self.map.to_global(self.rank, i).astype(np.int64)
        else:
            s, gi = np.empty((nq, 0), np.float32), np.empty((nq, 0), np.int64)
        ps = np.full((nq, k), -np.inf, np.float32)
        pi = np.full((nq, k), _PAD_SLOT, np.int64)
        ps[:, : s.shape[1]], pi[:, : gi.shape[1]] = s, gi
        ts, ti = torch.from_numpy(ps).to(self.device), torch.from_numpy(pi).to(self.device)
        if self.world > 1:
            gs = [torch.empty_like(ts) for _ in range(self.world)]
            gl = [torch.empty_like(ti) for _ in range(self.world)]
            dist.all_gather(gs, ts, group=self._group)
            dist.all_gather(gl, ti, group=self._group)
            ts, ti = torch.cat(gs, 1), torch.cat(gl, 1)
        ms, mi = merge_topk(torch, ts, ti, k)
        ms, mi = ms.cpu().numpy(), mi.cpu().numpy()
        k_eff = int((mi[0] != _PAD_SLOT).sum()) if nq else min(k, self.n_total)
        return ms[:, :k_eff].copy(), mi[:, :k_eff].copy()

    # ---- removal: the globally last row moves into the hole (turbovec/src/lib.rs:2864-3028) ----
    def swap_remove(self, idx: int) -> int:
        torch, dist = self._torch, self._dist
        if not 0 <= idx < self.n_total:
            raise IndexError(f"index {idx} out of bounds (n_vectors = {self.n_total})")
        last = self.n_total - 1
        hole_owner, last_owner = int(self.map.owner(idx)), int(self.map.owner(last))
        hole_local, last_local = int(self.map.to_local(idx)), int(self.map.to_local(last))
        if hole_owner == last_owner:
            if self.rank == hole_owner:
                moved = self.local.swap_remove(hole_local)
                assert moved == last_local
        else:
            nbytes = self.local.row_bytes()
            buf = torch.zeros(nbytes + 4, dtype=torch.uint8, device=self.device)
            if self.rank == last_owner:
                codes, scale = self.local.get_row(last_local)
                row = np.concatenate([codes, np.frombuffer(np.float32(scale).tobytes(), np.uint8)])
                buf = torch.from_numpy(row).to(self.device)
            dist.broadcast(buf, src=dist.get_global_rank(self._group, last_owner) if self._group else last_owner, group=self._group)
            if self.rank == hole_owner:
                row = buf.cpu().numpy()
                self.local.set_row(hole_local, row[:nbytes].copy(), float(np.frombuffer(row[nbytes:].tobytes(), np.float32)[0]))
            if self.rank == last_owner:
                self.local.swap_remove(last_local)          # drops the (moved) last row
        self.n_total = last
        return last
