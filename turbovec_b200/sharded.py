"""Slot-sharded index over several GPUs: one process per GPU, `torch.distributed` for the exchange.

The reference scans block ranges on different cores and merges per-range candidates by
(score descending, slot ascending) (turbovec/src/search.rs:3455-3499, 4285-4298).  Here the ranges live on
different GPUs.  Global slot numbering is kept (it carries the tie-break, the masks and swap_remove's
semantics); ownership is arithmetic:

    global block b = slot // 32,  chunk = b // C,  owner = chunk % G,
    local block    = (chunk // G) * C + b % C                       (C = chunk_blocks, G = world size)

so appends stay balanced at any length.  Every rank makes the same calls with the same arguments (SPMD).
A search is: the local scan on every rank with results as 64-bit keys (tv_search_device_keys) -> ONE all-gather of
`nq x k` keys per rank -> one merge kernel per rank (tv_merge_keys_device_chunked, which also turns local slots
into global ones) -- nothing passes through host memory.  Removal moves the globally last row into the hole; when
the two rows live on different ranks the row (ngroups code bytes + one scale) is broadcast from its owner.

`ShardedIndex` mirrors TurboQuantIndex (positional), `ShardedIdMapIndex` mirrors IdMapIndex: ids live in a
replicated host table (tv_idtable_*), exactly the two tables the reference keeps around its inner index
(turbovec/src/id_map.rs:221-272), and never reach the device.

Process groups on CPU (gloo) are supported for the routing, masking and merge logic with a caller-supplied
per-rank index (`local_factory`): the merge then runs on host tensors.  On a GPU the per-rank index is this
library's and the device path is the only one.
"""
from __future__ import annotations

import ctypes as C

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

    def local_mask_words(self, torch, words, rank: int, n_total: int):
        """The mask words of `rank`'s slots out of the global packed mask (a 1-D int64 tensor, bit i of word
        i // 64 = global slot i): whole chunks are runs of chunk_slots / 64 words, so this is one strided gather."""
        wpc = self.chunk_slots // 64                     # words per chunk
        n_local = self.local_len(rank, n_total)
        if n_local == 0:
            return words.new_zeros(0)
        stride = wpc * self.world
        rounds = (words.numel() + stride - 1) // stride
        if rounds * stride != words.numel():
            padded = words.new_zeros(rounds * stride)
            padded[: words.numel()] = words
            words = padded
        local = words.view(rounds, self.world, wpc)[:, rank, :].reshape(-1)
        return local[: (n_local + 63) // 64].contiguous()


def merge_topk(torch, scores, slots, k: int):
    """[nq, m] candidates -> best k under (score desc, slot asc) on host tensors (CPU process groups).  Padding
    entries carry score -inf and the largest slot, so they sort last."""
    order = torch.argsort(slots, dim=1, stable=True)
    s, i = torch.gather(scores, 1, order), torch.gather(slots, 1, order)
    order = torch.argsort(s, dim=1, descending=True, stable=True)
    return torch.gather(s, 1, order)[:, :k].contiguous(), torch.gather(i, 1, order)[:, :k].contiguous()


_PAD_SLOT = np.iinfo(np.int64).max


def pack_mask_words(torch, flags):
    """uint8 / bool flags (one per slot, length a multiple of 64) -> int64 words, bit i of word i // 64 = slot i."""
    shifts = torch.arange(64, device=flags.device, dtype=torch.int64)
    return (flags.view(-1, 64).to(torch.int64) << shifts).sum(dim=1)


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
        self._on_gpu = device.type == "cuda"
        self._buffers = {}

    def __len__(self) -> int:
        return self.n_total

    def _buf(self, name, shape, dtype):
        t = self._buffers.get(name)
        if t is None or t.shape != tuple(shape) or t.dtype != dtype:
            t = self._torch.empty(shape, dtype=dtype, device=self.device)
            self._buffers[name] = t
        return t

    # ---- ingest: each rank encodes the rows whose global slot it owns; no exchange ----
    def add(self, vectors: np.ndarray) -> None:
        n = vectors.shape[0]
        mine = [vectors[off:off + ln] for owner, off, ln in self.map.runs(self.n_total, n) if owner == self.rank]
        if mine:
            self.local.add(np.ascontiguousarray(np.concatenate(mine) if len(mine) > 1 else mine[0]))
        self.n_total += n
        assert len(self.local) == self.map.local_len(self.rank, self.n_total)

    def add_device(self, rows) -> float:
        """`rows`: the whole batch as a float32 tensor on this rank's device (every rank passes the same batch).
        Returns the device time (ms) of this rank's ingest kernels."""
        n, ms = rows.shape[0], 0.0
        for owner, off, ln in self.map.runs(self.n_total, n):
            if owner == self.rank:
                part = rows[off:off + ln]
                assert part.is_contiguous()
                self.local.add_device(part.data_ptr(), ln, self.dim)
                ms += self.local.last_main_kernel()[0]
        self.n_total += n
        assert len(self.local) == self.map.local_len(self.rank, self.n_total)
        return ms

    # ---- search: local scan, one all-gather of keys, one merge kernel ----
    def search_device(self, queries, k: int, *, mask_words=None):
        """queries: float32 tensor [nq, dim] on this rank's device; mask_words: None or the GLOBAL packed slot mask
        as an int64 tensor on the device (the same on every rank).  Returns (scores [nq, k], global slots [nq, k])
        as device tensors; rows hold min(k, len, n_allowed) results followed by (-inf, 0) padding."""
        torch, dist = self._torch, self._dist
        from . import merge_keys_device
        nq = queries.shape[0]
        k = min(int(k), self.n_total)
        scores = self._buf("scores", (nq, k), torch.float32)
        slots = self._buf("slots", (nq, k), torch.int64)
        if nq == 0 or k == 0:
            return scores, slots
        local_words = None
        if mask_words is not None:
            local_words = self.map.local_mask_words(torch, mask_words, self.rank, self.n_total)
        keys_all = self._buf("keys_all", (self.world, nq, k), torch.int64)
        keys_local = keys_all[self.rank] if self.world == 1 else self._buf("keys_local", (nq, k), torch.int64)
        if len(self.local) == 0:
            keys_local.fill_(-1)                                     # every key empty
        else:
            self.local.search_device_keys(queries.data_ptr(), nq, k, keys_local.data_ptr(), 0,
                                          local_words.data_ptr() if local_words is not None and local_words.numel() else 0)
        if self.world > 1:
            dist.all_gather_into_tensor(keys_all, keys_local, group=self._group)
        merge_keys_device(keys_all.data_ptr(), self.world, nq, k, scores.data_ptr(), slots.data_ptr(),
                          device=self.device.index or 0, stream=torch.cuda.current_stream(self.device).cuda_stream,
                          chunk_slots=self.map.chunk_slots)
        return scores, slots

    def search(self, queries: np.ndarray, k: int, *, mask=None):
        """Host arrays in, host arrays out; rows are min(k, len, n_allowed) wide as the reference's."""
        torch = self._torch
        nq = queries.shape[0]
        if mask is not None and mask.size != self.n_total:
            raise ValueError(f"mask length {mask.size} does not match index size {self.n_total}")
        if not self._on_gpu:
            return self._search_host_merge(queries, k, mask)
        words = None
        k_eff = min(k, self.n_total)
        if mask is not None:
            flags = torch.zeros(((self.n_total + 63) // 64) * 64, dtype=torch.uint8, device=self.device)
            flags[: self.n_total] = torch.from_numpy(np.ascontiguousarray(mask).view(np.uint8)).to(self.device)
            words = pack_mask_words(torch, flags)
            k_eff = min(k_eff, int(mask.sum()))
        q = torch.from_numpy(np.ascontiguousarray(queries, dtype=np.float32)).to(self.device)
        s, i = self.search_device(q, k, mask_words=words)
        return s[:, :k_eff].cpu().numpy(), i[:, :k_eff].cpu().numpy()

    def _search_host_merge(self, queries, k, mask):
        torch, dist = self._torch, self._dist
        nq = queries.shape[0]
        n_local = len(self.local)
        local_mask = None
        if mask is not None:
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


class IdTable:
    """Host-side id <-> global slot tables (tv_idtable_*): the replicated half of a sharded id-mapped index."""

    def __init__(self):
        from . import _native
        self._lib = _native.load()
        self._h = C.c_void_p()
        if self._lib.tv_idtable_create(C.byref(self._h)) != 0:
            raise RuntimeError("tv_idtable_create failed")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.tv_idtable_destroy(h)

    def _check(self, rc):
        if rc == 0:
            return
        msg = self._lib.tv_idtable_last_error(self._h, None).decode()
        if rc == 21:
            raise KeyError(msg)
        raise ValueError(msg)

    def __len__(self):
        return int(self._lib.tv_idtable_len(self._h))

    def add(self, ids: np.ndarray) -> None:
        self._check(self._lib.tv_idtable_add(self._h, ids.ctypes.data_as(C.c_void_p), ids.size))

    def truncate(self, n: int) -> None:
        self._check(self._lib.tv_idtable_truncate(self._h, n))

    def remove(self, id: int):
        removed, slot, moved = C.c_int(0), C.c_uint64(0), C.c_uint64(0)
        self._check(self._lib.tv_idtable_remove(self._h, C.c_uint64(id), C.byref(removed), C.byref(slot), C.byref(moved)))
        return bool(removed.value), int(slot.value), int(moved.value)

    def contains(self, id: int) -> bool:
        present = C.c_int(0)
        self._check(self._lib.tv_idtable_contains(self._h, C.c_uint64(id), C.byref(present)))
        return bool(present.value)

    def resolve(self, ids: np.ndarray) -> np.ndarray:
        out = np.empty(ids.size, np.uint64)
        self._check(self._lib.tv_idtable_resolve(self._h, ids.ctypes.data_as(C.c_void_p), ids.size, out.ctypes.data_as(C.c_void_p)))
        return out

    def ids_of(self, slots: np.ndarray) -> np.ndarray:
        slots = np.ascontiguousarray(slots, np.int64)
        out = np.empty(slots.shape, np.uint64)
        self._check(self._lib.tv_idtable_ids_of(self._h, slots.ctypes.data_as(C.c_void_p), slots.size, out.ctypes.data_as(C.c_void_p)))
        return out

    def ids(self) -> np.ndarray:
        out = np.empty(len(self), np.uint64)
        self._check(self._lib.tv_idtable_ids(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out


class ShardedIdMapIndex(ShardedIndex):
    """IdMapIndex over the ranks of a process group: add_with_ids / remove / search(allowlist=) / contains with
    caller-chosen uint64 ids (turbovec/src/id_map.rs:373-469, 520-567, 664-712).  Every rank holds the id tables."""

    def __init__(self, dim: int, bit_width: int = 4, **kw):
        super().__init__(dim, bit_width, **kw)
        self.table = IdTable()

    def _check_ids(self, ids, n):
        if not isinstance(ids, np.ndarray) or ids.dtype != np.uint64 or ids.ndim != 1:
            raise TypeError("ids must be a 1-D uint64 numpy array")
        if ids.size != n:
            raise ValueError(f"ids length {ids.size} does not match number of vectors {n}")
        return np.ascontiguousarray(ids)

    def add_with_ids(self, vectors: np.ndarray, ids: np.ndarray) -> None:
        ids = self._check_ids(ids, vectors.shape[0])
        before = len(self.table)
        self.table.add(ids)                      # validates ids before anything changes (id_map.rs:396-434)
        try:
            self.add(vectors)
        except Exception:
            self.table.truncate(before)
            raise

    def add_with_ids_device(self, rows, ids: np.ndarray) -> float:
        ids = self._check_ids(ids, rows.shape[0])
        before = len(self.table)
        self.table.add(ids)
        try:
            return self.add_device(rows)
        except Exception:
            self.table.truncate(before)
            raise

    def remove(self, id: int) -> bool:
        removed, slot, moved_from = self.table.remove(int(id))
        if removed:
            got = self.swap_remove(slot)
            assert got == moved_from
        return removed

    def contains(self, id: int) -> bool:
        return self.table.contains(int(id))

    __contains__ = contains

    def ids(self) -> np.ndarray:
        return self.table.ids()

    def allowlist_words(self, allowlist: np.ndarray):
        """The global packed slot mask of an allowlist, on this rank's device.  Unknown ids raise KeyError, an
        empty list ValueError (id_map.rs:672-677).  Returns (words, n_allowed)."""
        torch = self._torch
        if not isinstance(allowlist, np.ndarray) or allowlist.dtype != np.uint64 or allowlist.ndim != 1:
            raise TypeError("allowlist must be a 1-D uint64 numpy array")
        if allowlist.size == 0:
            raise ValueError("allowlist is empty")
        slots = self.table.resolve(np.ascontiguousarray(allowlist))
        flags = torch.zeros(((self.n_total + 63) // 64) * 64, dtype=torch.uint8, device=self.device)
        flags[torch.from_numpy(slots.astype(np.int64)).to(self.device)] = 1
        return pack_mask_words(torch, flags), int(flags.sum().item())

    def search(self, queries: np.ndarray, k: int, *, allowlist=None):
        """(scores, ids) with rows min(k, len, n_allowed) wide."""
        torch = self._torch
        if not self._on_gpu:
            mask = None
            if allowlist is not None:
                if allowlist.size == 0:
                    raise ValueError("allowlist is empty")
                mask = np.zeros(self.n_total, bool)
                mask[self.table.resolve(np.ascontiguousarray(allowlist)).astype(np.int64)] = True
            s, i = self._search_host_merge(queries, k, mask)
            return s, self.table.ids_of(i)
        words, k_eff = None, min(k, self.n_total)
        if allowlist is not None:
            words, n_allowed = self.allowlist_words(allowlist)
            k_eff = min(k_eff, n_allowed)
        q = torch.from_numpy(np.ascontiguousarray(queries, dtype=np.float32)).to(self.device)
        s, i = self.search_device(q, k, mask_words=words)
        s, i = s[:, :k_eff].cpu().numpy(), i[:, :k_eff].cpu().numpy()
        return s, self.table.ids_of(i)
