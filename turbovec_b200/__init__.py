"""turbovec_b200 — B200-native encode-and-scan path of turbovec behind the reference's index API.

The two classes mirror the reference's Python classes (turbovec-python/src/lib.rs:416-947 and
:952-1540): same method names, argument meaning, result shapes and exception types.  Everything
below them runs in libturbovec_b200.so on the GPU; nothing is computed in Python.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native
from ._native import (OPT_FAIL_NEXT, OPT_FORCE_CAREFUL, OPT_INGEST_PIPELINE, OPT_MMA_MIN_BATCH, OPT_PD_SPLIT, OPT_SCORE_MODE, OPT_SMALL_SCAN,
                      OPT_DENSE_PAIR, OPT_EXPANDED_BYTES, OPT_TC_EXPANDED, OPT_TC_TILES, OPT_TC_WIDE, SCORE_AUTO, SCORE_LUT_FLUSH, SCORE_LUT_MULADD, SCORE_PERMUTE_DOT)

__all__ = ["TurboQuantIndex", "IdMapIndex", "MultiGpuIndex", "BATCH_CHUNK_SIZE"]

# turbovec-python/python/turbovec/__init__.py:17 — batches above this are fed in slices
BATCH_CHUNK_SIZE = 4096


def _f32_2d(name: str, a) -> np.ndarray:
    # turbovec-python/src/lib.rs:56-63: float32, 2-D, C-contiguous, no silent conversion
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or a.ndim != 2:
        kind = f"{type(a).__name__}" if not isinstance(a, np.ndarray) else f"ndarray of dtype {a.dtype}, {a.ndim}-D"
        raise TypeError(f"{name} must be a 2-D float32 numpy array, got {kind}")
    if not a.flags.c_contiguous:
        raise ValueError(f"{name} must be C-contiguous")
    return a


def _typed_1d(name: str, a, dtype, label: str) -> np.ndarray:
    if not isinstance(a, np.ndarray) or a.dtype != dtype or a.ndim != 1:
        kind = f"{type(a).__name__}" if not isinstance(a, np.ndarray) else f"ndarray of dtype {a.dtype}, {a.ndim}-D"
        raise TypeError(f"{name} must be a 1-D {label} numpy array, got {kind}")
    if not a.flags.c_contiguous:
        raise ValueError(f"{name} must be C-contiguous")
    return a


def _size(name: str, v) -> int:
    # turbovec-python/src/lib.rs:153-179
    if isinstance(v, bool) or not isinstance(v, (int, np.integer)):
        raise TypeError(f"{name} must be an int, got {type(v).__name__}")
    if v < 0:
        raise ValueError(f"{name} must be non-negative, got {v}")
    return int(v)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class _Base:
    _KIND = 0

    def __init__(self, dim=None, bit_width=None, *, device: int = 0):
        self._lib = _native.load()
        self._h = C.c_void_p()
        d = 0 if dim is None else _size("dim", dim)
        if dim is not None and d == 0:
            raise ValueError("dim must be a positive multiple of 8, got 0")
        bits = 4 if bit_width is None else _size("bit_width", bit_width)
        rc = self._lib.tv_index_create(d, bits, self._KIND, int(device), C.byref(self._h))
        if rc != 0:
            msg = self._lib.tv_last_error(None).decode()
            raise (RuntimeError if rc >= 90 else ValueError)(msg)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.tv_index_destroy(h)

    # ---- helpers ----
    def _check(self, rc: int):
        if rc == 0:
            return
        msg = self._lib.tv_last_error(self._h).decode()
        if rc in _native.ERR_ID_KEYERROR:
            raise KeyError(msg)
        if rc in _native.ERR_INDEXERROR:
            raise IndexError(msg)
        if rc >= 90:
            raise RuntimeError(msg)
        raise ValueError(msg)

    def __len__(self) -> int:
        return int(self._lib.tv_len(self._h))

    @property
    def dim(self):
        d = int(self._lib.tv_dim(self._h))
        return d if d else None

    @property
    def bit_width(self) -> int:
        return int(self._lib.tv_bit_width(self._h))

    @property
    def calibration_state(self) -> str:
        flag = C.c_int(0)
        self._lib.tv_calibration(self._h, None, None, 0, C.byref(flag))
        return "calibrated" if flag.value else "uncalibrated"

    def prepare(self) -> None:
        self._check(self._lib.tv_prepare(self._h))

    def set_option(self, option: int, value: int) -> None:
        self._check(self._lib.tv_set_option(self._h, option, value))

    def get_option(self, option: int) -> int:
        return int(self._lib.tv_get_option(self._h, option))

    @property
    def launch_count(self) -> int:
        return int(self._lib.tv_launch_count(self._h))

    @property
    def last_kernel_ms(self) -> float:
        return float(self._lib.tv_last_kernel_ms(self._h))

    def last_main_kernel(self):
        """(summed ms, launches) of the dominant kernel (block scan / ingest) in the last call."""
        n = C.c_int(0)
        ms = float(self._lib.tv_last_main_kernel_ms(self._h, C.byref(n)))
        return ms, int(n.value)

    def set_calibration(self, shift: np.ndarray, scale: np.ndarray) -> None:
        shift = _typed_1d("shift", shift, np.float32, "float32")
        scale = _typed_1d("scale", scale, np.float32, "float32")
        if shift.shape != scale.shape:
            raise ValueError("shift and scale must have the same length")
        self._check(self._lib.tv_set_calibration(self._h, shift.size, _ptr(shift), _ptr(scale)))

    def calibrate(self, sample: np.ndarray) -> None:
        sample = _f32_2d("sample", sample)
        self._check(self._lib.tv_calibrate(self._h, _ptr(sample), sample.shape[0], sample.shape[1]))

    def calibration(self):
        """(shift, scale) of the TQ+ pair, or None while uncalibrated (tqplus_shift / tqplus_scale)."""
        d = self.dim or 0
        shift, scale = np.empty(d, np.float32), np.empty(d, np.float32)
        flag = C.c_int(0)
        self._check(self._lib.tv_calibration(self._h, _ptr(shift), _ptr(scale), d, C.byref(flag)))
        return (shift, scale) if flag.value else None

    def codebook(self):
        bits = self.bit_width
        b = np.empty((1 << bits) - 1, np.float32)
        c = np.empty(1 << bits, np.float32)
        self._check(self._lib.tv_codebook(self._h, _ptr(b), _ptr(c)))
        return b, c

    def rotate(self, rows: np.ndarray) -> np.ndarray:
        rows = _f32_2d("rows", rows)
        out = np.empty_like(rows)
        self._check(self._lib.tv_rotate(self._h, _ptr(rows), rows.shape[0], rows.shape[1], _ptr(out)))
        return out

    def codes_blocked_seq(self) -> np.ndarray:
        out = np.empty(int(self._lib.tv_blocked_bytes(self._h)), np.uint8)
        self._check(self._lib.tv_export_blocked(self._h, _ptr(out), out.size, None, 0))
        return out

    def scales(self) -> np.ndarray:
        out = np.empty(len(self), np.float32)
        self._check(self._lib.tv_export_blocked(self._h, None, 0, _ptr(out), out.size))
        return out

    def packed_codes(self) -> np.ndarray:
        d = self.dim or 0
        out = np.empty((len(self), self.bit_width * d // 8), np.uint8)
        self._check(self._lib.tv_export_packed(self._h, _ptr(out), out.size))
        return out

    def row_bytes(self) -> int:
        d = self.dim or 0
        return d // (8 // self.bit_width)

    def get_row(self, slot: int):
        """(byte-groups uint8[ngroups], scale) of one stored row."""
        out = np.empty(self.row_bytes(), np.uint8)
        scale = C.c_float(0)
        self._check(self._lib.tv_get_row(self._h, _size("slot", slot), _ptr(out), out.size, C.byref(scale)))
        return out, float(scale.value)

    def set_row(self, slot: int, groups: np.ndarray, scale: float) -> None:
        groups = np.ascontiguousarray(groups, np.uint8)
        self._check(self._lib.tv_set_row(self._h, _size("slot", slot), _ptr(groups), groups.size, float(scale)))

    # ---- persistence (the reference's v7 container) ----
    def to_bytes(self) -> bytes:
        buf = np.empty(int(self._lib.tv_image_bytes(self._h)), np.uint8)
        self._check(self._lib.tv_to_bytes(self._h, _ptr(buf), buf.size))
        return buf.tobytes()

    def write(self, path: str, *, durable: bool = True) -> None:
        rc = self._lib.tv_write(self._h, str(path).encode())
        if rc == 95:                                              # file errors raise OSError, as the reference's binding does
            raise OSError(f"{self._lib.tv_last_error(self._h).decode()}")
        self._check(rc)

    def sync(self, path: str) -> None:
        """Persist the changes since the last sync to `path` incrementally (`sync`, turbovec-python/src/lib.rs:744,
        1378): the first sync of a path writes the whole index, later ones only completed blocks, redo records of
        removals and a commit header.  File errors raise OSError, as the reference's binding does."""
        rc = self._lib.tv_sync(self._h, str(path).encode())
        if rc in (30, 95, 96):
            raise OSError(f"{self._lib.tv_last_error(self._h).decode()}: {path}")
        self._check(rc)

    def _sync_state(self):
        """(bound, generation, pending redo slots, dirtied slots) of the sync binding; for tests."""
        b, g, p, f = C.c_int(), C.c_uint64(), C.c_size_t(), C.c_size_t()
        self._check(self._lib.tv_sync_state(self._h, C.byref(b), C.byref(g), C.byref(p), C.byref(f)))
        return bool(b.value), int(g.value), int(p.value), int(f.value)

    @classmethod
    def _adopt(cls, handle):
        self = cls.__new__(cls)
        self._lib = _native.load()
        self._h = handle
        return self

    @classmethod
    def from_bytes(cls, data, *, device: int = 0):
        if not isinstance(data, (bytes, bytearray, memoryview)):
            raise TypeError(f"data must be bytes-like, got {type(data).__name__}")
        lib = _native.load()
        buf = np.frombuffer(bytes(data), np.uint8)
        h = C.c_void_p()
        rc = lib.tv_from_bytes(_ptr(buf), buf.size, cls._KIND, int(device), C.byref(h))
        if rc != 0:
            raise (RuntimeError if rc >= 90 else ValueError)(lib.tv_last_error(None).decode())
        return cls._adopt(h)

    @classmethod
    def load(cls, path: str, *, device: int = 0):
        lib = _native.load()
        h = C.c_void_p()
        rc = lib.tv_load(str(path).encode(), cls._KIND, int(device), C.byref(h))
        if rc == 95:
            raise OSError(lib.tv_last_error(None).decode())
        if rc != 0:
            raise (RuntimeError if rc >= 91 else ValueError)(lib.tv_last_error(None).decode())
        return cls._adopt(h)

    def __reduce__(self):
        return (type(self).from_bytes, (self.to_bytes(),))

    def search_device(self, q_ptr: int, nq: int, k: int, scores_ptr: int, slots_ptr: int, mask_words_ptr: int = 0) -> int:
        """Device-resident search; returns k_eff.  Output rows have stride k_eff."""
        k_eff = C.c_size_t(0)
        self._check(self._lib.tv_search_device(self._h, C.c_void_p(q_ptr), nq, k,
                                                C.c_void_p(mask_words_ptr) if mask_words_ptr else None,
                                                C.c_void_p(scores_ptr), C.c_void_p(slots_ptr), C.byref(k_eff)))
        return int(k_eff.value)

    def search_device_keys(self, q_ptr: int, nq: int, k: int, keys_ptr: int, slot_offset: int = 0,
                           mask_words_ptr: int = 0) -> int:
        """Device-resident search of one shard of a slot-sharded index: writes rows of k 64-bit result keys
        (ascending key = score descending, then global slot ascending; padded with EMPTY_KEY) with
        `slot_offset` added to every slot.  All-gather the rows of every rank and pass them to
        merge_keys_device.  Returns this shard's k_eff."""
        k_eff = C.c_size_t(0)
        self._check(self._lib.tv_search_device_keys(self._h, C.c_void_p(q_ptr), nq, k,
                                                     C.c_void_p(mask_words_ptr) if mask_words_ptr else None,
                                                     C.c_uint64(slot_offset), C.c_void_p(keys_ptr), C.byref(k_eff)))
        return int(k_eff.value)

    def search_device_noalloc(self, q_ptr: int, nq: int, k: int, scores_ptr: int, slots_ptr: int) -> int:
        """Like search_device (unfiltered) but guaranteed not to allocate: scratch is a fixed array inside
        the library.  For callers that must keep away from the CUDA allocator while serving.  Limits:
        nq <= 8, k <= 128, dim <= 4096.  Returns k_eff."""
        k_eff = C.c_size_t(0)
        self._check(self._lib.tv_search_device_noalloc(self._h, C.c_void_p(q_ptr), nq, k, C.c_void_p(scores_ptr),
                                                        C.c_void_p(slots_ptr), C.byref(k_eff)))
        return int(k_eff.value)

    # ---- one filter, many searches (no counterpart in the reference, which rebuilds the mask on every call) ----
    def prepare_mask_device(self, mask_words_ptr: int) -> None:
        """Keeps the packed slot mask at `mask_words_ptr` (device memory, ceil(len/64) uint64 words, bit i of word
        i // 64 = slot i) prepared on the device: its live code blocks are compacted once, and search_prepared /
        search_device_prepared reuse them until the index changes."""
        self._check(self._lib.tv_mask_prepare_device(self._h, C.c_void_p(mask_words_ptr)))

    def prepare_mask_words(self, words: np.ndarray) -> None:
        words = _typed_1d("words", words, np.uint64, "uint64")
        self._check(self._lib.tv_mask_prepare_words(self._h, _ptr(words), words.size))

    def search_prepared(self, queries: np.ndarray, k: int):
        """search() under the prepared mask.  Returns (scores, slots) on a positional index, (scores, ids) on an
        id-mapped one."""
        idmap = self._KIND == 1
        extra_fn = self._lib.tv_search_prepared
        queries = _f32_2d("queries", queries)
        k = _size("k", k)
        nq, ncols = queries.shape
        kk = min(k, len(self))
        scores = np.empty((nq, max(kk, 1)), np.float32)
        out = np.empty((nq, max(kk, 1)), np.uint64 if idmap else np.int64)
        k_eff = C.c_size_t(0)
        self._check(extra_fn(self._h, _ptr(queries), nq, ncols, k, _ptr(scores), None if idmap else _ptr(out),
                             _ptr(out) if idmap else None, C.byref(k_eff)))
        ke = int(k_eff.value)
        return (scores.ravel()[: nq * ke].reshape(nq, ke).copy(), out.ravel()[: nq * ke].reshape(nq, ke).copy())

    def search_device_prepared(self, q_ptr: int, nq: int, k: int, scores_ptr: int, slots_ptr: int) -> int:
        k_eff = C.c_size_t(0)
        self._check(self._lib.tv_search_device_prepared(self._h, C.c_void_p(q_ptr), nq, k, C.c_void_p(scores_ptr),
                                                         C.c_void_p(slots_ptr), C.byref(k_eff)))
        return int(k_eff.value)


    def _search_sliced(self, queries, k, fn, extra, out_dtype, chunk_size):
        """Per-query results do not depend on the other queries of a batch, so slices concatenate to exactly
        the result of one call."""
        slices = None
        if isinstance(queries, np.ndarray) and queries.ndim == 2:
            slices = _slice_rows(chunk_size, queries.shape[0])
        if slices is None:
            return self._search_raw(queries, k, fn, extra, out_dtype)
        parts = [self._search_raw(queries[a:b], k, fn, extra, out_dtype) for a, b in slices]
        return np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts])

    def _search_raw(self, queries, k, fn, extra, out_dtype):
        queries = _f32_2d("queries", queries)
        k = _size("k", k)
        nq, ncols = queries.shape
        idx_dim = self.dim
        if idx_dim is not None and ncols != idx_dim:
            raise ValueError(f"query dim {ncols} does not match index dim {idx_dim}")
        kk = min(k, len(self))
        scores = np.empty((nq, max(kk, 1)), np.float32)
        ids = np.empty((nq, max(kk, 1)), out_dtype)
        k_eff = C.c_size_t(0)
        self._check(fn(self._h, _ptr(queries), nq, ncols, k, *extra, _ptr(scores), _ptr(ids), C.byref(k_eff)))
        ke = int(k_eff.value)
        if nq == 0:
            return np.empty((0, ke), np.float32), np.empty((0, ke), out_dtype)
        return (scores.ravel()[: nq * ke].reshape(nq, ke).copy(), ids.ravel()[: nq * ke].reshape(nq, ke).copy())


def _slice_rows(chunk_size, n_rows):
    """Slices of a batch for the `chunk_size=` keyword of search / add / add_with_ids
    (turbovec-python/python/turbovec/_interruptible.py): a value > 0 makes the call go through the library in
    slices of that many rows, so that a pending KeyboardInterrupt is raised between slices; None, 0 or a
    negative value runs the call whole.  Unlike the reference, whose default slices at BATCH_CHUNK_SIZE rows,
    the default here is one call: the library already works through large batches in bounded chunks on the
    device, and a call of that size returns in milliseconds."""
    cs = 0 if chunk_size is None else int(chunk_size)
    if cs <= 0 or n_rows <= cs:
        return None
    return [(a, min(a + cs, n_rows)) for a in range(0, n_rows, cs)]


class TurboQuantIndex(_Base):
    """Positional index: results are slot numbers.  Mirrors turbovec-python/src/lib.rs:416-947."""
    _KIND = 0

    def add(self, vectors: np.ndarray, *, chunk_size=None) -> None:
        vectors = _f32_2d("vectors", vectors)
        slices = _slice_rows(chunk_size, vectors.shape[0])
        if slices is not None and bool(np.all(np.abs(vectors) < np.float32(1e16))):
            # a batch that would be rejected goes to the library whole, so that nothing is committed
            for a, b in slices:
                part = vectors[a:b]
                self._check(self._lib.tv_add(self._h, _ptr(part), part.shape[0], part.shape[1]))
            return
        self._check(self._lib.tv_add(self._h, _ptr(vectors), vectors.shape[0], vectors.shape[1]))

    def add_device(self, device_ptr: int, n: int, dim: int) -> None:
        """Adds n rows that already sit in device memory (row-major float32 at `device_ptr`)."""
        self._check(self._lib.tv_add_device(self._h, C.c_void_p(device_ptr), n, dim))

    def search(self, queries: np.ndarray, k: int, *, mask=None, chunk_size=None):
        extra = (None, 0)
        if mask is not None:
            mask = _typed_1d("mask", mask, np.bool_, "bool")
            if mask.size != len(self):
                raise ValueError(f"mask length {mask.size} does not match index size {len(self)}")
            extra = (_ptr(mask), mask.size)
        return self._search_sliced(queries, k, self._lib.tv_search, extra, np.int64, chunk_size)

    def search_mask_words(self, queries: np.ndarray, k: int, words: np.ndarray):
        words = _typed_1d("words", words, np.uint64, "uint64")
        return self._search_raw(queries, k, self._lib.tv_search_mask_words, (_ptr(words), words.size), np.int64)

    def swap_remove(self, idx: int) -> int:
        idx = _size("idx", idx)
        moved = C.c_size_t(0)
        self._check(self._lib.tv_swap_remove(self._h, idx, C.byref(moved)))
        return int(moved.value)

    @classmethod
    def from_parts(cls, dim: int, bit_width: int, packed: np.ndarray, scales: np.ndarray, *, device: int = 0):
        self = cls(dim, bit_width, device=device)
        packed = np.ascontiguousarray(packed, np.uint8)
        scales = np.ascontiguousarray(scales, np.float32)
        self._check(self._lib.tv_import_packed(self._h, dim, _ptr(packed), scales.size, _ptr(scales), None))
        return self

    def __repr__(self):
        return f"TurboQuantIndex(dim={self.dim}, bit_width={self.bit_width}, len={len(self)})"


class IdMapIndex(_Base):
    """Index addressed by caller-chosen uint64 ids.  Mirrors turbovec-python/src/lib.rs:952-1540."""
    _KIND = 1

    def add_with_ids(self, vectors: np.ndarray, ids: np.ndarray, *, chunk_size=None) -> None:
        vectors = _f32_2d("vectors", vectors)
        ids = _typed_1d("ids", ids, np.uint64, "uint64")
        if ids.size != vectors.shape[0]:
            raise ValueError(f"ids length {ids.size} does not match number of vectors {vectors.shape[0]}")
        slices = _slice_rows(chunk_size, vectors.shape[0])
        if slices is not None and bool(np.all(np.abs(vectors) < np.float32(1e16))) and np.unique(ids).size == ids.size \
                and not any(self.contains(int(i)) for i in ids):
            # pre-validated like the library's own up-front check: a batch that would be rejected goes to it
            # whole, so that nothing is committed
            for a, b in slices:
                part, part_ids = vectors[a:b], ids[a:b]
                self._check(self._lib.tv_add_with_ids(self._h, _ptr(part), part.shape[0], part.shape[1], _ptr(part_ids)))
            return
        self._check(self._lib.tv_add_with_ids(self._h, _ptr(vectors), vectors.shape[0], vectors.shape[1], _ptr(ids)))

    def add_with_ids_device(self, device_ptr: int, n: int, dim: int, ids: np.ndarray) -> None:
        """Adds n rows that already sit in device memory (row-major float32 at `device_ptr`) under host `ids`."""
        ids = _typed_1d("ids", ids, np.uint64, "uint64")
        if ids.size != n:
            raise ValueError(f"ids length {ids.size} does not match number of vectors {n}")
        self._check(self._lib.tv_add_with_ids_device(self._h, C.c_void_p(device_ptr), n, dim, _ptr(ids)))

    def remove(self, id) -> bool:
        if isinstance(id, bool) or not isinstance(id, (int, np.integer)):
            raise TypeError(f"id must be an int, got {type(id).__name__}")
        if id < 0 or id >= 1 << 64:
            return False
        removed = C.c_int(0)
        self._check(self._lib.tv_remove(self._h, int(id), C.byref(removed)))
        return bool(removed.value)

    def contains(self, id) -> bool:
        if isinstance(id, bool) or not isinstance(id, (int, np.integer)):
            raise TypeError(f"id must be an int, got {type(id).__name__}")
        if id < 0 or id >= 1 << 64:
            return False
        present = C.c_int(0)
        self._check(self._lib.tv_contains(self._h, int(id), C.byref(present)))
        return bool(present.value)

    __contains__ = contains

    def ids(self) -> np.ndarray:
        out = np.empty(len(self), np.uint64)
        self._check(self._lib.tv_ids(self._h, _ptr(out), out.size))
        return out

    def search(self, queries: np.ndarray, k: int, *, allowlist=None, chunk_size=None):
        extra = (None, 0)
        if allowlist is not None:
            allowlist = _typed_1d("allowlist", allowlist, np.uint64, "uint64")
            if allowlist.size == 0:
                raise ValueError("allowlist is empty")
            extra = (_ptr(allowlist), allowlist.size)
        return self._search_sliced(queries, k, self._lib.tv_search_allowlist, extra, np.uint64, chunk_size)

    def prepare_allowlist(self, allowlist: np.ndarray) -> None:
        """Resolves the ids once and keeps the resulting slot mask prepared on the device for search_prepared."""
        allowlist = _typed_1d("allowlist", allowlist, np.uint64, "uint64")
        if allowlist.size == 0:
            raise ValueError("allowlist is empty")
        self._check(self._lib.tv_mask_prepare_allowlist(self._h, _ptr(allowlist), allowlist.size))

    def __repr__(self):
        return f"IdMapIndex(dim={self.dim}, bit_width={self.bit_width}, len={len(self)})"


EMPTY_KEY = 0xFFFFFFFFFFFFFFFF


class MultiGpuIndex:
    """One index over several GPUs of this process (tv_multi_*): the rows are dealt to the devices round-robin in
    chunks of 32 * chunk_blocks global slots, a search scans every device at the same time and merges on the first
    one.  `id_mapped=False` mirrors TurboQuantIndex (add / search(mask=) / swap_remove over global slots),
    `id_mapped=True` mirrors IdMapIndex (add_with_ids / search(allowlist=) / remove / contains / ids).  Results are
    identical to a single index holding all the rows.  A device may be listed more than once."""

    def __init__(self, dim: int, bit_width: int = 4, *, devices=(0,), id_mapped: bool = False, chunk_blocks: int = 1024):
        self._lib = _native.load()
        self._h = C.c_void_p()
        self._idmap = bool(id_mapped)
        devs = (C.c_int * len(devices))(*[int(d) for d in devices])
        rc = self._lib.tv_multi_create(_size("dim", dim), int(bit_width), 1 if id_mapped else 0, devs, len(devices), int(chunk_blocks),
                                       C.byref(self._h))
        if rc != 0:
            raise (RuntimeError if rc >= 90 else ValueError)(self._lib.tv_multi_last_error(None).decode())

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.tv_multi_destroy(h)

    def _check(self, rc: int):
        if rc == 0:
            return
        msg = self._lib.tv_multi_last_error(self._h).decode()
        if rc == 21:
            raise KeyError(msg)
        if rc == 31:
            raise IndexError(msg)
        raise (RuntimeError if rc >= 90 else ValueError)(msg)

    def __len__(self) -> int:
        return int(self._lib.tv_multi_len(self._h))

    @property
    def n_shards(self) -> int:
        return int(self._lib.tv_multi_shards(self._h))

    def shard_len(self, i: int) -> int:
        return int(self._lib.tv_len(self._lib.tv_multi_shard(self._h, int(i))))

    def set_shard_option(self, option: int, value: int) -> None:
        for i in range(self.n_shards):
            rc = self._lib.tv_set_option(self._lib.tv_multi_shard(self._h, i), int(option), int(value))
            if rc != 0:
                raise ValueError(f"option {option} refused by shard {i}")

    def add(self, vectors: np.ndarray) -> None:
        vectors = _f32_2d("vectors", vectors)
        self._check(self._lib.tv_multi_add(self._h, _ptr(vectors), vectors.shape[0], vectors.shape[1]))

    def add_with_ids(self, vectors: np.ndarray, ids: np.ndarray) -> None:
        vectors = _f32_2d("vectors", vectors)
        ids = _typed_1d("ids", ids, np.uint64, "uint64")
        if ids.size != vectors.shape[0]:
            raise ValueError(f"ids length {ids.size} does not match number of vectors {vectors.shape[0]}")
        self._check(self._lib.tv_multi_add_with_ids(self._h, _ptr(vectors), vectors.shape[0], vectors.shape[1], _ptr(ids)))

    def swap_remove(self, idx: int) -> int:
        moved = C.c_size_t(0)
        self._check(self._lib.tv_multi_swap_remove(self._h, _size("idx", idx), C.byref(moved)))
        return int(moved.value)

    def remove(self, id: int) -> bool:
        removed = C.c_int(0)
        self._check(self._lib.tv_multi_remove(self._h, int(id), C.byref(removed)))
        return bool(removed.value)

    def contains(self, id: int) -> bool:
        present = C.c_int(0)
        self._check(self._lib.tv_multi_contains(self._h, int(id), C.byref(present)))
        return bool(present.value)

    __contains__ = contains

    def ids(self) -> np.ndarray:
        out = np.empty(len(self), np.uint64)
        self._check(self._lib.tv_multi_ids(self._h, _ptr(out), out.size))
        return out

    def search(self, queries: np.ndarray, k: int, *, mask=None, allowlist=None):
        """(scores, slots) or, id-mapped, (scores, ids); rows are min(k, len, n_allowed) wide."""
        queries = _f32_2d("queries", queries)
        k = _size("k", k)
        nq, dim = queries.shape
        width = max(min(k, len(self)), 1)
        scores = np.empty((nq, width), np.float32)
        k_eff = C.c_size_t(0)
        if self._idmap:
            if mask is not None:
                raise TypeError("an id-mapped index is filtered by allowlist=")
            out = np.empty((nq, width), np.uint64)
            ptr, count = None, 0
            if allowlist is not None:
                allowlist = _typed_1d("allowlist", allowlist, np.uint64, "uint64")
                if allowlist.size == 0:
                    raise ValueError("allowlist is empty")
                ptr, count = _ptr(allowlist), allowlist.size
            self._check(self._lib.tv_multi_search_allowlist(self._h, _ptr(queries), nq, dim, k, ptr, count, _ptr(scores), _ptr(out), C.byref(k_eff)))
        else:
            if allowlist is not None:
                raise TypeError("a positional index is filtered by mask=")
            out = np.empty((nq, width), np.int64)
            ptr, count = None, 0
            if mask is not None:
                mask = _typed_1d("mask", mask, np.bool_, "bool")
                ptr, count = _ptr(mask), mask.size
            self._check(self._lib.tv_multi_search(self._h, _ptr(queries), nq, dim, k, ptr, count, _ptr(scores), _ptr(out), C.byref(k_eff)))
        ke = int(k_eff.value)
        return (scores.ravel()[: nq * ke].reshape(nq, ke).copy(), out.ravel()[: nq * ke].reshape(nq, ke).copy())


def measure_int8_peak(device: int = 0, seconds: float = 0.0) -> float:
    """int8 tensor rate of `device` in ops/s for the library's MMA form (multiply-add = 2 ops), measured by a kernel
    that only issues MMAs: a burst of a few milliseconds (seconds = 0), or the rate sustained over `seconds`."""
    lib = _native.load()
    out = C.c_double(0.0)
    rc = lib.tv_measure_int8_peak_for(int(device), float(seconds), C.byref(out))
    if rc != 0:
        raise RuntimeError(lib.tv_last_error(None).decode())
    return float(out.value)


def merge_keys_device(keys_ptr: int, n_lists: int, nq: int, k: int, scores_ptr: int, slots_ptr: int, *, device: int = 0,
                      stream: int = 0, chunk_slots: int = 0) -> None:
    """keys[n_lists][nq][k] (device memory, e.g. all-gathered search_device_keys rows) -> per query the k best,
    decoded into scores[nq][k] (float32) and global slots[nq][k] (int64).  Enqueued on `stream` (a raw
    cudaStream_t value, 0 = default stream) without synchronising.  chunk_slots > 0: list r carries local slots of the
    shard that owns the slot chunks r, r + n_lists, ... of that size; they are made global before the merge."""
    lib = _native.load()
    rc = lib.tv_merge_keys_device_chunked(device, C.c_void_p(keys_ptr), n_lists, nq, k, chunk_slots, C.c_void_p(scores_ptr),
                                          C.c_void_p(slots_ptr), C.c_void_p(stream) if stream else None)
    if rc != 0:
        raise RuntimeError(lib.tv_last_error(None).decode() or f"tv_merge_keys_device failed with status {rc}")
