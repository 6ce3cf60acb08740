"""Host logic of the multi-device handle (csrc/multi.cpp) on a machine without a GPU.

multi.cpp is written against the public C ABI only, so it is compiled here with g++ against a stand-in backend
(tests/fake_backend: a brute-force single-"device" index and a CUDA runtime whose device memory is host memory) together
with the real id tables (csrc/idtable.cpp).  What is under test is everything multi.cpp adds: the round-robin chunk
ownership, the per-shard masks, the merge call, cross-shard removal, the id tables around the shards and the
all-or-nothing add.  A handle of several shards must behave exactly like a handle of one.
"""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_H = C.c_void_p
_szp = C.POINTER(C.c_size_t)


@pytest.fixture(scope="module")
def lib(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake") / "libtvmulti_fake.so"
    src = [os.path.join(ROOT, "turbovec_b200", "csrc", "multi.cpp"), os.path.join(ROOT, "turbovec_b200", "csrc", "idtable.cpp"),
           os.path.join(ROOT, "tests", "fake_backend", "fake_index.cpp")]
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-I", os.path.join(ROOT, "tests", "fake_backend"),
                           "-o", str(out), *src, "-lpthread"])
    lib = C.CDLL(str(out))
    sig = {
        "tv_multi_create": (C.c_int, [C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int, C.c_size_t, C.POINTER(_H)]),
        "tv_multi_destroy": (None, [_H]),
        "tv_multi_last_error": (C.c_char_p, [_H]),
        "tv_multi_len": (C.c_size_t, [_H]),
        "tv_multi_shard": (_H, [_H, C.c_int]),
        "tv_len": (C.c_size_t, [_H]),
        "tv_multi_add": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t]),
        "tv_multi_add_with_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
        "tv_multi_swap_remove": (C.c_int, [_H, C.c_size_t, _szp]),
        "tv_multi_remove": (C.c_int, [_H, C.c_uint64, C.POINTER(C.c_int)]),
        "tv_multi_contains": (C.c_int, [_H, C.c_uint64, C.POINTER(C.c_int)]),
        "tv_multi_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
        "tv_multi_search": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, _szp]),
        "tv_multi_search_allowlist": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, _szp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


class Handle:
    def __init__(self, lib, dim, shards, idmap=False, chunk_blocks=2):
        self.lib, self.dim, self.idmap, self.shards = lib, dim, idmap, shards
        self.h = _H()
        devs = (C.c_int * shards)(*([0] * shards))
        assert lib.tv_multi_create(dim, 4, 1 if idmap else 0, devs, shards, chunk_blocks, C.byref(self.h)) == 0

    def __del__(self):
        self.lib.tv_multi_destroy(self.h)

    def __len__(self):
        return int(self.lib.tv_multi_len(self.h))

    def err(self):
        return self.lib.tv_multi_last_error(self.h).decode()

    def shard_lens(self):
        return [int(self.lib.tv_len(self.lib.tv_multi_shard(self.h, i))) for i in range(self.shards)]

    def add(self, x, ids=None):
        x = np.ascontiguousarray(x, np.float32)
        if ids is None:
            return self.lib.tv_multi_add(self.h, x.ctypes.data, x.shape[0], x.shape[1])
        ids = np.ascontiguousarray(ids, np.uint64)
        return self.lib.tv_multi_add_with_ids(self.h, x.ctypes.data, x.shape[0], x.shape[1], ids.ctypes.data)

    def search(self, q, k, mask=None, allow=None):
        q = np.ascontiguousarray(q, np.float32)
        nq = q.shape[0]
        width = max(1, min(k, len(self)))
        s = np.empty((nq, width), np.float32)
        ke = C.c_size_t(0)
        if self.idmap:
            out = np.empty((nq, width), np.uint64)
            a = None if allow is None else np.ascontiguousarray(allow, np.uint64)
            rc = self.lib.tv_multi_search_allowlist(self.h, q.ctypes.data, nq, q.shape[1], k, None if a is None else a.ctypes.data,
                                                    0 if a is None else a.size, s.ctypes.data, out.ctypes.data, C.byref(ke))
        else:
            out = np.empty((nq, width), np.int64)
            m = None if mask is None else np.ascontiguousarray(mask, np.bool_)
            rc = self.lib.tv_multi_search(self.h, q.ctypes.data, nq, q.shape[1], k, None if m is None else m.ctypes.data,
                                          0 if m is None else m.size, s.ctypes.data, out.ctypes.data, C.byref(ke))
        w = int(ke.value)
        return rc, s.ravel()[: nq * w].reshape(nq, w).copy(), out.ravel()[: nq * w].reshape(nq, w).copy()

    def swap_remove(self, slot):
        moved = C.c_size_t(0)
        return self.lib.tv_multi_swap_remove(self.h, slot, C.byref(moved)), int(moved.value)

    def remove(self, id):
        removed = C.c_int(0)
        assert self.lib.tv_multi_remove(self.h, int(id), C.byref(removed)) == 0
        return bool(removed.value)

    def ids(self):
        out = np.empty(len(self), np.uint64)
        assert self.lib.tv_multi_ids(self.h, out.ctypes.data, out.size) == 0
        return out


def _rows(n, dim, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n, dim)) * np.exp(0.3 * rng.standard_normal(dim))).astype(np.float32)


def _same(a, b):
    return a[0] == b[0] == 0 and np.array_equal(a[2], b[2]) and np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))


@pytest.mark.parametrize("shards", [2, 3, 5])
def test_positional_handle_of_several_shards_equals_one_shard(lib, shards):
    dim, n = 32, 1500
    x, q = _rows(n, dim, 1), _rows(6, dim, 2)
    one, many = Handle(lib, dim, 1), Handle(lib, dim, shards)
    for a, b in ((0, 1), (1, 70), (70, 700), (700, n)):
        assert one.add(x[a:b]) == 0 and many.add(x[a:b]) == 0
    assert len(many) == n and sum(many.shard_lens()) == n
    assert max(many.shard_lens()) - min(many.shard_lens()) <= 64          # one chunk of 2 blocks at most
    assert _same(many.search(q, 10), one.search(q, 10)) and _same(many.search(q, 200), one.search(q, 200))
    rng = np.random.default_rng(3)
    mask = rng.random(n) < 0.07
    assert _same(many.search(q, 10, mask=mask), one.search(q, 10, mask=mask))
    few = np.zeros(n, bool)
    few[[3, 64, 1499]] = True
    rc, s, i = many.search(q, 10, mask=few)
    assert rc == 0 and i.shape == (6, 3) and set(i[0]) == {3, 64, 1499} and _same((rc, s, i), one.search(q, 10, mask=few))
    assert many.search(q, 10, mask=np.zeros(n, bool))[2].shape == (6, 0)
    assert many.search(q, 10, mask=np.ones(n - 1, bool))[0] == 24           # TV_ERR_MASK_LENGTH_MISMATCH
    assert many.search(_rows(2, dim + 8, 4), 10)[0] == 10                   # TV_ERR_DIM_MISMATCH
    for victim in (0, 63, 64, 900, -1, 17, 128):
        victim = len(many) - 1 if victim < 0 else victim
        assert many.swap_remove(victim) == one.swap_remove(victim)
        assert sum(many.shard_lens()) == len(many)
    assert many.swap_remove(len(many))[0] == 31                             # TV_ERR_SLOT_OUT_OF_RANGE
    assert _same(many.search(q, 25), one.search(q, 25))
    assert many.add(x[:333]) == 0 and one.add(x[:333]) == 0
    assert _same(many.search(q, 25), one.search(q, 25))


def test_idmapped_handle_of_several_shards_equals_one_shard(lib):
    dim, n = 32, 1200
    x, q = _rows(n, dim, 5), _rows(4, dim, 6)
    ids = (np.random.default_rng(7).permutation(n) + 10**12).astype(np.uint64)
    one, many = Handle(lib, dim, 1, idmap=True), Handle(lib, dim, 3, idmap=True)
    for a, b in ((0, 500), (500, 501), (501, n)):
        assert one.add(x[a:b], ids[a:b]) == 0 and many.add(x[a:b], ids[a:b]) == 0
    assert _same(many.search(q, 10), one.search(q, 10))
    allow = ids[::7]
    assert _same(many.search(q, 10, allow=allow), one.search(q, 10, allow=allow))
    assert _same(many.search(q, 500, allow=allow), one.search(q, 500, allow=allow))         # n_allowed < k
    assert many.search(q, 5, allow=np.array([3], np.uint64))[0] == 21                       # TV_ERR_UNKNOWN_ID
    assert many.search(q, 5, allow=np.array([], np.uint64))[0] == 20                        # TV_ERR_ALLOWLIST_EMPTY
    assert many.add(x[:2], ids[5:7]) == 15 and len(many) == n                               # TV_ERR_ID_ALREADY_PRESENT
    assert many.add(x[:2], np.array([1, 1], np.uint64)) == 16 and len(many) == n            # TV_ERR_DUPLICATE_ID_IN_BATCH
    rng = np.random.default_rng(8)
    for victim in rng.choice(ids, 80, replace=False):
        assert many.remove(victim) and one.remove(victim)
    assert not many.remove(12345)
    assert np.array_equal(many.ids(), one.ids())
    live = one.ids()
    assert _same(many.search(q, 10), one.search(q, 10)) and _same(many.search(q, 10, allow=live[::3]), one.search(q, 10, allow=live[::3]))


def test_failed_add_is_taken_back_from_every_shard(lib):
    dim = 32
    x, q = _rows(700, dim, 9), _rows(3, dim, 10)
    many = Handle(lib, dim, 3)
    assert many.add(x[:100]) == 0
    before, lens = many.search(q, 10), many.shard_lens()
    bad = x[100:600].copy()
    bad[450, 7] = np.inf
    assert many.add(bad) == 17 and "vector 450 coordinate 7" in many.err()   # TV_ERR_INVALID_INPUT_VALUE, index in the batch
    assert len(many) == 100 and many.shard_lens() == lens
    assert _same(many.search(q, 10), before)
    ids_handle = Handle(lib, dim, 3, idmap=True)
    ids = np.arange(600, dtype=np.uint64)
    assert ids_handle.add(x[:100], ids[:100]) == 0
    assert ids_handle.add(bad, ids[100:600]) == 17
    assert len(ids_handle) == 100 and np.array_equal(ids_handle.ids(), ids[:100])            # the id tables were rolled back too
    assert ids_handle.add(x[100:600], ids[100:600]) == 0 and len(ids_handle) == 600
