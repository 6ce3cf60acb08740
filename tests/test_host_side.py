"""CPU-only checks: the shared library loads and exports the whole C ABI, host-side argument validation
works without a device, and the product never reaches for the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from turbovec_b200 import build, _native
    build.build()
    return _native.load()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "turbovec_b200.h")).read()
    declared = set(re.findall(r"\b(tv_[a-z_0-9]+)\s*\(", header))
    declared -= {"tv_status", "tv_index"}
    assert len(declared) >= 30
    from turbovec_b200 import _native
    assert declared == set(_native.SIGNATURES), declared ^ set(_native.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name


def test_constructor_validation_needs_no_device(lib):
    h = ctypes.c_void_p()
    assert lib.tv_index_create(1536, 5, 0, 0, ctypes.byref(h)) == 1       # BitWidthOutOfRange
    assert lib.tv_index_create(1537, 4, 0, 0, ctypes.byref(h)) == 2       # DimNotPositiveMultipleOf8
    assert lib.tv_index_create(16392, 4, 0, 0, ctypes.byref(h)) == 3      # DimTooLarge
    assert b"16384" in lib.tv_last_error(None)


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    import turbovec_b200 as T
    with pytest.raises(RuntimeError, match="no CPU path"):
        T.TurboQuantIndex(64, 4)


def test_python_argument_errors():
    import turbovec_b200 as T
    with pytest.raises(TypeError):
        T._f32_2d("vectors", np.zeros((2, 8), np.float64))
    with pytest.raises(ValueError):
        T._f32_2d("vectors", np.zeros((8, 2), np.float32).T)
    with pytest.raises(TypeError):
        T._size("k", 1.5)
    with pytest.raises(ValueError):
        T._size("k", -1)


def test_product_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "turbovec_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def test_key_order_matches_reference_order():
    """(score desc, slot asc) <=> ascending u64 key; checked on the host twin of the device transform."""
    import struct

    def desc_bits(s):
        if s == 0.0:
            s = 0.0
        u = struct.unpack("<I", struct.pack("<f", s))[0]
        asc = (~u & 0xFFFFFFFF) if u & 0x80000000 else (u | 0x80000000)
        return ~asc & 0xFFFFFFFF

    vals = [-np.inf, -3.5, -1e-30, -0.0, 0.0, 1e-38, 2.0, 2.0000002, np.inf]
    keys = [(desc_bits(np.float32(v)) << 32) | 5 for v in vals]
    assert keys[3] == keys[4]                                   # the two zeros tie
    dedup = [k for j, k in enumerate(keys) if j != 3]
    assert dedup == sorted(dedup, reverse=True)                 # larger score -> smaller key
    assert ((desc_bits(np.float32(1.0)) << 32) | 3) < ((desc_bits(np.float32(1.0)) << 32) | 4)


def test_container_checksum(lib):
    """CRC-32C check value, and the three-way split the reference uses from 4096 bytes on (io_v7.rs:128-141)."""
    import zlib  # noqa: F401  (zlib has CRC-32 only; the Castagnoli reference below is bitwise)

    def crc32c(data: bytes) -> int:
        crc = 0xFFFFFFFF
        for b in data:
            crc ^= b
            for _ in range(8):
                crc = (crc >> 1) ^ 0x82F63B78 if crc & 1 else crc >> 1
        return crc ^ 0xFFFFFFFF

    msg = np.frombuffer(b"123456789", np.uint8)
    assert lib.tv_crc32c(msg.ctypes.data_as(ctypes.c_void_p), msg.size) == 0xE3069283
    big = np.random.default_rng(0).integers(0, 256, 5000, dtype=np.uint8)
    third = 5000 // 3
    parts = [crc32c(big[:third].tobytes()), crc32c(big[third:2 * third].tobytes()), crc32c(big[2 * third:].tobytes())]
    want = crc32c(b"".join(int(p).to_bytes(4, "little") for p in parts))
    assert lib.tv_crc32c(big.ctypes.data_as(ctypes.c_void_p), big.size) == want
    small = big[:4095].copy()
    assert lib.tv_crc32c(small.ctypes.data_as(ctypes.c_void_p), small.size) == crc32c(small.tobytes())


@pytest.mark.parametrize("dim,bits", [(128, 4), (256, 2), (384, 3), (768, 4), (1024, 2), (1536, 4), (1536, 3), (2048, 4), (2048, 2)])
def test_quantisation_grid_counts_boundaries_exactly(lib, dim, bits):
    """The pipelined ingest kernel quantises through a grid table; its lookup must equal the plain count of
    boundaries strictly below the value for every float, in particular at and next to each boundary."""
    from oracle import oracle as O
    b, _ = O.codebook(bits, dim)
    rng = np.random.default_rng(dim * 10 + bits)
    near = np.concatenate([np.nextafter(b, np.float32(-np.inf)), b, np.nextafter(b, np.float32(np.inf))])
    for _ in range(3):
        near = np.concatenate([near, np.nextafter(near, np.float32(-np.inf)), np.nextafter(near, np.float32(np.inf))])
    spread = (rng.standard_normal(200_000) / np.sqrt(dim)).astype(np.float32)
    wide = rng.uniform(-1.5, 1.5, 20_000).astype(np.float32)
    edge = np.array([0.0, -0.0, 1.0, -1.0, 1e-30, -1e-30, 3e16, -3e16, 1e-45, -1e-45], dtype=np.float32)
    mids = ((b[:-1].astype(np.float64) + b[1:]) / 2).astype(np.float32)
    x = np.ascontiguousarray(np.concatenate([near, spread, wide, edge, mids]).astype(np.float32))
    want = (x[:, None] > b[None, :]).sum(axis=1).astype(np.uint8)
    got = np.empty(x.size, dtype=np.uint8)
    bb = np.ascontiguousarray(b)
    rc = lib.tv_quantise_grid_lookup(bb.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), bb.size,
                                     x.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), x.size,
                                     got.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
    assert rc == 0
    assert np.array_equal(got, want), np.flatnonzero(got != want)[:10]


def test_quantisation_grid_refuses_crowded_boundaries(lib):
    b = np.array([0.0, 1e-9, 1.0], dtype=np.float32)     # two boundaries inside one cell
    out = np.empty(1, dtype=np.uint8)
    x = np.zeros(1, dtype=np.float32)
    rc = lib.tv_quantise_grid_lookup(b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), 3,
                                     x.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), 1,
                                     out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
    assert rc == 93   # TV_ERR_UNSUPPORTED: the index then keeps to the block-at-a-time kernel


@pytest.mark.parametrize("dim", [128, 256, 384, 512, 768, 1024, 1536, 2048, 3072])
def test_exchange_layout_is_conflict_free(lib, dim):
    """Edge colouring of the store/gather instruction graph: with the layout no warp instruction of the
    pipelined ingest kernel's round-1 store or round-2 gather has two lanes on one shared-memory bank."""
    v = [ctypes.c_int(0) for _ in range(4)]
    assert lib.tv_exchange_layout_conflicts(dim, *[ctypes.byref(x) for x in v]) == 0
    store_plain, gather_plain, store_layout, gather_layout = [x.value for x in v]
    assert store_plain == 1 and gather_plain >= 2      # plain rows: contiguous stores, random gathers
    assert store_layout == 1 and gather_layout == 1


def test_sync_planner_matches_a_restatement():
    """`plan_incremental` (io_v7.rs:674-735) restated with Python sets against the library's planner."""
    import ctypes as C
    from turbovec_b200 import _native
    lib = _native.load()
    rng = np.random.default_rng(5)

    def plan(n_synced, n, pending, fresh):
        pa, fa = np.array(sorted(pending), np.uint64), np.array(sorted(fresh), np.uint64)
        mat, car = np.zeros(4096, np.uint64), np.zeros(4096, np.uint64)
        nm, nc, a0, a1 = C.c_size_t(mat.size), C.c_size_t(car.size), C.c_size_t(), C.c_size_t()
        rc = lib.tv_v7_plan_sync(n_synced, n, pa.ctypes.data, pa.size, fa.ctypes.data, fa.size, mat.ctypes.data, C.byref(nm),
                                 car.ctypes.data, C.byref(nc), C.byref(a0), C.byref(a1))
        if rc != 0:
            return rc
        return list(map(int, mat[: nm.value])), list(map(int, car[: nc.value])), a0.value, a1.value

    for case in range(300):
        n_synced = int(rng.integers(0, 2000))
        n = int(rng.integers(0, 2000))
        watermark = n_synced // 32 * 32
        pending = set(map(int, rng.integers(0, max(1, watermark), int(rng.integers(0, 40))))) if watermark else set()
        fresh = set(map(int, rng.integers(0, max(1, watermark), int(rng.integers(0, 40))))) if watermark else set()
        live = min(n_synced // 32, n // 32) * 32
        fresh_units = {s // 32 for s in fresh if s < live}
        want_mat = sorted({s // 32 for s in pending if s < live and s // 32 not in fresh_units})
        want_car = sorted({s for s in pending | fresh if s < live and s // 32 in fresh_units})
        assert plan(n_synced, n, pending, fresh) == (want_mat, want_car, n_synced // 32, n // 32), case
    # one header carries at most 1,024 redo ops
    many = set(range(0, 4000, 3))
    assert len(many) > 1024 and plan(4096, 4096, set(), many) == 93
    assert plan(4096, 4096, set(), set(list(many)[:1024]))[1] == sorted(list(many)[:1024])
