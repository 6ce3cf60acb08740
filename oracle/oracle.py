"""ctypes front end of the CPU oracle (``tv_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of the benchmark, never by the ``turbovec_b200`` package.
The arithmetic lives in C; this module only marshals numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from functools import lru_cache

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libtv_oracle.so")

MODE_AUTO, MODE_PD, MODE_LUT_MULADD, MODE_LUT_FLUSH, MODE_LUT_SCALAR = 0, 1, 2, 3, 4


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (no-op when up to date)."""
    src = os.path.join(_HERE, "tv_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "libtv_oracle.so"])
    return _SO


@lru_cache(maxsize=1)
def _lib():
    build()
    lib = C.CDLL(_SO)
    f32p, u8p, i8p = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.POINTER(C.c_int8)
    u32p, u64p, i64p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_int64)
    lib.tvo_rotation_tables.argtypes = [C.c_int, f32p, u32p]
    lib.tvo_rotate_rows.argtypes = [f32p, C.c_int, C.c_int, f32p]
    lib.tvo_codebook.argtypes = [C.c_int, C.c_int, f32p, f32p]
    lib.tvo_beta_cdf.argtypes = [C.c_double] * 3
    lib.tvo_beta_cdf.restype = C.c_double
    lib.tvo_norm.argtypes = [f32p, C.c_int]
    lib.tvo_norm.restype = C.c_float
    lib.tvo_first_invalid.argtypes = [f32p, C.c_int64]
    lib.tvo_first_invalid.restype = C.c_int64
    lib.tvo_rotate_batch.argtypes = [f32p, C.c_int64, C.c_int, f32p, f32p]
    lib.tvo_fit_calibration.argtypes = [f32p, C.c_int64, C.c_int, f32p, C.c_int, f32p, f32p]
    lib.tvo_encode.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, f32p, f32p, f32p, f32p, u8p, f32p, u8p, f32p]
    lib.tvo_reencode.argtypes = [u8p, f32p, C.c_int64, C.c_int, C.c_int, f32p, f32p, f32p, f32p, f32p, f32p, u8p, f32p]
    lib.tvo_boundary_distance.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, f32p, f32p, f32p, f32p]
    lib.tvo_extract_codes_flat.argtypes = [u8p, C.c_int64, C.c_int, C.c_int, u8p]
    lib.tvo_pack_blocked_seq.argtypes = [u8p, C.c_int64, C.c_int, u8p]
    lib.tvo_seq_to_packed.argtypes = [u8p, C.c_int64, C.c_int, C.c_int, u8p]
    lib.tvo_resolve_mode.argtypes = [C.c_int] * 3
    lib.tvo_resolve_mode.restype = C.c_int
    lib.tvo_search.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, u8p, f32p, C.c_int64, f32p, f32p, f32p,
                               C.c_int64, u64p, C.c_int, f32p, i64p]
    lib.tvo_search.restype = C.c_int64
    lib.tvo_query_tables.argtypes = [f32p, C.c_int64, C.c_int, C.c_int, f32p, f32p, f32p, C.c_int, f32p, u8p,
                                     i8p, i8p, f32p, f32p]
    lib.tvo_fnv1a.argtypes = [u8p, C.c_int64]
    lib.tvo_fnv1a.restype = C.c_uint64
    lib.tvo_lcg_vectors.argtypes = [C.c_int64, C.c_uint64, f32p]
    return lib


def _p(a, t):
    return None if a is None else a.ctypes.data_as(C.POINTER(t))


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def fnv1a(data) -> int:
    b = np.frombuffer(bytes(data) if not isinstance(data, np.ndarray) else np.ascontiguousarray(data).tobytes(),
                      dtype=np.uint8)
    return int(_lib().tvo_fnv1a(_p(b, C.c_uint8), b.size))


def lcg_vectors(n: int, dim: int, seed: int) -> np.ndarray:
    out = np.empty(n * dim, dtype=np.float32)
    _lib().tvo_lcg_vectors(n * dim, seed, _p(out, C.c_float))
    return out.reshape(n, dim)


def rotation_tables(dim: int):
    signs = np.empty((2, dim), dtype=np.float32)
    perms = np.empty((2, dim), dtype=np.uint32)
    _lib().tvo_rotation_tables(dim, _p(signs, C.c_float), _p(perms, C.c_uint32))
    return signs, perms


def rotate_rows(x: np.ndarray) -> np.ndarray:
    x = _f32(np.atleast_2d(x))
    out = np.empty_like(x)
    _lib().tvo_rotate_rows(_p(x, C.c_float), x.shape[0], x.shape[1], _p(out, C.c_float))
    return out


@lru_cache(maxsize=64)
def codebook(bits: int, dim: int):
    b = np.empty((1 << bits) - 1, dtype=np.float32)
    c = np.empty(1 << bits, dtype=np.float32)
    _lib().tvo_codebook(bits, dim, _p(b, C.c_float), _p(c, C.c_float))
    b.setflags(write=False)
    c.setflags(write=False)
    return b, c


def beta_cdf(a: float, b: float, x: float) -> float:
    return float(_lib().tvo_beta_cdf(a, b, x))


def norm(row: np.ndarray) -> np.float32:
    row = _f32(row)
    return np.float32(_lib().tvo_norm(_p(row, C.c_float), row.size))


def first_invalid(x: np.ndarray) -> int:
    x = _f32(x).ravel()
    return int(_lib().tvo_first_invalid(_p(x, C.c_float), x.size))


def rotate_batch(x: np.ndarray):
    x = _f32(x)
    n, dim = x.shape
    rot = np.empty_like(x)
    norms = np.empty(n, dtype=np.float32)
    _lib().tvo_rotate_batch(_p(x, C.c_float), n, dim, _p(rot, C.c_float), _p(norms, C.c_float))
    return rot, norms


def fit_calibration(x: np.ndarray, bits: int):
    """TQ+ fit from raw (unrotated) sample rows -> (shift, scale)."""
    rot, _ = rotate_batch(x)
    n, dim = rot.shape
    _, cent = codebook(bits, dim)
    cent = np.array(cent)
    shift = np.empty(dim, dtype=np.float32)
    scale = np.empty(dim, dtype=np.float32)
    _lib().tvo_fit_calibration(_p(rot, C.c_float), n, dim, _p(cent, C.c_float), cent.size,
                               _p(shift, C.c_float), _p(scale, C.c_float))
    return shift, scale


def encode(x: np.ndarray, bits: int, shift=None, scale=None, want_codes=False, want_rotated=False):
    """Returns dict(packed=bit-plane rows, scales, [codes], [rotated])."""
    x = _f32(x)
    n, dim = x.shape
    bnd, cent = (np.array(a) for a in codebook(bits, dim))
    shift, scale = _f32(shift), _f32(scale)
    packed = np.empty((n, bits * dim // 8), dtype=np.uint8)
    scales = np.empty(n, dtype=np.float32)
    codes = np.empty((n, dim), dtype=np.uint8) if want_codes else None
    rot = np.empty((n, dim), dtype=np.float32) if want_rotated else None
    _lib().tvo_encode(_p(x, C.c_float), n, dim, bits, _p(bnd, C.c_float), _p(cent, C.c_float),
                      _p(shift, C.c_float), _p(scale, C.c_float), _p(packed, C.c_uint8), _p(scales, C.c_float),
                      _p(codes, C.c_uint8), _p(rot, C.c_float))
    out = {"packed": packed, "scales": scales}
    if want_codes:
        out["codes"] = codes
    if want_rotated:
        out["rotated"] = rot
    return out


def reencode(codes: np.ndarray, scales: np.ndarray, bits: int, old_shift=None, old_scale=None, new_shift=None,
             new_scale=None):
    """Stored rows (one code per coordinate, [n, dim]) re-encoded under a new TQ+ pair; returns (codes, scales)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    n, dim = codes.shape
    bnd, cent = (np.array(a) for a in codebook(bits, dim))
    scales = _f32(scales)
    out_codes = np.empty_like(codes)
    out_scales = np.empty(n, dtype=np.float32)
    os_, osc, ns, nsc = _f32(old_shift), _f32(old_scale), _f32(new_shift), _f32(new_scale)
    _lib().tvo_reencode(_p(codes, C.c_uint8), _p(scales, C.c_float), n, dim, bits, _p(bnd, C.c_float), _p(cent, C.c_float),
                        _p(os_, C.c_float), _p(osc, C.c_float), _p(ns, C.c_float), _p(nsc, C.c_float),
                        _p(out_codes, C.c_uint8), _p(out_scales, C.c_float))
    return out_codes, out_scales


def boundary_distance(rotated: np.ndarray, bits: int, shift=None, scale=None) -> np.ndarray:
    rotated = _f32(rotated)
    n, dim = rotated.shape
    bnd = np.array(codebook(bits, dim)[0])
    shift, scale = _f32(shift), _f32(scale)
    out = np.empty((n, dim), dtype=np.float32)
    _lib().tvo_boundary_distance(_p(rotated, C.c_float), n, dim, bits, _p(bnd, C.c_float),
                                 _p(shift, C.c_float), _p(scale, C.c_float), _p(out, C.c_float))
    return out


def ngroups(dim: int, bits: int) -> int:
    return dim // (8 // bits)


def packed_to_blocked(packed: np.ndarray, bits: int, dim: int) -> np.ndarray:
    """Bit-plane rows -> sequential-blocked bytes (pack.rs repack_seq)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    n = packed.shape[0]
    ng = ngroups(dim, bits)
    flat = np.empty((n, ng), dtype=np.uint8)
    _lib().tvo_extract_codes_flat(_p(packed, C.c_uint8), n, bits, dim, _p(flat, C.c_uint8))
    nb = (n + 31) // 32
    blocked = np.empty(nb * ng * 32, dtype=np.uint8)
    _lib().tvo_pack_blocked_seq(_p(flat, C.c_uint8), n, ng, _p(blocked, C.c_uint8))
    return blocked


def blocked_to_packed(blocked: np.ndarray, n: int, bits: int, dim: int) -> np.ndarray:
    blocked = np.ascontiguousarray(blocked, dtype=np.uint8)
    packed = np.empty((n, bits * dim // 8), dtype=np.uint8)
    _lib().tvo_seq_to_packed(_p(blocked, C.c_uint8), n, bits, dim, _p(packed, C.c_uint8))
    return packed


def resolve_mode(mode: int, bits: int, dim: int) -> int:
    return int(_lib().tvo_resolve_mode(mode, bits, ngroups(dim, bits)))


def pack_mask(mask_bool: np.ndarray) -> np.ndarray:
    """bool[n] -> little-endian u64 words, bit i of word i//64 = slot i (lib.rs:1435-1456)."""
    m = np.asarray(mask_bool, dtype=bool)
    n = m.size
    padded = np.zeros(((n + 63) // 64) * 64, dtype=np.uint8)
    padded[:n] = m
    return np.packbits(padded, bitorder="little").view(np.uint64).copy()


def search(queries, blocked, scales, n, dim, bits, k, mask_words=None, shift=None, scale=None, mode=MODE_AUTO):
    """Returns (scores[nq,k_eff], slots[nq,k_eff])."""
    q = _f32(np.atleast_2d(queries))
    nq = q.shape[0]
    blocked = np.ascontiguousarray(blocked, dtype=np.uint8)
    scales = _f32(scales)
    cent = np.array(codebook(bits, dim)[1])
    shift, scale = _f32(shift), _f32(scale)
    kk = max(min(k, n), 0)
    s_out = np.empty((nq, max(kk, 1)), dtype=np.float32)
    i_out = np.empty((nq, max(kk, 1)), dtype=np.int64)
    mw = None if mask_words is None else np.ascontiguousarray(mask_words, dtype=np.uint64)
    k_eff = int(_lib().tvo_search(_p(q, C.c_float), nq, dim, bits, _p(blocked, C.c_uint8), _p(scales, C.c_float),
                                  n, _p(cent, C.c_float), _p(shift, C.c_float), _p(scale, C.c_float), kk,
                                  _p(mw, C.c_uint64), mode, _p(s_out, C.c_float), _p(i_out, C.c_int64)))
    # the C routine writes rows with stride k_eff
    s = s_out.ravel()[: nq * k_eff].reshape(nq, k_eff).copy()
    i = i_out.ravel()[: nq * k_eff].reshape(nq, k_eff).copy()
    return s, i


def query_tables(queries, dim, bits, shift=None, scale=None, mode=MODE_AUTO):
    q = _f32(np.atleast_2d(queries))
    nq = q.shape[0]
    ng = ngroups(dim, bits)
    cent = np.array(codebook(bits, dim)[1])
    shift, scale = _f32(shift), _f32(scale)
    q_rot = np.empty((nq, dim), dtype=np.float32)
    luts = np.zeros((nq, ng * 32), dtype=np.uint8)
    weights = np.zeros((nq, dim), dtype=np.int8)
    levels = np.zeros(16, dtype=np.int8)
    sc = np.empty(nq, dtype=np.float32)
    bi = np.empty(nq, dtype=np.float32)
    _lib().tvo_query_tables(_p(q, C.c_float), nq, dim, bits, _p(cent, C.c_float), _p(shift, C.c_float),
                            _p(scale, C.c_float), mode, _p(q_rot, C.c_float), _p(luts, C.c_uint8),
                            _p(weights, C.c_int8), _p(levels, C.c_int8), _p(sc, C.c_float), _p(bi, C.c_float))
    return {"q_rot": q_rot, "luts": luts, "weights": weights, "levels": levels, "scale": sc, "bias": bi,
            "mode": resolve_mode(mode, bits, dim)}


# ---------------------------------------------------------------------------------------------------
# AVX-512 VNNI restatement of the reference's permute-dot scan (cpu_simd_baseline.cpp): CPU arm only.
# ---------------------------------------------------------------------------------------------------
_SIMD_SO = os.path.join(_HERE, "libtv_cpu_simd.so")


@lru_cache(maxsize=1)
def _simd_lib():
    src = os.path.join(_HERE, "cpu_simd_baseline.cpp")
    if not os.path.exists(_SIMD_SO) or os.path.getmtime(_SIMD_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "libtv_cpu_simd.so"])
    lib = C.CDLL(_SIMD_SO)
    u8p, f32p, i8p = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_int8)
    lib.tvs_available.restype = C.c_int
    lib.tvs_to_vector_major.argtypes = [u8p, C.c_int64, C.c_int, u8p]
    lib.tvs_search_pd.argtypes = [u8p, f32p, C.c_int64, C.c_int, i8p, i8p, f32p, f32p, C.c_int64, C.c_int64,
                                  C.POINTER(C.c_uint64), C.c_int, f32p, C.POINTER(C.c_int64)]
    lib.tvs_search_pd.restype = C.c_int64
    return lib


def simd_available() -> bool:
    try:
        return bool(_simd_lib().tvs_available())
    except Exception:
        return False


def to_vector_major(blocked: np.ndarray, n: int, dim: int) -> np.ndarray:
    blocked = np.ascontiguousarray(blocked, dtype=np.uint8)
    out = np.empty_like(blocked)
    _simd_lib().tvs_to_vector_major(_p(blocked, C.c_uint8), (n + 31) // 32, dim // 2, _p(out, C.c_uint8))
    return out


def search_simd(queries, vm_codes, scales, n, dim, k, mask_words=None, threads=None):
    """4-bit permute-dot search on the vector-major layout with AVX-512 VNNI, all host threads by default."""
    tabs = query_tables(queries, dim, 4, mode=MODE_PD)
    nq = tabs["weights"].shape[0]
    scales = _f32(scales)
    kk = max(min(k, n), 1)
    s_out = np.empty((nq, kk), np.float32)
    i_out = np.empty((nq, kk), np.int64)
    mw = None if mask_words is None else np.ascontiguousarray(mask_words, dtype=np.uint64)
    threads = threads or (os.cpu_count() or 1)
    ke = int(_simd_lib().tvs_search_pd(_p(vm_codes, C.c_uint8), _p(scales, C.c_float), n, dim, _p(tabs["levels"], C.c_int8),
                                       _p(tabs["weights"], C.c_int8), _p(tabs["scale"], C.c_float), _p(tabs["bias"], C.c_float),
                                       nq, min(k, n), _p(mw, C.c_uint64), threads, _p(s_out, C.c_float), _p(i_out, C.c_int64)))
    return (s_out.ravel()[: nq * ke].reshape(nq, ke).copy(), i_out.ravel()[: nq * ke].reshape(nq, ke).copy())
