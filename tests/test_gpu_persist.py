"""The v7 container: byte-identical to the reference's snapshot (frozen `file` hashes), and round trips."""
import pickle

import numpy as np
import pytest

from oracle import oracle as O
from tests.golden import reference_goldens as G
from tests.util import anisotropic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    import turbovec_b200
    return turbovec_b200


@pytest.mark.parametrize("row", G.ENCODE_FINGERPRINT, ids=lambda r: f"d{r[0]}b{r[1]}")
def test_file_fingerprint(T, row):
    """fnv1a(to_bytes()) of the reference's fixture (calibrate, then add 2000 LCG rows)."""
    dim, bits, *_rest, g_file = row
    x = O.lcg_vectors(2000, dim, G.cell_seed(dim, bits))
    idx = T.TurboQuantIndex(dim, bits)
    idx.calibrate(x)
    idx.add(x)
    assert O.fnv1a(idx.to_bytes()) == g_file


@pytest.mark.parametrize("n", [0, 1, 31, 32, 33, 1000])
def test_roundtrip_positional(T, tmp_path, n):
    dim, bits = 256, 4
    x = anisotropic(max(n, 1), dim, seed=61)[:n]
    a = T.TurboQuantIndex(dim, bits)
    if n:
        a.add(x)
    blob = a.to_bytes()
    b = T.TurboQuantIndex.from_bytes(blob)
    assert len(b) == n and b.dim == dim and b.bit_width == bits
    assert b.to_bytes() == blob
    path = tmp_path / "index.tv"
    a.write(str(path))
    assert path.read_bytes() == blob
    c = T.TurboQuantIndex.load(str(path))
    d = pickle.loads(pickle.dumps(a))
    if n:
        q = anisotropic(5, dim, seed=61, offset=9)
        ref = a.search(q, 10)
        for other in (b, c, d):
            s, i = other.search(q, 10)
            assert np.array_equal(i, ref[1]) and np.array_equal(s, ref[0])
        b.add(anisotropic(3, dim, seed=63))            # a loaded index keeps working
        assert len(b) == n + 3


def test_roundtrip_idmap_and_errors(T):
    dim, n = 128, 77
    x = anisotropic(n, dim, seed=62)
    ids = (np.arange(n) * 3 + 1000).astype(np.uint64)
    a = T.IdMapIndex(dim, 2)
    a.add_with_ids(x, ids)
    blob = a.to_bytes()
    b = T.IdMapIndex.from_bytes(blob)
    assert list(b.ids()) == list(ids) and int(ids[5]) in b
    q = anisotropic(3, dim, seed=62, offset=1)
    sa, ia = a.search(q, 5, allowlist=ids[::2].copy())
    sb, ib = b.search(q, 5, allowlist=ids[::2].copy())
    assert np.array_equal(ia, ib) and np.array_equal(sa, sb)
    with pytest.raises(ValueError, match="IdMapIndex"):
        T.TurboQuantIndex.from_bytes(blob)
    bad = bytearray(blob)
    bad[30] ^= 0x40                                    # inside the superblock
    with pytest.raises(ValueError, match="checksum"):
        T.IdMapIndex.from_bytes(bytes(bad))
    with pytest.raises(ValueError, match="not a v7"):
        T.IdMapIndex.from_bytes(b"nonsense-bytes")
    lazy = T.TurboQuantIndex(None, 3)
    again = T.TurboQuantIndex.from_bytes(lazy.to_bytes())
    assert again.dim is None and again.bit_width == 3 and len(again) == 0


def test_file_errors_are_os_errors(tmp_path):
    """A path that cannot be opened or written is an I/O error (OSError, status 95), not an argument error."""
    import turbovec_b200 as T
    with pytest.raises(OSError):
        T.TurboQuantIndex.load(str(tmp_path / "missing.tv"))
    idx = T.TurboQuantIndex(64, 4)
    idx.add(anisotropic(40, 64, seed=3))
    with pytest.raises(OSError):
        idx.write(str(tmp_path / "no_such_dir" / "x.tv"))
    idx.write(str(tmp_path / "ok.tv"))
    assert len(T.TurboQuantIndex.load(str(tmp_path / "ok.tv"))) == 40
