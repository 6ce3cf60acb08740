"""The AVX-512 VNNI CPU baseline returns exactly what the scalar oracle returns."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.util import anisotropic


@pytest.mark.skipif(not O.simd_available(), reason="host CPU has no AVX-512 VNNI")
@pytest.mark.parametrize("n,nq,threads", [(5003, 19, 4), (700, 3, 1), (20000, 9, 8)])
def test_simd_baseline_equals_scalar_oracle(n, nq, threads):
    dim, bits = 512, 4
    x = anisotropic(n, dim, seed=3)
    q = anisotropic(nq, dim, seed=3, offset=5)
    enc = O.encode(x, bits)
    blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    vm = O.to_vector_major(blocked, n, dim)
    for k in (1, 10):
        s, i = O.search_simd(q, vm, enc["scales"], n, dim, k, threads=threads)
        rs, ri = O.search(q, blocked, enc["scales"], n, dim, bits, k, mode=O.MODE_PD)
        assert np.array_equal(i, ri) and np.array_equal(s, rs)
    mask = np.random.default_rng(0).random(n) < 0.03
    s, i = O.search_simd(q, vm, enc["scales"], n, dim, 10, mask_words=O.pack_mask(mask), threads=threads)
    rs, ri = O.search(q, blocked, enc["scales"], n, dim, bits, 10, mask_words=O.pack_mask(mask), mode=O.MODE_PD)
    assert np.array_equal(i, ri) and np.array_equal(s, rs)
