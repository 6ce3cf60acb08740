"""The allocation-free search entry point against the regular device search.

Some users of the library cannot let a search call reach the CUDA allocator: a serving loop with a latency
limit, a process whose device memory is already fully assigned, a framework that forbids allocator traffic
after warm-up.  tv_search_device_noalloc keeps its scratch in a fixed array inside the library; this test
calls it through the C ABI, twice in a row (the second call starts from the first call's leftovers in that
array), and requires exactly the results of tv_search_device.  It is collected last on purpose.
"""
import numpy as np
import pytest

from tests.util import anisotropic

pytestmark = pytest.mark.gpu


def _run(idx, torch, q, k, noalloc):
    nq = q.shape[0]
    scores = torch.full((nq, k), float("nan"), dtype=torch.float32, device="cuda")
    slots = torch.full((nq, k), -1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    fn = idx.search_device_noalloc if noalloc else idx.search_device
    ke = fn(q.data_ptr(), nq, k, scores.data_ptr(), slots.data_ptr())
    s = scores.view(-1)[: nq * ke].view(nq, ke).cpu().numpy()
    i = slots.view(-1)[: nq * ke].view(nq, ke).cpu().numpy()
    return ke, s, i


@pytest.mark.parametrize("dim,bits,n", [(1536, 4, 9000), (768, 2, 5000)])
def test_noalloc_search_equals_regular_search(dim, bits, n):
    import torch
    import turbovec_b200 as T
    x = anisotropic(n, dim, seed=31)
    idx = T.TurboQuantIndex(dim, bits)
    idx.add(x)
    for round_no, (nq, k) in enumerate([(8, 10), (3, 128)]):
        q = torch.from_numpy(anisotropic(nq, dim, seed=31, offset=50 + round_no)).cuda()
        ke_ref, s_ref, i_ref = _run(idx, torch, q, k, noalloc=False)
        # two calls in a row on the shared scratch array
        for _ in range(2):
            ke, s, i = _run(idx, torch, q, k, noalloc=True)
            assert ke == ke_ref == min(k, n)
            assert np.array_equal(i, i_ref)
            assert np.array_equal(s, s_ref)          # same kernels, same arithmetic: bit-identical


def test_noalloc_search_rejects_oversized_requests():
    import torch
    import turbovec_b200 as T
    dim = 256
    idx = T.TurboQuantIndex(dim, 4)
    idx.add(anisotropic(100, dim, seed=2))
    q = torch.zeros((9, dim), dtype=torch.float32, device="cuda")
    out_s = torch.empty((9, 200), dtype=torch.float32, device="cuda")
    out_i = torch.empty((9, 200), dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="at most 8 queries"):
        idx.search_device_noalloc(q.data_ptr(), 9, 10, out_s.data_ptr(), out_i.data_ptr())
    with pytest.raises(RuntimeError, match="k up to 128"):
        idx.search_device_noalloc(q.data_ptr(), 2, 129, out_s.data_ptr(), out_i.data_ptr())
