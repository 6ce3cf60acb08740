"""The allocation-free search entry point against the CPU oracle and the regular device search.

Some users of the library cannot let a search call reach the CUDA allocator: a serving loop with a latency
limit, a process whose device memory is already fully assigned, a framework that forbids allocator traffic
after warm-up.  tv_search_device_noalloc keeps its scratch in a fixed array inside the library; this test
calls it through the C ABI, twice in a row (the second call starts from the first call's leftovers in that
array), and requires exactly the oracle's results, which are also those of tv_search_device.  It covers 2-, 3-
and 4-bit indexes, a calibrated one, the largest supported dimension, an index large enough for several chunks
of the schedule, a rejected query and the limits, and checks that the device's free memory does not move across
a call.  It is collected last on purpose.
"""
import numpy as np
import pytest

from oracle import oracle as O
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


@pytest.mark.parametrize("dim,bits,n,calibrated", [(1536, 4, 9000, False), (768, 2, 5000, False), (1024, 3, 4000, False),
                                                    (512, 4, 6000, True), (4096, 4, 1500, False), (64, 4, 140_000, False)])
def test_noalloc_search_equals_oracle_and_regular_search(dim, bits, n, calibrated):
    import torch
    import turbovec_b200 as T
    x = anisotropic(n, dim, seed=31)
    idx = T.TurboQuantIndex(dim, bits)
    shift = scale = None
    if calibrated:
        idx.calibrate(anisotropic(2000, dim, seed=32))
        shift, scale = idx.calibration()
    idx.add(x)
    enc = O.encode(x, bits, shift, scale)
    blocked = O.packed_to_blocked(enc["packed"], bits, dim)
    for round_no, (nq, k) in enumerate([(8, 10), (3, 128), (1, 10)]):
        qh = anisotropic(nq, dim, seed=31, offset=50 + round_no)
        q = torch.from_numpy(qh).cuda()
        ref_s, ref_i = O.search(qh, blocked, enc["scales"], n, dim, bits, k, shift=shift, scale=scale)
        ke_ref, s_ref, i_ref = _run(idx, torch, q, k, noalloc=False)
        assert np.array_equal(i_ref, ref_i) and np.array_equal(s_ref, ref_s)
        _run(idx, torch, q, k, noalloc=True)         # warm-up: loads this batch size's kernels
        # two calls in a row on the shared scratch array; the device's free memory must not move
        for _ in range(2):
            free_before = torch.cuda.mem_get_info()[0]
            ke, s, i = _run(idx, torch, q, k, noalloc=True)
            assert ke == ke_ref == min(k, n)
            assert np.array_equal(i, ref_i)
            assert np.array_equal(s, ref_s)          # integer sums are exact, the float steps replay the oracle's order
        out_s = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        out_i = torch.empty((nq, k), dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        idx.search_device_noalloc(q.data_ptr(), nq, k, out_s.data_ptr(), out_i.data_ptr())
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"


def test_noalloc_search_rejects_oversized_requests_and_bad_queries():
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
    q[1, 17] = float("inf")
    with pytest.raises(ValueError, match="query 1 coordinate 17"):
        idx.search_device_noalloc(q.data_ptr(), 3, 5, out_s.data_ptr(), out_i.data_ptr())
    q[1, 17] = 0.0
    assert idx.search_device_noalloc(q.data_ptr(), 3, 5, out_s.data_ptr(), out_i.data_ptr()) == 5
