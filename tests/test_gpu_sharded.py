"""The slot-sharded index on real devices.

One GPU: the shards of W ranks are built side by side on the same device and searched one after the other (no
process group, no kernel waits on another), their result keys are merged by the device merge with the round-robin
slot map, and the result must equal one index holding every vector.  Two GPUs (skipped with fewer): two NCCL ranks
run ShardedIdMapIndex end to end -- id-mapped adds, allowlist searches, removals that move a row between the GPUs
-- against a single-device IdMapIndex fed the same calls.
"""
import os
import socket

import numpy as np
import pytest

from tests.util import anisotropic

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,nq,k", [(2, 5, 10), (3, 70, 100), (8, 3, 10)])
def test_round_robin_shards_merged_on_device_equal_the_whole_index(world, nq, k):
    import torch
    import turbovec_b200 as T
    from turbovec_b200.sharded import SlotMap, pack_mask_words
    n, dim, cb = 9000, 256, 4                              # 128-slot chunks: 70 chunks over the ranks, ragged tail
    x = anisotropic(n, dim, seed=33)
    q = anisotropic(nq, dim, seed=33, offset=7)
    whole = T.TurboQuantIndex(dim, 4)
    whole.add(x)
    m = SlotMap(world, cb)
    shards = []
    for r in range(world):
        idx = T.TurboQuantIndex(dim, 4)
        for owner, off, ln in m.runs(0, n):
            if owner == r:
                idx.add(x[off:off + ln])
        assert len(idx) == m.local_len(r, n)
        shards.append(idx)
    mask = np.random.default_rng(9).random(n) < 0.05
    flags = torch.zeros(((n + 63) // 64) * 64, dtype=torch.uint8, device="cuda")
    flags[:n] = torch.from_numpy(mask.view(np.uint8)).cuda()
    words = pack_mask_words(torch, flags)
    qd = torch.from_numpy(q).cuda()
    for use_mask in (False, True):
        want_s, want_i = whole.search(q, k, mask=mask) if use_mask else whole.search(q, k)
        keys = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
        for r, idx in enumerate(shards):
            lw = m.local_mask_words(torch, words, r, n) if use_mask else None
            idx.search_device_keys(qd.data_ptr(), nq, k, keys[r].data_ptr(), 0, lw.data_ptr() if lw is not None else 0)
        s = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        i = torch.empty((nq, k), dtype=torch.int64, device="cuda")
        T.merge_keys_device(keys.data_ptr(), world, nq, k, s.data_ptr(), i.data_ptr(), device=0,
                            stream=torch.cuda.current_stream().cuda_stream, chunk_slots=m.chunk_slots)
        torch.cuda.synchronize()
        ke = want_s.shape[1]
        assert np.array_equal(i.cpu().numpy()[:, :ke], want_i) and np.array_equal(s.cpu().numpy()[:, :ke], want_s)


def _nccl_worker(rank, world, port, results):
    import torch
    import torch.distributed as dist
    import turbovec_b200 as T
    from turbovec_b200.sharded import ShardedIdMapIndex
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dim, n = 256, 6000
        x = anisotropic(n, dim, seed=44)
        ids = (np.random.default_rng(44).permutation(n) + 10**9).astype(np.uint64)
        q = anisotropic(9, dim, seed=44, offset=3)
        sh = ShardedIdMapIndex(dim, 4, chunk_blocks=8)          # 256-slot chunks
        ref = T.IdMapIndex(dim, 4, device=rank)
        ok = True
        for a, b in ((0, 1000), (1000, 1001), (1001, n)):
            sh.add_with_ids(x[a:b], ids[a:b])
            ref.add_with_ids(x[a:b], ids[a:b])
        ok &= len(sh) == n

        def same(k, allow=None):
            s, got = sh.search(q, k, allowlist=allow)
            rs, rid = ref.search(q, k, allowlist=allow)
            return bool(np.array_equal(got, rid) and np.array_equal(s, rs))

        ok &= same(10) and same(100)
        allow = np.ascontiguousarray(ids[::11])
        ok &= same(10, allow) and same(1000, allow)              # n_allowed < k
        rng = np.random.default_rng(5)
        for victim in [int(v) for v in rng.choice(ids, 40, replace=False)]:   # same-GPU and cross-GPU moves
            ok &= sh.remove(victim) == ref.remove(victim)
        ok &= len(sh) == len(ref) and bool(np.array_equal(sh.ids(), ref.ids()))
        ok &= same(10) and same(10, np.ascontiguousarray(sh.ids()[::7]))
        more = anisotropic(700, dim, seed=45)
        more_ids = (np.arange(700) + 5 * 10**9).astype(np.uint64)
        sh.add_with_ids(more, more_ids)
        ref.add_with_ids(more, more_ids)
        ok &= same(10) and same(50, more_ids)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_idmap_index_on_two_gpus():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_nccl_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}
