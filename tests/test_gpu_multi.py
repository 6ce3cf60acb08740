"""One handle over several devices of one process (tv_multi_*, turbovec_b200.MultiGpuIndex).

The shards of a handle may share a device, so everything here runs on one GPU (devices = [0, 0, 0]) and, where two
are present, once more on devices [0, 1].  The handle must behave exactly like one index holding all the rows:
same scores bit for bit, same slots / ids, same errors, through adds, masks, allowlists and removals that move a row
from one shard to another.
"""
import numpy as np
import pytest

from tests.util import anisotropic

pytestmark = pytest.mark.gpu


def _device_lists():
    import torch
    lists = [[0, 0, 0]]
    if torch.cuda.device_count() >= 2:
        lists.append([0, 1])
    return lists


@pytest.mark.parametrize("bits,dim", [(4, 256), (2, 128)])
def test_positional_handle_equals_one_index(bits, dim):
    import turbovec_b200 as T
    n = 3000
    x = anisotropic(n, dim, seed=81)
    q = anisotropic(40, dim, seed=81, offset=5)
    rng = np.random.default_rng(8)
    for devices in _device_lists():
        one = T.TurboQuantIndex(dim, bits)
        many = T.MultiGpuIndex(dim, bits, devices=devices, chunk_blocks=2)         # 64-slot chunks
        assert many.n_shards == len(devices)
        for a, b in ((0, 1), (1, 70), (70, 1000), (1000, n)):                      # runs that start and end inside chunks
            one.add(x[a:b])
            many.add(x[a:b])
        assert len(many) == n and sum(many.shard_len(i) for i in range(many.n_shards)) == n

        def same(k, mask=None):
            want = one.search(q, k, mask=mask) if mask is not None else one.search(q, k)
            got = many.search(q, k, mask=mask)
            return np.array_equal(got[1], want[1]) and np.array_equal(got[0].view(np.uint32), want[0].view(np.uint32))

        assert same(10) and same(100) and same(1)
        mask = rng.random(n) < 0.1
        assert same(10, mask)
        few = np.zeros(n, bool)
        few[[5, 64, 2999]] = True                                                   # n_allowed < k, one shard without any
        assert same(10, few)
        none = np.zeros(n, bool)
        s, i = many.search(q, 10, mask=none)
        assert s.shape == (40, 0) and i.shape == (40, 0)
        with pytest.raises(ValueError, match="mask length"):
            many.search(q, 10, mask=np.ones(n - 1, bool))
        for victim in (0, 63, 64, 1500, -1, 17):                                     # same-shard and cross-shard moves, the last row
            victim = len(many) - 1 if victim < 0 else victim
            assert many.swap_remove(victim) == one.swap_remove(victim)
        assert len(many) == len(one) and same(10) and same(10, mask[: len(one)])
        with pytest.raises(IndexError):
            many.swap_remove(len(many))
        many.add(x[:500])
        one.add(x[:500])
        assert same(50)


def test_idmapped_handle_equals_one_index():
    import turbovec_b200 as T
    dim, n = 256, 4000
    x = anisotropic(n, dim, seed=82)
    ids = (np.random.default_rng(82).permutation(n) + 10**12).astype(np.uint64)
    q = anisotropic(7, dim, seed=82, offset=3)
    rng = np.random.default_rng(9)
    for devices in _device_lists():
        one = T.IdMapIndex(dim, 4)
        many = T.MultiGpuIndex(dim, 4, devices=devices, id_mapped=True, chunk_blocks=4)
        for a, b in ((0, 999), (999, 1000), (1000, n)):
            one.add_with_ids(x[a:b], ids[a:b])
            many.add_with_ids(x[a:b], ids[a:b])

        def same(k, allow=None):
            want = one.search(q, k, allowlist=allow)
            got = many.search(q, k, allowlist=allow)
            return np.array_equal(got[1], want[1]) and np.array_equal(got[0].view(np.uint32), want[0].view(np.uint32))

        assert same(10) and same(200)
        allow = np.ascontiguousarray(ids[::9])
        assert same(10, allow) and same(1000, allow)
        with pytest.raises(KeyError):
            many.search(q, 5, allowlist=np.array([3], np.uint64))
        with pytest.raises(ValueError, match="empty"):
            many.search(q, 5, allowlist=np.array([], np.uint64))
        with pytest.raises(ValueError, match="already present"):
            many.add_with_ids(x[:2], ids[5:7])
        with pytest.raises(ValueError):
            many.add_with_ids(x[:2], np.array([1, 1], np.uint64))
        assert len(many) == n
        for victim in [int(v) for v in rng.choice(ids, 60, replace=False)]:
            assert many.remove(victim) and one.remove(victim)
            assert not many.contains(victim)
        assert not many.remove(12345)
        assert len(many) == len(one) and np.array_equal(many.ids(), one.ids())
        assert same(10) and same(10, np.ascontiguousarray(one.ids()[::5]))


def test_failed_add_leaves_every_shard_unchanged():
    """A batch whose invalid value lands in a later shard: the runs already appended to other shards are taken back
    (all or nothing, turbovec/src/lib.rs:889-930) and the offender is reported by its index in the batch."""
    import turbovec_b200 as T
    dim = 128
    x = anisotropic(700, dim, seed=83)
    q = anisotropic(5, dim, seed=83, offset=1)
    many = T.MultiGpuIndex(dim, 4, devices=[0, 0, 0], chunk_blocks=2)
    many.add(x[:100])
    before = many.search(q, 10)
    lens = [many.shard_len(i) for i in range(3)]
    bad = x[100:600].copy()
    bad[450, 7] = np.inf
    with pytest.raises(ValueError, match="vector 450 coordinate 7"):
        many.add(bad)
    assert len(many) == 100 and [many.shard_len(i) for i in range(3)] == lens
    after = many.search(q, 10)
    assert np.array_equal(before[1], after[1]) and np.array_equal(before[0], after[0])
    many.add(x[100:])
    one = T.TurboQuantIndex(dim, 4)
    one.add(x)
    assert np.array_equal(many.search(q, 10)[1], one.search(q, 10)[1])
