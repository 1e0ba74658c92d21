"""In-pool eviction kernels against the PyTorch statement on a copy of the pool."""
import pytest
import torch

from fastcache_b200.compress.inpool import evict_in_pool, evict_reference

pytestmark = pytest.mark.gpu


def _pool(L=3, nb=40, bs=16, H=2, D=128, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(L, 2, nb, H, bs, D, generator=g).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("method", ["knorm", "knorm_ref", "streaming_llm", "random"])
@pytest.mark.parametrize("D", [128, 64])
def test_evict_matches_reference(method, D):
    pool = _pool(D=D)
    tables = [[3, 7, 1, 9, 12, 30, 31], [5, 6, 20, 21, 22, 23, 24, 25, 26, 2, 4], [8]]
    lens = [100, 170, 9]
    kept = [50, 85, 4]
    want = pool.clone()
    for bt, n, k in zip(tables, lens, kept):
        evict_reference(want, bt, n, method, k, None, {})
    got = pool.clone()
    out = evict_in_pool(got, tables, lens, method, kept, None, {})
    torch.cuda.synchronize()
    assert out == kept
    bs = pool.shape[4]
    for bt, k in zip(tables, kept):
        nb = -(-k // bs)
        idx = torch.tensor(bt[:nb], device="cuda")
        a = got[:, :, idx].permute(0, 1, 2, 4, 3, 5).reshape(pool.shape[0], 2, -1, pool.shape[3], D)[:, :, :k]
        b = want[:, :, idx].permute(0, 1, 2, 4, 3, 5).reshape(pool.shape[0], 2, -1, pool.shape[3], D)[:, :, :k]
        assert torch.equal(a, b)
