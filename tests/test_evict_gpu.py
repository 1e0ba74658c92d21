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


@pytest.mark.parametrize("D,Hq,H,w,tc", [(128, 8, 2, 64, True), (128, 8, 2, 64, False), (64, 4, 4, 32, False),
                                         (128, 4, 1, 64, True), (128, 4, 2, 32, True), (128, 2, 2, 64, True)])
def test_snapkv_scores_kernel_matches_torch_statement(D, Hq, H, w, tc):
    """tc: the tcgen05 kernel (Q K^T by query row for the row statistics, K Q^T by key for the votes); else mma.sync."""
    from fastcache_b200.ops import ext as _ext
    before = _ext().snapkv_tensor_cores()
    _ext().set_snapkv_tensor_cores(tc)
    try:
        _snapkv_case(D, Hq, H, w)
    finally:
        _ext().set_snapkv_tensor_cores(before)


def test_snapkv_tensor_core_kernel_long_rows_block_256():
    """Many key tiles (the three-stage ring and both accumulators wrap several times), block size 256, requests
    that end inside a tile and one whose evictable part is a single tile."""
    _snapkv_case(128, 8, 2, 64, nb=24, bs=256, tables=[[3, 7, 1, 9, 12, 20, 21, 22, 23], [5, 6, 2], [4]],
                 lens=[2100, 641, 130])


def _snapkv_case(D, Hq, H, w, nb=40, bs=16, tables=None, lens=None):
    from fastcache_b200.compress.inpool import _rows
    from fastcache_b200.compress.scorers import snapkv
    from fastcache_b200.ops import ext
    from fastcache_b200.ops.compress_cuda import _batch_meta
    from fastcache_b200.ops.snapkv import snapkv_scores_cuda
    L = 2
    pool = _pool(L=L, nb=nb, bs=bs, H=H, D=D, seed=3)
    if tables is None:
        tables = [[3, 7, 1, 9, 12, 30, 31, 33, 34, 35, 36, 37, 38], [5, 6, 20, 21, 22, 23, 24, 25, 26, 2, 4]]
        lens = [200, 170]
    g = torch.Generator().manual_seed(9)
    window_q = [{l: torch.randn(w, Hq, D, generator=g).to(torch.bfloat16).cuda() for l in range(L)} for _ in lens]
    bt_d, lens_d = _batch_meta(pool, tables, lens)
    status = ext().status_tensor(0)
    got = snapkv_scores_cuda(pool, bt_d, lens_d, max(lens), window_q, {"window": w, "kernel_size": 5}, status)
    torch.cuda.synchronize()
    assert got is not None and ext().read_status(0) == 0
    for i, (bt, n) in enumerate(zip(tables, lens)):
        blocks = torch.as_tensor(bt, dtype=torch.long, device="cuda")
        for l in range(L):
            k = _rows(pool[l, 0], blocks, n).permute(1, 0, 2)
            want = snapkv(k, None, window_q[i][l].permute(1, 0, 2), window=w, kernel_size=5)     # [H, n]
            a, b = got[i, l, :, :n - w], want[:, :n - w]
            assert (a - b).abs().max().item() < 2e-3 * b.abs().max().item() + 1e-6
            assert torch.all(got[i, l, :, n - w:n] > 1e37) and torch.all(torch.isinf(got[i, l, :, n:]))


def test_snapkv_eviction_in_pool_keeps_window_and_top_votes():
    pool = _pool(L=2, nb=40, bs=16, H=2, D=128, seed=5)
    tables, lens, kept = [[3, 7, 1, 9, 12, 30, 31, 33, 34, 35, 36, 37, 38]], [200], [100]
    g = torch.Generator().manual_seed(2)
    wq = [{l: torch.randn(64, 8, 128, generator=g).to(torch.bfloat16).cuda() for l in range(2)}]
    before = pool.clone()
    out = evict_in_pool(pool, tables, lens, "snapkv", kept, wq, {"window": 64, "kernel_size": 5})
    torch.cuda.synchronize()
    assert out == kept
    # the last 64 rows of the request (the window) end up as the last 64 kept rows, in order
    idx = torch.tensor(tables[0], device="cuda")
    flat = lambda p: p[:, :, idx].permute(0, 1, 2, 4, 3, 5).reshape(2, 2, -1, 2, 128)   # noqa: E731
    assert torch.equal(flat(pool)[:, :, 36:100], flat(before)[:, :, 136:200])


@pytest.mark.parametrize("D,Hq,H,w,tc", [(128, 8, 2, 64, True), (128, 8, 2, 64, False), (64, 4, 4, 32, False)])
def test_expected_attention_scores_kernel_matches_torch_statement(D, Hq, H, w, tc):
    """tc: the tcgen05 kernel (K Sigma as a tensor-core product, Sigma as hi + lo bf16); else the FP32-pipe kernel."""
    from fastcache_b200.ops import ext as _ext
    before = _ext().ea_tensor_cores()
    _ext().set_ea_tensor_cores(tc)
    try:
        _expected_attention_case(D, Hq, H, w)
    finally:
        _ext().set_ea_tensor_cores(before)


def test_expected_attention_tensor_core_kernel_long_rows_block_256():
    """Several 128-key tiles per CTA and several CTAs per (layer, head, request); block size 256 (one TMA box per
    tile) and lengths that end inside a tile."""
    from fastcache_b200.compress.inpool import _rows
    from fastcache_b200.compress.scorers import expected_attention
    from fastcache_b200.ops import ext
    from fastcache_b200.ops.compress_cuda import _batch_meta
    from fastcache_b200.ops.snapkv import stack_window_queries
    L, H, Hq, D, w = 2, 2, 8, 128, 64
    pool = (_pool(L=L, nb=24, bs=256, H=H, D=D, seed=9).float() * 0.5).to(torch.bfloat16)
    tables = [[3, 7, 1, 9, 12, 20, 21, 22, 23], [5, 6, 2, 4, 0]]
    lens = [2100, 1153]
    g = torch.Generator().manual_seed(5)
    window_q = [{l: (torch.randn(w, Hq, D, generator=g) * 0.5).to(torch.bfloat16).cuda() for l in range(L)}
                for _ in lens]
    bt_d, lens_d = _batch_meta(pool, tables, lens)
    status = ext().status_tensor(0)
    assert ext().ea_tensor_cores()
    got = ext().expected_attention_scores(pool, bt_d, lens_d, max(lens), stack_window_queries(window_q, L), 4, status)
    torch.cuda.synchronize()
    assert ext().read_status(0) == 0
    for i, (bt, n) in enumerate(zip(tables, lens)):
        blocks = torch.as_tensor(bt, dtype=torch.long, device="cuda")
        for l in range(L):
            k = _rows(pool[l, 0], blocks, n).permute(1, 0, 2)
            v = _rows(pool[l, 1], blocks, n).permute(1, 0, 2)
            want = expected_attention(k, v, window_q[i][l].permute(1, 0, 2), n_sink=4)
            diff = got[i, l, :, 4:n] - torch.log(want[:, 4:n])
            assert (diff - diff.mean(dim=1, keepdim=True)).abs().max().item() < 2e-2
            assert torch.all(got[i, l, :, :4] > 1e37) and torch.all(torch.isinf(got[i, l, :, n:]))


def _expected_attention_case(D, Hq, H, w):
    from fastcache_b200.compress.inpool import _rows
    from fastcache_b200.compress.scorers import expected_attention
    from fastcache_b200.ops import ext
    from fastcache_b200.ops.compress_cuda import _batch_meta
    from fastcache_b200.ops.snapkv import stack_window_queries
    L = 2
    pool = (_pool(L=L, nb=40, bs=16, H=H, D=D, seed=7).float() * 0.5).to(torch.bfloat16)
    tables = [[3, 7, 1, 9, 12, 30, 31, 33, 34, 35, 36, 37, 38], [5, 6, 20, 21, 22, 23, 24, 25, 26, 2, 4]]
    lens = [200, 170]
    g = torch.Generator().manual_seed(4)
    window_q = [{l: (torch.randn(w, Hq, D, generator=g) * 0.5).to(torch.bfloat16).cuda() for l in range(L)}
                for _ in lens]
    bt_d, lens_d = _batch_meta(pool, tables, lens)
    status = ext().status_tensor(0)
    got = ext().expected_attention_scores(pool, bt_d, lens_d, max(lens), stack_window_queries(window_q, L), 4, status)
    torch.cuda.synchronize()
    assert ext().read_status(0) == 0
    for i, (bt, n) in enumerate(zip(tables, lens)):
        blocks = torch.as_tensor(bt, dtype=torch.long, device="cuda")
        for l in range(L):
            k = _rows(pool[l, 0], blocks, n).permute(1, 0, 2)
            v = _rows(pool[l, 1], blocks, n).permute(1, 0, 2)
            want = expected_attention(k, v, window_q[i][l].permute(1, 0, 2), n_sink=4)        # [H, n]
            diff = got[i, l, :, 4:n] - torch.log(want[:, 4:n])
            assert (diff - diff.mean(dim=1, keepdim=True)).abs().max().item() < 2e-2          # same up to a constant
            assert torch.all(got[i, l, :, :4] > 1e37) and torch.all(torch.isinf(got[i, l, :, n:]))
