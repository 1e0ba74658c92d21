"""CCM merge compressors: module semantics, checkpoint layout, in-pool forms (CPU) and the fused kernel (GPU)."""
import pytest
import torch

from fastcache_b200.compress import (KVCacheHybridCompressor, KVCacheLinearCompressor,
                                     KVCacheLinearDecoupleCompressor, MiniCPMKVCompressor, ccm_output_len,
                                     load_compressor, save_compressor)
from fastcache_b200.compress.inpool import _rows, ccm_compress_in_pool, ccm_compress_reference
from helpers import random_compressor


def test_decouple_semantics_and_lengths():
    m = random_compressor(KVCacheLinearDecoupleCompressor, 2, 16, 4)
    k, v = torch.randn(2, 3, 37, 16), torch.randn(2, 3, 37, 16)
    out = m([(k, v), (k, v)], it_len=[10, 27])
    # image 10 -> 2 + 2 remainder, text 27 -> 6 + 3 remainder
    assert out[0][0].shape == (2, 3, 13, 16) and m.output_len(37, 10) == 13 == ccm_output_len(37, 10, 4, 1)
    z = k[:, :, 10:34].reshape(2, 3, 6, 64)
    assert torch.allclose(out[1][0][:, :, 4:10], m.compress_tk[1](z), atol=1e-6)
    assert torch.equal(out[0][0][:, :, 2:4], k[:, :, 8:10]) and torch.equal(out[0][1][:, :, 10:], v[:, :, 34:])
    # a segment shorter than min_seq_len * f stays as it is
    m2 = random_compressor(KVCacheLinearDecoupleCompressor, 1, 16, 4, min_seq_len=2)
    assert m2([(k, v)], it_len=[5, 32])[0][0].shape[2] == 5 + 8


def test_checkpoint_layouts_round_trip(tmp_path):
    m = random_compressor(KVCacheLinearDecoupleCompressor, 3, 16, 5)
    keys = set(m.state_dict())
    assert "compress_tk.2.6.bias" in keys and "compress_iv.0.0.weight" in keys and "attention.1.weight" in keys
    assert m.state_dict()["compress_ik.0.0.weight"].shape == (16, 80)
    path = str(tmp_path / "c.pth")
    save_compressor(m, path, epoch=3, loss=0.5)
    blob = torch.load(path, weights_only=False)
    assert set(blob) == {"epoch", "model_state_dict", "optimizer_state_dict", "scheduler_state_dict", "loss"}
    m2 = load_compressor(path)
    assert isinstance(m2, KVCacheLinearDecoupleCompressor) and m2.compression_factor == 5 and m2.n_layer == 3
    x = [(torch.randn(1, 2, 23, 16), torch.randn(1, 2, 23, 16))] * 3
    assert torch.equal(m(x, [7, 16])[2][1], m2(x, [7, 16])[2][1])
    # the two other accepted wrappings: {'model_state_dict': sd} and a bare state dict
    assert load_compressor({"model_state_dict": m.state_dict()}).n_layer == 3
    h = random_compressor(KVCacheHybridCompressor, 2, 16, 4)
    assert not any(k.startswith(("compress_ik", "attention")) for k in h.state_dict())
    assert isinstance(load_compressor(h.state_dict()), KVCacheHybridCompressor)
    assert isinstance(load_compressor(m.state_dict(), kind="minicpm"), MiniCPMKVCompressor)
    lin = random_compressor(KVCacheLinearCompressor, 2, 16, 2)
    assert set(k.split(".")[0] for k in lin.state_dict()) == {"compress_k", "compress_v", "attention"}
    assert isinstance(load_compressor(lin.state_dict()), KVCacheLinearCompressor)


def _pool(L, nb, H, bs, D, dtype=torch.float32, device="cpu"):
    g = torch.Generator().manual_seed(0)
    return torch.randn(L, 2, nb, H, bs, D, generator=g).to(dtype).to(device)


@pytest.mark.parametrize("cls", [KVCacheLinearDecoupleCompressor, KVCacheHybridCompressor])
def test_in_pool_matches_module(cls):
    L, H, D, bs, f = 2, 2, 16, 8, 4
    m = random_compressor(cls, L, D, f)
    pool = _pool(L, 12, H, bs, D)
    table, n, img = [5, 2, 9, 0, 7], 37, 10
    blocks = torch.tensor(table)
    hf = [(_rows(pool[l, 0], blocks, n).permute(1, 0, 2)[None].clone(),
           _rows(pool[l, 1], blocks, n).permute(1, 0, 2)[None].clone()) for l in range(L)]
    want = m(hf, it_len=[img, n - img])
    new = ccm_compress_in_pool(pool, [table], [n], [img], m.pack())
    assert new == [want[0][0].shape[2]] == [m.output_len(n, img)]
    for l in range(L):
        for kv in (0, 1):
            got = _rows(pool[l, kv], blocks, new[0]).permute(1, 0, 2)
            assert torch.allclose(got, want[l][kv][0], atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("cls,f", [(KVCacheLinearDecoupleCompressor, 4), (KVCacheHybridCompressor, 5),
                                   (KVCacheLinearDecoupleCompressor, 2)])
def test_fused_kernel_matches_reference(cls, f):
    from fastcache_b200.ops.loader import ext
    L, H, D, bs = 3, 2, 128, 64
    m = random_compressor(cls, L, D, f)
    w = m.pack(torch.bfloat16, "cuda")
    pool = _pool(L, 40, H, bs, D, torch.bfloat16, "cuda")
    tables = [[3, 7, 1, 9, 12, 30, 31, 33, 35, 20, 21], [5, 6, 22, 23], [8], [10, 11]]
    lens, imgs = [640, 200, 9, 100], [576, 0, 4, 100]
    want = pool.clone()
    new_ref = [ccm_compress_reference(want, bt, n, i, w) for bt, n, i in zip(tables, lens, imgs)]
    new = ccm_compress_in_pool(pool, tables, lens, imgs, w)
    torch.cuda.synchronize()
    assert ext().read_status(0) == 0
    assert new == new_ref
    for bt, n in zip(tables, new):
        blocks = torch.tensor(bt, device="cuda")
        for l in range(L):
            for kv in (0, 1):
                a = _rows(pool[l, kv], blocks, n).float()
                b = _rows(want[l, kv], blocks, n).float()
                assert (a - b).abs().max().item() < 3e-2 * max(1.0, b.abs().max().item())


@pytest.mark.gpu
def test_fused_kernel_layer_chunks_equal_whole():
    L, H, D, bs, f = 4, 2, 128, 32, 4
    m = random_compressor(KVCacheLinearDecoupleCompressor, L, D, f)
    w = m.pack(torch.bfloat16, "cuda")
    a = _pool(L, 16, H, bs, D, torch.bfloat16, "cuda")
    b = a.clone()
    tables, lens, imgs = [[1, 2, 3, 4, 5, 6]], [170], [64]
    ccm_compress_in_pool(a, tables, lens, imgs, w)
    ccm_compress_in_pool(b, tables, lens, imgs, w, 0, 1)
    ccm_compress_in_pool(b, tables, lens, imgs, w, 1, 4)
    assert torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_fused_kernel_head_groups(G):
    """A tile holds 128 / G output rows of G heads: every grouping gives the rows of the PyTorch statement."""
    from fastcache_b200.ops.compress_cuda import _batch_meta
    from fastcache_b200.ops.loader import ext
    L, H, D, bs, f = 2, 8, 128, 64, 4
    m = random_compressor(KVCacheLinearDecoupleCompressor, L, D, f)
    w = m.pack(torch.bfloat16, "cuda")
    pool = _pool(L, 24, H, bs, D, torch.bfloat16, "cuda")
    tables = [[3, 7, 1, 9, 12, 20, 21, 22, 23, 2, 11], [5, 6, 14, 15], [8]]
    lens, imgs = [650, 203, 9], [577, 0, 4]
    want = pool.clone()
    new = [ccm_compress_reference(want, bt, n, i, w) for bt, n, i in zip(tables, lens, imgs)]
    bt_d, lens_d = _batch_meta(pool, tables, lens)
    img_d = torch.tensor(imgs, dtype=torch.int32, device="cuda")
    e = ext()
    e.ccm_compress(pool, bt_d, lens_d, img_d, w.w1, w.b1, w.w2, w.b2, w.w3, w.b3, 0, L, 0, f, int(w.min_seq_len),
                   bool(w.single_segment), e.status_tensor(0), G)
    torch.cuda.synchronize()
    assert e.read_status(0) == 0
    for bt, n in zip(tables, new):
        blocks = torch.tensor(bt, device="cuda")
        for l in range(L):
            for kv in (0, 1):
                a = _rows(pool[l, kv], blocks, n).float()
                b = _rows(want[l, kv], blocks, n).float()
                assert (a - b).abs().max().item() < 3e-2 * max(1.0, b.abs().max().item())


def test_heads_per_tile_minimises_tiles():
    from fastcache_b200.ops.ccm_cuda import heads_per_tile
    assert heads_per_tile(32, [640] * 15, [576] * 15, 4, 1, False) == 8      # 144 + 16 output rows per head
    assert heads_per_tile(8, [4096] * 8, [0] * 8, 2, 1, False) == 1          # long segments fill tiles by themselves
    assert heads_per_tile(3, [640], [576], 4, 1, False) == 1                 # 3 heads: no other group divides them
