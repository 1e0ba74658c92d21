"""Distillation loop of the merge compressor on a toy differentiable reader of the KV cache."""
import os

import torch

from fastcache_b200.compress import KVCacheLinearDecoupleCompressor, load_compressor
from fastcache_b200.compress.train import FinetuneConfig, KVCacheCompressionLoss, finetune_compressor


def _toy(D=8, V=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(D, generator=g)
    head = torch.randn(V, D, generator=g)

    def forward_with_kv(batch, kv):
        if kv is None:
            return None, [], batch
        hs = []
        for k, v in kv:
            a = torch.softmax((k @ q) / D ** 0.5, dim=-1)           # [B, H, S]
            hs.append((a[..., None] * v).sum(2).mean(1))            # [B, D]
        h = torch.stack(hs).mean(0)
        return h @ head.T, hs, kv
    return forward_with_kv


def test_loss_terms_and_accuracy():
    loss = KVCacheCompressionLoss("logit")
    a, b = torch.randn(4, 10), torch.randn(4, 10)
    total, parts = loss(a, b, None, [torch.randn(4, 8)], [torch.randn(4, 8)])
    assert total > 0 and {"js", "l1", "ce", "mse", "cos"} <= set(parts)
    same, _ = loss(a, a)
    assert same < total and loss.accuracy(a, a) == 1.0
    lab = KVCacheCompressionLoss("label")(a, b, torch.randint(0, 10, (4,)))[1]
    assert set(lab) == {"ce"}


def test_finetune_improves_and_checkpoints(tmp_path):
    torch.manual_seed(0)
    fwd = _toy()
    comp = KVCacheLinearDecoupleCompressor(None, 2, 1, n_layer=2, nhead=2, head_dim=8)
    mk = lambda s: [(torch.randn(4, 2, 12, 8, generator=torch.Generator().manual_seed(s + l)),
                     torch.randn(4, 2, 12, 8, generator=torch.Generator().manual_seed(100 + s + l)))
                    for l in range(2)]
    train, val = [mk(s) for s in range(0, 60, 10)], [mk(1000)]
    cfg = FinetuneConfig(lr=5e-3, epochs=6, compression_factor=2, out_dir=str(tmp_path), name="toy")
    out = finetune_compressor(comp, fwd, train, val, cfg, it_len_of=lambda b: (4, 8))
    h = out["history"]
    assert len(h) == 6 and h[-1]["train_loss"] < h[0]["train_loss"]
    assert os.path.exists(out["last"]) and os.path.exists(out["best"])
    again = load_compressor(out["last"])
    assert again.compression_factor == 2 and again.n_layer == 2
    cfg2 = FinetuneConfig(lr=5e-3, epochs=7, out_dir=str(tmp_path), name="toy", is_continue=True)
    more = finetune_compressor(again, fwd, train, val, cfg2, it_len_of=lambda b: (4, 8))
    assert [r["epoch"] for r in more["history"]] == [6]


def test_named_recipes_pick_the_compressor_family(tmp_path):
    from types import SimpleNamespace
    from fastcache_b200.compress import KVCacheHybridCompressor
    from fastcache_b200.compress.train import finetune_com_minicpm, finetune_llava

    torch.manual_seed(0)
    fwd = _toy()
    cfg = SimpleNamespace(num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, hidden_size=16,
                          head_dim=8)
    mk = lambda s: [(torch.randn(2, 2, 12, 8, generator=torch.Generator().manual_seed(s + l)),
                     torch.randn(2, 2, 12, 8, generator=torch.Generator().manual_seed(50 + s + l)))
                    for l in range(2)]
    samples = [mk(s) for s in range(5)]
    comp, out = finetune_com_minicpm(SimpleNamespace(config=cfg), samples, forward_with_kv=fwd,
                                     it_len_of=lambda b: (0, 12), out_dir=str(tmp_path), num_epochs=2,
                                     compression_ratio=2, compressor_save_name="mini")
    assert isinstance(comp, KVCacheHybridCompressor) and not hasattr(comp, "compress_ik")
    assert len(out["history"]) == 2 and os.path.basename(out["best"]) == "best_mini.pth"
    comp2, out2 = finetune_llava(SimpleNamespace(config=cfg), samples, forward_with_kv=fwd,
                                 it_len_of=lambda b: (4, 8), out_dir=str(tmp_path), num_epochs=1,
                                 compression_ratio=2, compressor_save_name="lv")
    assert isinstance(comp2, KVCacheLinearDecoupleCompressor) and len(out2["history"]) == 1
    # resume from the saved file through the load path of the recipe
    comp3, _ = finetune_llava(SimpleNamespace(config=cfg), samples, forward_with_kv=fwd,
                              it_len_of=lambda b: (4, 8), out_dir=str(tmp_path), num_epochs=1,
                              compression_ratio=2, compressor_save_name="lv2",
                              compressor_load_path=out2["last"])
    assert comp3.compression_factor == 2
