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


def test_probability_space_loss_interface():
    from fastcache_b200.compress.research import count_true_segments_with_zeros, logits_to_onehot

    torch.manual_seed(0)
    loss = KVCacheCompressionLoss("logit")
    loss.alpha, loss.beta = 0.4, 0.4
    a = torch.softmax(torch.randn(2, 6, 10), -1)
    b = torch.softmax(torch.randn(2, 6, 10), -1)
    assert loss.prob_loss(a, a) < loss.prob_loss(a, b)
    # top-p mask: smallest prefix of the sorted tokens whose mass reaches the threshold
    m = loss.get_top_p_mask(a)
    kept = (a * m).sum(-1)
    assert bool((kept >= loss.p_threshold - 1e-6).all())
    smallest = torch.where(m, a, torch.ones_like(a)).min(-1).values
    assert bool((kept - smallest < loss.p_threshold).all())               # dropping the last one falls short
    assert loss.indices_to_mask(torch.tensor([[1, 0]]), 3).tolist() == [[[False, True, False], [True, False, False]]]
    hs = [torch.randn(2, 6, 8) for _ in range(3)]
    same = loss.forward_attn(a, a, (2, 3, 0), hs, hs)
    diff = loss.forward_attn(a, b, (2, 3, 0), hs, [h + 0.5 * torch.randn_like(h) for h in hs])
    assert same < diff
    steps = [[torch.full((2, 1, 4), float(t * 10 + l)) for l in range(3)] for t in range(5)]
    per_layer = loss.cvt_hidden_states(steps)
    assert len(per_layer) == 3 and per_layer[1].shape == (2, 5, 4) and per_layer[1][0, :, 0].tolist() == [1, 11, 21, 31, 41]
    acc, ta, tb = loss.calc_metrics(a, a)
    assert acc == 1.0 and torch.equal(ta, tb)
    acc3, run3, ppl, _, _ = loss.calc_metrics3(a, a)
    assert acc3 == 1.0 and run3 == 12.0 and ppl > 1.0
    assert loss.calc_metrics4(a, b, a)[1:3] == (1.0, 1.0)
    assert len(loss.calc_metrics2(a, b, b[:, :4])) == 5 and loss.loss_gen(a, b, b[:, :4]) > 0
    assert KVCacheCompressionLoss("label").loss_weight(a, b) > KVCacheCompressionLoss("label").prob_loss(a, b)
    w, o = loss.compute_attention_patterns(torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8))
    assert torch.allclose(w.sum(-1), torch.ones(1, 2, 4)) and o.shape == (1, 2, 4, 8)
    assert count_true_segments_with_zeros(torch.tensor([True, True, False, True])) == [3, 1]
    assert count_true_segments_with_zeros(torch.tensor([False, True, True, False])) == [1, 3, 0]
    assert logits_to_onehot(torch.tensor([[0.1, 0.9]])).tolist() == [[0, 1]]


def test_training_datasets_encode_turns():
    from fastcache_b200.compress.train_data import CustomDataset, CustomImageTextDataset

    class Tok:
        def __call__(self, text, **kw):
            n = min(len(text.split()), kw.get("max_length", 512))
            if kw.get("padding") == "max_length":
                n = kw["max_length"]
            return {"input_ids": torch.arange(n)[None], "attention_mask": torch.ones(1, n, dtype=torch.long)}

    ds = CustomDataset(["a b c", "d e"], Tok(), max_length=4)
    assert len(ds) == 2 and ds[0]["input_ids"].tolist() == [0, 1, 2] and "draft_input_ids" not in ds[0]
    ds.new_tokenizer(Tok())
    assert ds[1]["draft_input_ids"].shape == (4,)

    class Proc:
        def __call__(self, images=None, text=None, **kw):
            n = kw.get("max_length", 3) if kw.get("padding") == "max_length" else 3
            return {"input_ids": torch.zeros(1, n, dtype=torch.long), "attention_mask": torch.ones(1, n, dtype=torch.long),
                    "pixel_values": torch.zeros(1, 3, 4, 4)}

    conv = [([("describe", "img0"), ("more", "img1"), ("text only", None)], [1, 1, 0])]
    items = CustomImageTextDataset(conv, Proc(), max_length=8)[0]
    assert len(items) == 2 and items[0]["input_ids"].shape == (8,) and items[0]["pixel_values"].shape == (3, 4, 4)
    assert CustomImageTextDataset(conv, Proc(), 8, launch_padding_flag=False)[0][0]["input_ids"].shape == (3,)


def test_script_level_helpers(tmp_path):
    import json
    from fastcache_b200.compress import train as T
    comp = KVCacheLinearDecoupleCompressor(None, 2, 1, n_layer=2, nhead=2, head_dim=8)
    opt = torch.optim.Adam(comp.parameters(), lr=1e-3)
    sched = torch.optim.lr_scheduler.ReduceLROnPlateau(opt)
    last = T.save_checkpoint(3, comp, opt, sched, 0.25, True, str(tmp_path), "c.pth")
    assert os.path.exists(last) and os.path.exists(tmp_path / "best_c.pth")
    other = KVCacheLinearDecoupleCompressor(None, 2, 1, n_layer=2, nhead=2, head_dim=8)
    assert T.load_checkpoint(other, torch.optim.Adam(other.parameters()), None, last) == (3, 0.25)
    assert all(torch.equal(a, b) for a, b in zip(comp.state_dict().values(), other.state_dict().values()))
    assert T.load_checkpoint(other, None, None, str(tmp_path / "none.pth")) == (0, float("inf"))
    assert T.load_finetune_compressor(last).compression_factor == 2
    assert T.parse_string_with_image("<image>\nWhat is this?") == ("What is this?", 1)
    assert T.parse_string_with_image("plain") == ("plain", 0)
    data = [{"conversations": [{"from": "human", "value": "a   b\nc"}, {"from": "gpt", "value": "x"}]},
            {"conversations": [{"from": "gpt", "value": "skip"}]}, {"conversations": []}]
    path = tmp_path / "t.json"
    path.write_text(json.dumps(data))
    assert T.load_text_data(str(path), -1) == ["a b c"]
    fwd = _toy()
    mk = lambda s: [(torch.randn(2, 2, 12, 8, generator=torch.Generator().manual_seed(s + l)),
                     torch.randn(2, 2, 12, 8, generator=torch.Generator().manual_seed(9 + s + l))) for l in range(2)]
    loss, acc = T.validate_llava(comp, fwd, [mk(0), mk(1)], it_len_of=lambda b: (4, 8))
    assert loss > 0 and 0.0 <= acc <= 1.0
    T.set_seed(3)
    a = torch.rand(1)
    T.set_seed(3)
    assert torch.equal(a, torch.rand(1)) and T.finetune_com is T.finetune_llava
