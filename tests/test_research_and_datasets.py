"""Research-path compressors / cache containers and the harness' dataset loaders (CPU)."""
import json
from types import SimpleNamespace

import torch

from fastcache_b200.compress.research import (CompressedDecoder, CompressedDecoder_OnlyMLP, CompressedKVCache,
                                              CompressibleCache, CrossModelKVCompressor,
                                              CrossModelRealKVCompressor, LLaMAKVCacheSampler, MAEEncoder,
                                              flatten_kv)
from fastcache_b200.serving.datasets import (DESCRIBE_PROMPT, load_image_data, load_image_data_milebench,
                                             synthetic_samples)


def _kv(layers=3, B=2, H=4, S=40, D=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B, H, S, D, generator=g), torch.randn(B, H, S, D, generator=g)) for _ in range(layers)]


def test_sampler_keeps_recent_rows_and_most_attended_older_rows():
    kv = _kv(S=40)
    # make row 5 of the last layer's keys point the same way as the newest key, scaled up
    kv[-1][0][:, :, 5, :] = 4.0 * kv[-1][0][:, :, -1, :]
    out, idx = LLaMAKVCacheSampler(recent_size=8).hybrid_sampling(kv, num_samples=12)
    assert idx.tolist() == sorted(idx.tolist()) and len(idx) == 12
    assert set(range(32, 40)) <= set(idx.tolist()) and 5 in idx.tolist()
    assert all(k.shape[2] == 12 and v.shape[2] == 12 for k, v in out)
    assert torch.equal(out[0][0], kv[0][0].index_select(2, idx))
    # fewer samples than the recent window: the window is what is kept
    _, idx2 = LLaMAKVCacheSampler(recent_size=8).hybrid_sampling(kv, num_samples=4)
    assert idx2.tolist() == list(range(32, 40))


def test_compressible_cache_lengths_and_clone():
    c = CompressibleCache.from_legacy_cache(_kv(layers=2, S=10))
    assert len(c) == 2 and c.get_seq_length() == 10 and c.get_actual_seq_length(1) == 10
    c.set_seen_tokens(100)                       # rows were compressed, positions keep counting
    k1 = torch.zeros(2, 4, 1, 16)
    c.update(k1, k1, 0)
    c.update(k1, k1, 1)
    assert c.get_seq_length() == 101 and c.get_actual_seq_length() == 11
    d = c.clone()
    d.key_cache[0].zero_()
    assert c.key_cache[0].abs().sum() > 0 and d.seen_tokens == 101
    assert len(c.to_legacy_cache()) == 2
    s = CompressedKVCache(2, 4, 16)
    s.update(k1, k1, 0)
    s.update(k1, k1, 0)
    assert s.get()[0][0].shape[2] == 2 and s.get()[1][0] is None


def test_mae_encoder_and_pooling_decoders_shapes():
    kv = _kv(layers=3, B=2, H=4, S=20, D=16)
    flat = flatten_kv(kv)
    assert flat.shape == (2, 3 * 20, 2 * 4 * 16)
    enc = MAEEncoder(input_dim=32, hidden_dim=64, num_layers=1, kv_dim=2 * 4 * 16, nhead=4).eval()
    h = enc(kv)
    assert h.shape == (2, 60, 32)
    # decoder rows carry one head's K|V features (F = 2 * D): [B, L * S, F]
    x = torch.randn(2, 3 * 20, 32)
    dec = CompressedDecoder(32, 64, 4 * 16, compression_ratio=5, num_layers=1, num_heads=4, num_llm_layers=3).eval()
    out = dec(x)
    assert len(out) == 3 and out[0][0].shape == (2, 4, 4, 16) and out[0][1].shape == (2, 4, 4, 16)
    assert dec.compress_with_len(x, 7)[1][0].shape == (2, 4, 7, 16)
    mlp = CompressedDecoder_OnlyMLP(32, 64, 4 * 16, compression_ratio=4, num_layers=3, num_heads=4).eval()
    assert mlp(x)[2][1].shape == (2, 4, 5, 16)


def test_cross_model_compressors_map_layers_heads_and_length():
    src = SimpleNamespace(num_hidden_layers=4, num_key_value_heads=4, num_attention_heads=4, hidden_size=64)
    tgt = SimpleNamespace(num_hidden_layers=2, num_key_value_heads=2, num_attention_heads=2, hidden_size=64)
    kv = _kv(layers=4, B=1, H=4, S=9, D=16)
    m = CrossModelKVCompressor(src, src.__class__(**{**tgt.__dict__, "num_key_value_heads": 4}), 2, tgt_dim=8).eval()
    out = m(kv)
    assert len(out) == 2 and out[0][0].shape == (1, 4, 5, 8)          # 9 rows -> 4 pairs + a padded pair
    w = m.layer_mixture(1)
    assert w.shape == (4,) and abs(float(w.detach().sum()) - 1.0) < 1e-5
    r = CrossModelRealKVCompressor(src, tgt, 3, tgt_dim=8).eval()
    o2 = r(kv)
    assert len(o2) == 2 and o2[1][1].shape == (1, 2, 3, 8)             # 2 source heads merged per target head
    # the mixture is differentiable end to end
    loss = sum(k.pow(2).mean() + v.pow(2).mean() for k, v in r(kv))
    loss.backward()
    assert r.layer_map_net[0].weight.grad is not None


def test_dataset_loaders(tmp_path):
    rows = [{"id": "a", "image": "gqa/1.jpg", "conversations": [{"from": "human", "value": "<image> q"},
                                                               {"from": "gpt", "value": "ans"}]},
            {"id": "b", "image": "coco/2.jpg", "conversations": [{"from": "human", "value": "q"}]},
            {"id": "c", "image": "gqa/3.jpg", "conversations": [{"from": "gpt", "value": "starts with the model"}]},
            {"id": "d", "conversations": [{"from": "human", "value": "text only"}]}]
    jp = tmp_path / "mix.json"
    jp.write_text(json.dumps(rows))
    s = load_image_data(str(jp), str(tmp_path / "imgs"), -1, seed=0)
    assert [x.source for x in s] == ["a"] and s[0].prompt == DESCRIBE_PROMPT and s[0].answers == ["ans"]
    assert isinstance(s[0].image, str) and s[0].image.endswith("gqa/1.jpg")     # file absent: the path is kept
    assert load_image_data(str(jp), str(tmp_path), 0) == []
    # MileBench layout
    for name, files in (("taskA", ["images/x.png", "images/sub/y.jpg", "images/notes.txt"]), ("noimgs", [])):
        d = tmp_path / "mile" / name
        d.mkdir(parents=True)
        (d / f"{name}.json").write_text("{}")
        for f in files:
            p = d / f
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_bytes(b"not really an image")
    (tmp_path / "mile" / "stray" / "images").mkdir(parents=True)               # no json beside it: ignored
    got = load_image_data_milebench(str(tmp_path / "mile"), -1, seed=1)
    assert sorted(x.source.split("/")[-1] for x in got) == ["x.png", "y.jpg"]
    assert len(load_image_data_milebench(str(tmp_path / "mile"), 1)) == 1
    syn = synthetic_samples(3, (28, 42), text_tokens=5, vocab=5000, seed=2)
    assert len(syn) == 3 and syn[0].image.shape == (3, 28, 42) and len(syn[0].prompt) == 5
    assert syn[0].prompt == synthetic_samples(3, (28, 42), 5, 5000, 2)[0].prompt
