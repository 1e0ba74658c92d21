"""Vision towers against HuggingFace `transformers` (CPU, fp32).

LLaVA-1.5 feeds its projector with hidden state -2 of the CLIP tower, class token dropped and without the final
layer norm (the reference applies all layers plus `post_layernorm`, nanovllm/models/llava.py:163-170; this package
follows the HuggingFace model the checkpoints were trained with and keeps the reference's behaviour as an option).
MiniCPM-V's SigLIP tower is compared on a full square grid, where the bucketed position ids reduce to the plain
table the HuggingFace model uses.
"""
import types

import pytest
import torch

transformers = pytest.importorskip("transformers")

from fastcache_b200.models.vision import CLIPVisionTower, SiglipVisionTower  # noqa: E402
from fastcache_b200.utils.loader import load_weights  # noqa: E402


def _cfg(**kw):
    return types.SimpleNamespace(**kw)


def test_clip_tower_matches_transformers_hidden_state_minus_two():
    from transformers import CLIPVisionConfig, CLIPVisionModel
    torch.manual_seed(0)
    hf_cfg = CLIPVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                              image_size=56, patch_size=14, hidden_act="quick_gelu", layer_norm_eps=1e-5)
    hf = CLIPVisionModel(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or n.endswith("bias"):
                p.add_(torch.randn_like(p) * 0.1)
    cfg = _cfg(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, image_size=56,
               patch_size=14, layer_norm_eps=1e-5)
    pixels = torch.randn(2, 3, 56, 56)
    with torch.no_grad():
        out = hf(pixel_values=pixels, output_hidden_states=True)
    for layer, post in ((-2, False), (-1, True)):
        tower = CLIPVisionTower(cfg, feature_layer=layer, apply_post_layernorm=post).float()
        stats = load_weights(tower, hf.state_dict().items())
        assert stats["unknown"] == 0 and stats["missing"] == []
        with torch.no_grad():
            got = tower(pixels)
        want = out.hidden_states[layer][:, 1:]
        if post:                                   # the reference's variant: all layers, then post_layernorm
            want = hf.vision_model.post_layernorm(out.hidden_states[-1])[:, 1:]
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


def test_siglip_tower_matches_transformers_on_a_full_grid():
    from transformers import SiglipVisionConfig, SiglipVisionModel
    torch.manual_seed(1)
    hf_cfg = SiglipVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                                image_size=56, patch_size=14, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6,
                                vision_use_head=False)
    hf = SiglipVisionModel(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or n.endswith("bias"):
                p.add_(torch.randn_like(p) * 0.1)
    cfg = _cfg(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, image_size=56,
               patch_size=14, layer_norm_eps=1e-6)
    tower = SiglipVisionTower(cfg).float()
    state = {k[len("vision_model."):]: v for k, v in hf.state_dict().items() if k.startswith("vision_model.")}
    stats = load_weights(tower, state.items())
    assert stats["unknown"] == 0 and stats["missing"] == []
    pixels = torch.randn(2, 3, 56, 56)
    with torch.no_grad():
        want = hf(pixel_values=pixels).last_hidden_state
        got, mask = tower(pixels, torch.tensor([[4, 4], [4, 4]]))
    assert bool(mask.all())
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


def test_minicpm_resampler_matches_its_published_statement():
    """The perceiver resampler of MiniCPM-V-2.6 stated with torch's own modules the way the model's published
    code does it (the reference borrows that code at load time, nanovllm/models/minicpm.py:329-340; it is not
    shipped with `transformers`): kv_proj -> LayerNorm, learned queries -> LayerNorm, nn.MultiheadAttention with the
    2-D sin-cos position table (w coordinate in the first half of the channels) added to the keys only and a key
    padding mask for ragged grids, LayerNorm, then `x @ proj`."""
    import numpy as np
    from torch import nn
    from fastcache_b200.models.vision import Resampler, sincos_2d
    torch.manual_seed(2)
    E, KV, Q, H = 64, 48, 8, 4
    ours = Resampler(Q, E, KV, num_heads=H, max_size=(10, 10)).float()
    for p in ours.parameters():
        torch.nn.init.normal_(p, std=0.2)

    # ---- the published statement
    def pos_1d(dim, pos):                                     # MAE-style table
        omega = 1.0 / 10000 ** (np.arange(dim // 2, dtype=np.float32) / (dim / 2))
        out = np.einsum("hw,d->hwd", pos, omega)
        return np.concatenate([np.sin(out), np.cos(out)], axis=-1)

    def pos_2d(dim, h, w):
        grid = np.meshgrid(np.arange(w, dtype=np.float32), np.arange(h, dtype=np.float32))   # w goes first
        return np.concatenate([pos_1d(dim // 2, grid[0]), pos_1d(dim // 2, grid[1])], axis=-1)

    table = torch.from_numpy(pos_2d(E, 10, 10)).float()
    torch.testing.assert_close(sincos_2d(E, 10, 10), table, rtol=1e-5, atol=1e-5)
    attn = nn.MultiheadAttention(E, H)
    kv_proj = nn.Linear(KV, E, bias=False)
    ln_q, ln_kv, ln_post = (nn.LayerNorm(E, eps=1e-6) for _ in range(3))
    with torch.no_grad():
        attn.in_proj_weight.copy_(ours.attn.in_proj_weight)
        attn.in_proj_bias.copy_(ours.attn.in_proj_bias)
        attn.out_proj.weight.copy_(ours.attn.out_proj.weight)
        attn.out_proj.bias.copy_(ours.attn.out_proj.bias)
        kv_proj.weight.copy_(ours.kv_proj.weight)
        for theirs, mine in ((ln_q, ours.ln_q), (ln_kv, ours.ln_kv), (ln_post, ours.ln_post)):
            theirs.weight.copy_(mine.weight)
            theirs.bias.copy_(mine.bias)
    tgt = torch.tensor([[3, 4], [2, 5], [4, 4]])
    counts = (tgt[:, 0] * tgt[:, 1]).tolist()
    L = max(counts)
    x = torch.randn(3, L, KV)
    pos = torch.zeros(3, L, E)
    pad = torch.zeros(3, L, dtype=torch.bool)
    for b, (h, w) in enumerate(tgt.tolist()):
        pos[b, : h * w] = table[:h, :w].reshape(h * w, E)
        pad[b, h * w:] = True
    with torch.no_grad():
        kv = ln_kv(kv_proj(x)).permute(1, 0, 2)                                    # L B E
        q = ln_q(ours.query)[:, None, :].expand(-1, 3, -1)
        out = attn(q, kv + pos.permute(1, 0, 2), kv, key_padding_mask=pad)[0].permute(1, 0, 2)
        want = ln_post(out) @ ours.proj
        got = ours(x, tgt, key_mask=~pad)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
