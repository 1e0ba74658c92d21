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
