"""LLaVA-1.5: CLIP ViT-L/14-336 + GELU MLP projector + Llama language model.

Parity: nanovllm/models/llava.py:440-590 (checkpoint prefixes `vision_tower.vision_model.*`,
`multi_modal_projector.linear_{1,2}.*`, `language_model.*`; the single `<image>`
placeholder (id 32000) is replaced by the patch features and later positions shift).
Differences: any number of images per prefill batch; the expansion of the placeholder is
done by the runner when it builds the step metadata, so the rows of the flattened batch
that receive image features arrive here as (row, count) pairs; the language model is
tensor-parallel.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn

from ..config import ModelConfig
from .llama import LlamaAttention, LlamaDecoderLayer, LlamaForCausalLM, LlamaMLP, LlamaModel  # noqa: F401
from .vision import (CLIP_MEAN, CLIP_STD, CLIPVisionTower, LlavaProjector, clip_vision_shapes, resize_normalize,
                     to_chw_float)

DEFAULT_CLIP = dict(hidden_size=1024, intermediate_size=4096, num_hidden_layers=24, num_attention_heads=16,
                    image_size=336, patch_size=14, layer_norm_eps=1e-5)


def _vision_cfg(cfg) -> Any:
    v = getattr(cfg, "vision_config", None)
    d = dict(DEFAULT_CLIP)
    if v is not None:
        d.update({k: getattr(v, k) for k in DEFAULT_CLIP if hasattr(v, k)})
    return ModelConfig(**d)


class LlavaForConditionalGeneration(nn.Module):
    packed_modules_mapping = LlamaForCausalLM.packed_modules_mapping
    # HF checkpoints of LLaVA-1.5 come in two layouts: "language_model.model.*" and "model.language_model.*"
    checkpoint_prefix_map = {"model.language_model.": "language_model.model.", "lm_head.": "language_model.lm_head.",
                             "model.vision_tower.": "vision_tower.", "model.multi_modal_projector.":
                             "multi_modal_projector."}

    def __init__(self, cfg):
        super().__init__()
        self.config = cfg
        self.text_config = cfg.text_config
        self.vision_config = _vision_cfg(cfg)
        self.image_token_id = int(getattr(cfg, "image_token_index", getattr(cfg, "image_token_id", 32000)))
        layer = int(getattr(cfg, "vision_feature_layer", -2))
        self.vision_tower = CLIPVisionTower(self.vision_config, feature_layer=layer,
                                            apply_post_layernorm=bool(getattr(cfg, "vision_post_layernorm", False)))
        self.multi_modal_projector = LlavaProjector(self.vision_config.hidden_size, self.text_config.hidden_size)
        self.language_model = LlamaForCausalLM(self.text_config)
        self.image_token_len = self.vision_tower.num_patches

    # -------------------------------------------------------------- images
    def preprocess_image(self, image: Any, device, dtype, processor: Any = None):
        size = self.vision_config.image_size
        px = resize_normalize(to_chw_float(image), (size, size), CLIP_MEAN, CLIP_STD)
        return px.to(device=device, dtype=dtype), {"rows": self.image_token_len}

    def num_image_rows(self, meta: Any) -> int:
        return self.image_token_len

    def encode_images(self, pixels: torch.Tensor) -> torch.Tensor:
        return self.multi_modal_projector(self.vision_tower(pixels))

    get_image_features = encode_images

    def merge_input_ids_with_image_features(self, input_ids: torch.Tensor, image_features: torch.Tensor,
                                            positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Flat (1-D) token ids with ONE image placeholder -> embeddings and positions with the
        placeholder replaced by the image's rows (nanovllm/models/llava.py:491-551).

        The engine does not call this: its runner expands the placeholder when it builds the step's
        rows, so the features are written into an embedding buffer of the final length.  It is
        kept for callers that drive the model directly."""
        embeds = self.language_model.get_input_embeddings(input_ids)
        if image_features.dim() == 3:
            image_features = image_features[0]
        where = (input_ids == self.image_token_id).nonzero(as_tuple=True)[0]
        if where.numel() == 0:
            return embeds, positions
        i, n = int(where[0]), image_features.shape[0]
        merged = torch.cat([embeds[:i], image_features.to(embeds.dtype), embeds[i + 1:]], 0)
        pos = torch.cat([positions[:i],
                         torch.arange(i, i + n, dtype=positions.dtype, device=positions.device),
                         positions[i + 1:] + (n - 1)])
        return merged, pos

    # -------------------------------------------------------------- forward
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor,
                images: Optional[List[Tuple[torch.Tensor, Any, int, int]]] = None) -> torch.Tensor:
        if not images:
            return self.language_model(input_ids, positions)
        embeds = self.language_model.get_input_embeddings(input_ids)
        feats = self.encode_images(torch.stack([im[0] for im in images]))
        for f, (_, _, row, cnt) in zip(feats, images):
            embeds[row:row + cnt] = f[:cnt].to(embeds.dtype)
        return self.language_model(None, positions, inputs_embeds=embeds)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.language_model.compute_logits(hidden)

    def finalize_weights(self) -> None:
        self.vision_tower.vision_model.embeddings.patch_embedding.finalize()
        for layer in self.vision_tower.vision_model.encoder.layers:
            layer.self_attn.fuse()

    @classmethod
    def hf_weight_shapes(cls, cfg) -> Dict[str, Tuple[int, ...]]:
        s = clip_vision_shapes(_vision_cfg(cfg), "vision_tower.vision_model.")
        v, t = _vision_cfg(cfg).hidden_size, cfg.text_config.hidden_size
        s.update({"multi_modal_projector.linear_1.weight": (t, v), "multi_modal_projector.linear_1.bias": (t,),
                  "multi_modal_projector.linear_2.weight": (t, t), "multi_modal_projector.linear_2.bias": (t,)})
        for k, shp in LlamaForCausalLM.hf_weight_shapes(cfg.text_config).items():
            s["language_model." + k] = shp
        return s


# ------------------------------------------------------------ reference names
# Classes of the reference's module (nanovllm/models/llava.py:28-199) -> the vision classes here.
from . import vision as _v  # noqa: E402

CLIPVisionEmbeddings = _v._CLIPEmbeddings
CLIPAttention = _v.VisionAttention
CLIPMLP = _v.VisionMLP
CLIPEncoderLayer = _v.VisionLayer
CLIPEncoder = _v._Encoder
CLIPVisionTransformer = _v._CLIPVisionModel
CLIPVisionModel = CLIPVisionTower
LlavaMultiModalProjector = LlavaProjector


class LlavaConfig:
    """Flat view of a LLaVA HuggingFace config (nanovllm/models/llava.py:410-437)."""

    def __init__(self, hf_config):
        text, vis = hf_config.text_config, _vision_cfg(hf_config)
        self.text_config, self.vision_config = text, vis
        self.vocab_size = text.vocab_size
        self.hidden_size = text.hidden_size
        self.num_hidden_layers = text.num_hidden_layers
        self.num_attention_heads = text.num_attention_heads
        self.num_key_value_heads = getattr(text, "num_key_value_heads", None) or text.num_attention_heads
        self.intermediate_size = text.intermediate_size
        self.rms_norm_eps = getattr(text, "rms_norm_eps", 1e-6)
        self.max_position_embeddings = getattr(text, "max_position_embeddings", 4096)
        self.rope_theta = getattr(text, "rope_theta", 10000.0)
        self.head_dim = getattr(text, "head_dim", None) or self.hidden_size // self.num_attention_heads
        self.vision_hidden_size = vis.hidden_size
        self.image_size, self.patch_size = vis.image_size, vis.patch_size
        self.num_channels = getattr(vis, "num_channels", 3)
        self.image_token_len = (self.image_size // self.patch_size) ** 2


def get_llava_weight_mapping() -> Dict[str, str]:
    """Checkpoint prefix -> module prefix for both HuggingFace layouts of LLaVA-1.5.  (The reference
    returns a partial identity table, nanovllm/models/llava.py:595-611; the loader here works from
    prefixes and `packed_modules_mapping`.)"""
    return dict(LlavaForConditionalGeneration.checkpoint_prefix_map)
