"""MiniCPM-V-2.6: SigLIP-style vision tower + perceiver resampler + Qwen2 language model.

Parity: nanovllm/models/minicpm.py:276-468 (checkpoint prefixes `llm.*`, `vpm.*`, `resampler.*`;
64 query tokens per slice; slices of 448 x 448 with 14-px patches).  The reference takes `vpm` and
`resampler` from the HuggingFace remote code; here both are native modules that load the same
tensor names.  An image is cut into a grid of slices plus a thumbnail (`slice_image`, at most
`max_slice_nums` slices); every slice yields 64 rows, and the rows of all slices of one image
replace the image placeholder of the prompt in order (thumbnail first).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn

from ..config import ModelConfig
from .qwen3 import Qwen2Attention, Qwen2DecoderLayer, Qwen2ForCausalLM, Qwen2MLP, Qwen2Model  # noqa: F401
from .vision import (SIGLIP_MEAN, SIGLIP_STD, Resampler, SiglipVisionTower, resampler_shapes, resize_normalize,
                     siglip_vision_shapes, to_chw_float)

DEFAULT_SIGLIP = dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16,
                      image_size=980, patch_size=14, layer_norm_eps=1e-6)


def _vision_cfg(cfg) -> Any:
    v = getattr(cfg, "vision_config", None)
    d = dict(DEFAULT_SIGLIP)
    if v is not None:
        d.update({k: getattr(v, k) for k in DEFAULT_SIGLIP if hasattr(v, k)})
    return ModelConfig(**d)


def _llm_cfg(cfg) -> Any:
    for name in ("text_config", "llm_config"):
        sub = getattr(cfg, name, None)
        if sub is not None:
            return sub
    return cfg                     # MiniCPM-V configs carry the Qwen2 fields at top level


def best_grid(width: int, height: int, max_slices: int, scale: int) -> Optional[Tuple[int, int]]:
    """Grid (cols, rows) whose aspect ratio is closest to the image's, or None when one slice is enough."""
    ratio = width * height / (scale * scale)
    n = math.ceil(ratio)
    if n <= 1 or max_slices <= 1:
        return None
    cands = [k for k in (n - 1, n, n + 1) if 1 < k <= max_slices] or [min(max_slices, max(2, n))]
    best, err = None, float("inf")
    log_r = math.log(width / height)
    for k in cands:
        for c in range(1, k + 1):
            if k % c:
                continue
            e = abs(log_r - math.log(c / (k // c)))
            if e < err:
                best, err = (c, k // c), e
    return best


def slice_image(chw: torch.Tensor, max_slices: int = 9, scale: int = 448, patch: int = 14
                ) -> List[torch.Tensor]:
    """Thumbnail first, then the grid slices row by row; each returned tensor is CHW float in [0, 1]
    whose sides are multiples of `patch` and whose area is about scale x scale."""
    _, H, W = chw.shape

    def fit(w: int, h: int) -> Tuple[int, int]:
        r = w / h
        hh = max(patch, int(round(scale / math.sqrt(r) / patch)) * patch)
        ww = max(patch, int(round(scale * math.sqrt(r) / patch)) * patch)
        return ww, hh

    def resize(x: torch.Tensor, w: int, h: int) -> torch.Tensor:
        return torch.nn.functional.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False,
                                               antialias=True)[0].clamp(0, 1)

    tw, th = fit(W, H)
    out = [resize(chw, tw, th)]
    grid = best_grid(W, H, max_slices, scale)
    if grid is not None:
        cols, rows = grid
        sw, sh = fit(W / cols, H / rows)
        big = resize(chw, sw * cols, sh * rows)
        for r in range(rows):
            for c in range(cols):
                out.append(big[:, r * sh:(r + 1) * sh, c * sw:(c + 1) * sw])
    return out


class MiniCPMForConditionalGeneration(nn.Module):
    packed_modules_mapping = Qwen2ForCausalLM.packed_modules_mapping

    def __init__(self, cfg):
        super().__init__()
        self.config = cfg
        self.text_config = _llm_cfg(cfg)
        if getattr(cfg, "text_config", None) is None:
            cfg.text_config = self.text_config
        self.vision_config = _vision_cfg(cfg)
        self.query_num = int(getattr(cfg, "query_num", 64))
        self.max_slice_nums = int(getattr(cfg, "max_slice_nums", 9))
        self.scale_resolution = int(getattr(cfg, "scale_resolution", 448))
        self.image_token_id = int(getattr(cfg, "image_token_id", getattr(self.text_config, "unk_token_id", 128244)
                                          or 128244))
        self.llm = Qwen2ForCausalLM(self.text_config)
        self.vpm = SiglipVisionTower(self.vision_config)
        side = self.vision_config.image_size // self.vision_config.patch_size
        self.resampler = Resampler(self.query_num, self.text_config.hidden_size, self.vision_config.hidden_size,
                                   max_size=(side, side))
        self.image_token_len = self.query_num        # rows per slice; an image gives rows_per_image(meta)

    # -------------------------------------------------------------- images
    def preprocess_image(self, image: Any, device, dtype, processor: Any = None):
        p = self.vision_config.patch_size
        slices = slice_image(to_chw_float(image), self.max_slice_nums, self.scale_resolution, p)
        sizes = [(s.shape[1] // p, s.shape[2] // p) for s in slices]
        Hm, Wm = max(s.shape[1] for s in slices), max(s.shape[2] for s in slices)
        batch = torch.zeros(len(slices), 3, Hm, Wm)
        for i, s in enumerate(slices):
            m = torch.tensor(SIGLIP_MEAN)[:, None, None]
            d = torch.tensor(SIGLIP_STD)[:, None, None]
            batch[i, :, : s.shape[1], : s.shape[2]] = (s - m) / d
        meta = {"tgt_sizes": torch.tensor(sizes, dtype=torch.long), "rows": len(slices) * self.query_num,
                "padded": (Hm, Wm)}
        return batch.to(device=device, dtype=dtype), meta

    def num_image_rows(self, meta: Any) -> int:
        return int(meta["rows"])

    def encode_images(self, pixels: torch.Tensor, meta: Any) -> torch.Tensor:
        """[slices, 3, H, W] -> [slices * query_num, hidden]"""
        p = self.vision_config.patch_size
        tgt = meta["tgt_sizes"]
        Hm, Wm = pixels.shape[2] // p, pixels.shape[3] // p
        # keep only the real patches of each slice, packed at the front (ragged grids inside a padded batch)
        feats, mask = self._tower(pixels, tgt, Hm, Wm)
        key_mask = None if bool(mask.all()) else mask
        out = self.resampler(feats, tgt, key_mask)
        return out.reshape(-1, out.shape[-1])

    def _tower(self, pixels, tgt, Hm, Wm):
        B = pixels.shape[0]
        same = bool((tgt[:, 0] == Hm).all() and (tgt[:, 1] == Wm).all())
        if same:
            return self.vpm(pixels, tgt)
        # ragged: run each distinct grid size as its own batch, then pad to the longest
        dim = self.vision_config.hidden_size
        L = int((tgt[:, 0] * tgt[:, 1]).max())
        feats = torch.zeros(B, L, dim, dtype=pixels.dtype, device=pixels.device)
        mask = torch.zeros(B, L, dtype=torch.bool, device=pixels.device)
        p = self.vision_config.patch_size
        for (h, w) in sorted(set(map(tuple, tgt.tolist()))):
            idx = [i for i, s in enumerate(tgt.tolist()) if tuple(s) == (h, w)]
            f, _ = self.vpm(pixels[idx][:, :, : h * p, : w * p].contiguous(), tgt[idx])
            feats[idx, : h * w] = f
            mask[idx, : h * w] = True
        return feats, mask

    def load_vision_modules(self, hf_model: Any) -> None:
        """Copy the vision tower and resampler weights out of a loaded HuggingFace MiniCPM-V model.
        The reference adopts the HF modules themselves (nanovllm/models/minicpm.py:329-340); here the
        native modules keep running and only take the tensors, so the sm_100a kernels stay in use."""
        for name in ("vpm", "resampler"):
            src = getattr(hf_model, name).state_dict()
            dst = getattr(self, name)
            own = dst.state_dict()
            take = {k: v.to(own[k].dtype).reshape(own[k].shape) for k, v in src.items()
                    if k in own and v.numel() == own[k].numel()}
            dst.load_state_dict(take, strict=False)
        self.finalize_weights()

    def get_vllm_embedding(self, data: Dict[str, Any]) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        """Batched entry of the HuggingFace-style harness (nanovllm/models/minicpm.py:342-432).

        `data`: `input_ids` [B, T]; `pixel_values`: per sample a list of [3, H, W] slices;
        `tgt_sizes`: per sample a [slices, 2] tensor of patch grids; `image_bound`: per sample a
        [n, 2] tensor of [start, end) spans of placeholder tokens.  Returns the input embeddings
        with each span overwritten by that slice's `query_num` rows, and the per-sample vision
        features.  The reference borrows the vision modules from the HF remote-code model; these
        are the native tower and resampler."""
        ids = data["input_ids"]
        if ids.dim() == 1:
            ids = ids[None]
        embeds = self.llm.get_input_embeddings(ids.reshape(-1)).reshape(*ids.shape, -1).clone()
        p = self.vision_config.patch_size
        bounds = data.get("image_bound") or [None] * ids.shape[0]
        vision: List[torch.Tensor] = []
        for b, slices in enumerate(data.get("pixel_values") or []):
            if slices is None or len(slices) == 0:
                vision.append(embeds.new_zeros(0, embeds.shape[-1]))
                continue
            tgt = torch.as_tensor(data["tgt_sizes"][b], dtype=torch.long).reshape(-1, 2)
            Hm, Wm = int(tgt[:, 0].max()) * p, int(tgt[:, 1].max()) * p
            batch = embeds.new_zeros(len(slices), 3, Hm, Wm)
            for i, sl in enumerate(slices):
                h, w = int(tgt[i, 0]) * p, int(tgt[i, 1]) * p
                batch[i, :, :h, :w] = sl.reshape(3, h, w).to(batch.dtype)
            feats = self.encode_images(batch, {"tgt_sizes": tgt.to(embeds.device)})
            feats = feats.reshape(len(slices), self.query_num, -1)
            vision.append(feats)
            span = bounds[b]
            if span is None:
                continue
            for i, (lo, hi) in enumerate(torch.as_tensor(span).reshape(-1, 2).tolist()):
                if i < feats.shape[0]:
                    embeds[b, lo:hi] = feats[i, : hi - lo].to(embeds.dtype)
        return embeds, vision

    # -------------------------------------------------------------- forward
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor,
                images: Optional[List[Tuple[torch.Tensor, Any, int, int]]] = None) -> torch.Tensor:
        if not images:
            return self.llm(input_ids, positions)
        embeds = self.llm.get_input_embeddings(input_ids)
        for pixels, meta, row, cnt in images:
            f = self.encode_images(pixels, meta)
            embeds[row:row + cnt] = f[:cnt].to(embeds.dtype)
        return self.llm(None, positions, inputs_embeds=embeds)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.llm.compute_logits(hidden)

    def finalize_weights(self) -> None:
        self.vpm.embeddings.patch_embedding.finalize()
        for layer in self.vpm.encoder.layers:
            layer.self_attn.fuse()

    @classmethod
    def hf_weight_shapes(cls, cfg) -> Dict[str, Tuple[int, ...]]:
        v, t = _vision_cfg(cfg), _llm_cfg(cfg)
        s = siglip_vision_shapes(v, "vpm.")
        s.update(resampler_shapes(t.hidden_size, v.hidden_size, int(getattr(cfg, "query_num", 64)), "resampler."))
        for k, shp in Qwen2ForCausalLM.hf_weight_shapes(t).items():
            s["llm." + k] = shp
        return s


class MiniCPMConfig:
    """Flat view of a MiniCPM-V HuggingFace config (nanovllm/models/minicpm.py:237-271)."""

    def __init__(self, hf_config):
        text = _llm_cfg(hf_config)
        self.vocab_size = text.vocab_size
        self.hidden_size = text.hidden_size
        self.num_hidden_layers = text.num_hidden_layers
        self.num_attention_heads = text.num_attention_heads
        self.num_key_value_heads = getattr(text, "num_key_value_heads", None) or text.num_attention_heads
        self.intermediate_size = text.intermediate_size
        self.rms_norm_eps = getattr(text, "rms_norm_eps", 1e-6)
        self.max_position_embeddings = getattr(text, "max_position_embeddings", 32768)
        self.rope_theta = getattr(text, "rope_theta", 1000000.0)
        self.head_dim = getattr(text, "head_dim", None) or self.hidden_size // self.num_attention_heads
        self.hidden_act = getattr(text, "hidden_act", "silu")
        self.vision_config = _vision_cfg(hf_config)
        self.vision_hidden_size = self.vision_config.hidden_size
        self.image_size = getattr(self.vision_config, "image_size", 980)
        self.patch_size = getattr(self.vision_config, "patch_size", 14)
        self.query_num = int(getattr(hf_config, "query_num", 64))
        self.image_token_len = self.query_num


def get_minicpm_weight_mapping() -> Dict[str, str]:
    """Checkpoint prefix -> module of this model: `llm.*` native language model, `vpm.*` SigLIP tower,
    `resampler.*` perceiver resampler (nanovllm/models/minicpm.py:280-303, :473-483)."""
    return {"llm.": "llm.", "vpm.": "vpm.", "resampler.": "resampler."}
