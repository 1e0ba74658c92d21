"""Vision towers and connectors written against this package's ops.

  * CLIPVisionTower — ViT-L/14 at 336 px as used by LLaVA-1.5 (reference:
    nanovllm/models/llava.py:28-181).  Patch embedding is an im2col + GEMM, attention never
    materialises the score matrix, the MLP activation (quick-GELU) is fused into the fc1 GEMM
    epilogue.  By default the features are the hidden states of layer -2 without the final
    LayerNorm and without the class token, as HuggingFace LLaVA-1.5 selects them; the
    reference runs all layers and applies the final LayerNorm, selectable with
    `feature_layer=-1, apply_post_layernorm=True`.
  * LlavaProjector — Linear, GELU, Linear (reference: nanovllm/models/llava.py:186-199).
  * SiglipVisionTower — SigLIP-400M style tower of MiniCPM-V-2.6 (27 layers, hidden 1152, 16 heads
    of 72, bucketed 2-D position table, key-padding mask for ragged slices).
  * Resampler — perceiver resampler: 64 learned queries cross-attend to the patch features of a
    slice with 2-D sin-cos position embeddings on the keys.  The reference borrows both MiniCPM
    modules from the HuggingFace remote code at load time (nanovllm/models/minicpm.py:329-340);
    here they are native and load the same checkpoint names.
The towers are replicated on every tensor-parallel rank, like the reference's.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import numpy as np
import torch
from torch import nn

from .. import ops

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)
SIGLIP_MEAN = (0.5, 0.5, 0.5)
SIGLIP_STD = (0.5, 0.5, 0.5)


def _param(*shape) -> nn.Parameter:
    return nn.Parameter(torch.zeros(*shape), requires_grad=False)


class VLinear(nn.Module):
    """Replicated linear with bias whose activation runs in the GEMM epilogue."""

    def __init__(self, in_f: int, out_f: int, bias: bool = True):
        super().__init__()
        self.weight = _param(out_f, in_f)
        self.bias = _param(out_f) if bias else None

    def forward(self, x: torch.Tensor, act: str = "none") -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, act)


class VLayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight, self.bias, self.eps = _param(dim), _param(dim), eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class VisionAttention(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads, self.head_dim = heads, dim // heads
        self.q_proj, self.k_proj, self.v_proj = VLinear(dim, dim), VLinear(dim, dim), VLinear(dim, dim)
        self.out_proj = VLinear(dim, dim)
        self._qkv_w: Optional[torch.Tensor] = None
        self._qkv_b: Optional[torch.Tensor] = None

    def fuse(self) -> None:
        """One GEMM for q, k and v (called after the weights are loaded)."""
        self._qkv_w = torch.cat([self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], dim=0).contiguous()
        self._qkv_b = torch.cat([self.q_proj.bias, self.k_proj.bias, self.v_proj.bias], dim=0).contiguous()

    def forward(self, x: torch.Tensor, key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, C = x.shape
        if self._qkv_w is None:
            self.fuse()
        qkv = ops.linear(x.reshape(B * S, C), self._qkv_w, self._qkv_b).view(B, S, 3, self.heads, self.head_dim)
        o = ops.dense_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], self.head_dim ** -0.5, key_mask)
        return self.out_proj(o.reshape(B * S, C)).view(B, S, C)


class VisionMLP(nn.Module):
    def __init__(self, dim: int, inter: int, act: str):
        super().__init__()
        self.fc1, self.fc2, self.act = VLinear(dim, inter), VLinear(inter, dim), act

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(self.fc1(x, self.act))


class VisionLayer(nn.Module):
    def __init__(self, dim: int, heads: int, inter: int, act: str, eps: float):
        super().__init__()
        self.layer_norm1, self.layer_norm2 = VLayerNorm(dim, eps), VLayerNorm(dim, eps)
        self.self_attn = VisionAttention(dim, heads)
        self.mlp = VisionMLP(dim, inter, act)

    def forward(self, x: torch.Tensor, key_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, C = x.shape
        x = x + self.self_attn(self.layer_norm1(x), key_mask)
        return x + self.mlp(self.layer_norm2(x).reshape(B * S, C)).view(B, S, C)


class _Encoder(nn.Module):
    def __init__(self, n: int, dim: int, heads: int, inter: int, act: str, eps: float):
        super().__init__()
        self.layers = nn.ModuleList(VisionLayer(dim, heads, inter, act, eps) for _ in range(n))


def _im2col(pixels: torch.Tensor, patch: int, pad_to: int) -> torch.Tensor:
    """[B, 3, H, W] -> [B, (H/p)*(W/p), pad_to] with the (c, ky, kx) order of a Conv2d weight."""
    B, C, H, W = pixels.shape
    x = pixels.unfold(2, patch, patch).unfold(3, patch, patch)            # [B, C, H/p, W/p, p, p]
    x = x.permute(0, 2, 3, 1, 4, 5).reshape(B, (H // patch) * (W // patch), C * patch * patch)
    if pad_to > x.shape[-1]:
        x = torch.nn.functional.pad(x, (0, pad_to - x.shape[-1]))
    return x.contiguous()


class _PatchEmbed(nn.Module):
    """Conv2d(3, dim, patch, stride=patch) as a GEMM; K is padded to a multiple of 8 for TMA."""

    def __init__(self, dim: int, patch: int, bias: bool):
        super().__init__()
        self.patch = patch
        self.k = 3 * patch * patch
        self.k_pad = -(-self.k // 8) * 8
        self.weight = _param(dim, 3, patch, patch)
        self.bias = _param(dim) if bias else None
        self._w2d: Optional[torch.Tensor] = None

    def finalize(self) -> None:
        w = self.weight.reshape(self.weight.shape[0], self.k)
        self._w2d = torch.nn.functional.pad(w, (0, self.k_pad - self.k)).contiguous()

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        if self._w2d is None:
            self.finalize()
        cols = _im2col(pixels.to(self.weight.dtype), self.patch, self.k_pad)
        B, N, K = cols.shape
        return ops.linear(cols.reshape(B * N, K), self._w2d, self.bias).view(B, N, -1)


# ------------------------------------------------------------------------- CLIP
class _CLIPEmbeddings(nn.Module):
    def __init__(self, dim: int, patch: int, image_size: int):
        super().__init__()
        self.class_embedding = _param(dim)
        self.patch_embedding = _PatchEmbed(dim, patch, bias=False)
        self.position_embedding = nn.Embedding(1 + (image_size // patch) ** 2, dim)
        self.position_embedding.weight.requires_grad_(False)


class _CLIPVisionModel(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        dim, eps = cfg.hidden_size, getattr(cfg, "layer_norm_eps", 1e-5)
        self.embeddings = _CLIPEmbeddings(dim, cfg.patch_size, cfg.image_size)
        self.pre_layrnorm = VLayerNorm(dim, eps)          # (sic) the checkpoint's spelling
        self.encoder = _Encoder(cfg.num_hidden_layers, dim, cfg.num_attention_heads, cfg.intermediate_size,
                                "quick_gelu", eps)
        self.post_layernorm = VLayerNorm(dim, eps)


class CLIPVisionTower(nn.Module):
    def __init__(self, cfg, feature_layer: int = -2, apply_post_layernorm: bool = False):
        super().__init__()
        self.cfg = cfg
        self.vision_model = _CLIPVisionModel(cfg)
        n = cfg.num_hidden_layers
        self.num_layers_run = n + 1 + feature_layer if feature_layer < 0 else feature_layer
        self.apply_post_layernorm = apply_post_layernorm
        self.num_patches = (cfg.image_size // cfg.patch_size) ** 2

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """[B, 3, S, S] -> patch features [B, num_patches, hidden] (class token dropped)."""
        vm = self.vision_model
        x = vm.embeddings.patch_embedding(pixels)
        B = x.shape[0]
        cls = vm.embeddings.class_embedding.to(x.dtype).expand(B, 1, -1)
        x = torch.cat([cls, x], dim=1) + vm.embeddings.position_embedding.weight.to(x.dtype)[None]
        x = vm.pre_layrnorm(x)
        for layer in vm.encoder.layers[: self.num_layers_run]:
            x = layer(x)
        if self.apply_post_layernorm:
            x = vm.post_layernorm(x)
        return x[:, 1:]


class LlavaProjector(nn.Module):
    def __init__(self, vision_dim: int, text_dim: int):
        super().__init__()
        self.linear_1, self.linear_2 = VLinear(vision_dim, text_dim), VLinear(text_dim, text_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, N, C = x.shape
        return self.linear_2(self.linear_1(x.reshape(B * N, C), "gelu")).view(B, N, -1)


def clip_vision_shapes(cfg, prefix: str) -> Dict[str, Tuple[int, ...]]:
    d, i, p = cfg.hidden_size, cfg.intermediate_size, cfg.patch_size
    n_pos = 1 + (cfg.image_size // p) ** 2
    s = {prefix + "embeddings.class_embedding": (d,), prefix + "embeddings.patch_embedding.weight": (d, 3, p, p),
         prefix + "embeddings.position_embedding.weight": (n_pos, d),
         prefix + "pre_layrnorm.weight": (d,), prefix + "pre_layrnorm.bias": (d,),
         prefix + "post_layernorm.weight": (d,), prefix + "post_layernorm.bias": (d,)}
    s.update(_encoder_shapes(prefix + "encoder.layers.", cfg.num_hidden_layers, d, i))
    return s


def _encoder_shapes(prefix: str, n: int, d: int, i: int) -> Dict[str, Tuple[int, ...]]:
    s: Dict[str, Tuple[int, ...]] = {}
    for l in range(n):
        p = f"{prefix}{l}."
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            s[p + f"self_attn.{proj}.weight"] = (d, d)
            s[p + f"self_attn.{proj}.bias"] = (d,)
        for ln in ("layer_norm1", "layer_norm2"):
            s[p + ln + ".weight"] = (d,)
            s[p + ln + ".bias"] = (d,)
        s[p + "mlp.fc1.weight"], s[p + "mlp.fc1.bias"] = (i, d), (i,)
        s[p + "mlp.fc2.weight"], s[p + "mlp.fc2.bias"] = (d, i), (d,)
    return s


# ----------------------------------------------------------------------- SigLIP
class _SiglipEmbeddings(nn.Module):
    def __init__(self, dim: int, patch: int, image_size: int):
        super().__init__()
        self.patch_embedding = _PatchEmbed(dim, patch, bias=True)
        self.num_patches_per_side = image_size // patch
        self.position_embedding = nn.Embedding(self.num_patches_per_side ** 2, dim)
        self.position_embedding.weight.requires_grad_(False)

    def position_ids(self, tgt_sizes: torch.Tensor, max_patches: int) -> torch.Tensor:
        """Bucketed 2-D positions for ragged patch grids (NaViT-style): a grid of h x w patches is
        mapped onto the side x side table by fractional coordinates."""
        side = self.num_patches_per_side
        ids = torch.zeros(tgt_sizes.shape[0], max_patches, dtype=torch.long)
        bounds = torch.arange(1 / side, 1.0, 1 / side)
        for b, (h, w) in enumerate(tgt_sizes.tolist()):
            fh = torch.arange(0, 1 - 1e-6, 1 / h)
            fw = torch.arange(0, 1 - 1e-6, 1 / w)
            bh = torch.bucketize(fh, bounds, right=True)
            bw = torch.bucketize(fw, bounds, right=True)
            ids[b, : h * w] = (bh[:, None] * side + bw[None, :]).flatten()
        return ids


class SiglipVisionTower(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        dim, eps = cfg.hidden_size, getattr(cfg, "layer_norm_eps", 1e-6)
        self.embeddings = _SiglipEmbeddings(dim, cfg.patch_size, cfg.image_size)
        self.encoder = _Encoder(cfg.num_hidden_layers, dim, cfg.num_attention_heads, cfg.intermediate_size,
                                "gelu_tanh", eps)
        self.post_layernorm = VLayerNorm(dim, eps)

    def forward(self, pixels: torch.Tensor, tgt_sizes: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """pixels [B, 3, H, W] (slices padded to a common size), tgt_sizes [B, 2] patch grids.
        Returns (features [B, max_patches, dim], key mask [B, max_patches])."""
        x = self.embeddings.patch_embedding(pixels)
        B, N, _ = x.shape
        counts = (tgt_sizes[:, 0] * tgt_sizes[:, 1]).to(x.device)
        mask = torch.arange(N, device=x.device)[None, :] < counts[:, None]
        pos = self.embeddings.position_ids(tgt_sizes.cpu(), N).to(x.device)
        x = x + self.embeddings.position_embedding.weight.to(x.dtype)[pos]
        key_mask = None if bool(mask.all()) else mask
        for layer in self.encoder.layers:
            x = layer(x, key_mask)
        return self.post_layernorm(x), mask


def siglip_vision_shapes(cfg, prefix: str) -> Dict[str, Tuple[int, ...]]:
    d, i, p = cfg.hidden_size, cfg.intermediate_size, cfg.patch_size
    s = {prefix + "embeddings.patch_embedding.weight": (d, 3, p, p), prefix + "embeddings.patch_embedding.bias": (d,),
         prefix + "embeddings.position_embedding.weight": ((cfg.image_size // p) ** 2, d),
         prefix + "post_layernorm.weight": (d,), prefix + "post_layernorm.bias": (d,)}
    s.update(_encoder_shapes(prefix + "encoder.layers.", cfg.num_hidden_layers, d, i))
    return s


# -------------------------------------------------------------------- resampler
def sincos_2d(dim: int, h: int, w: int) -> torch.Tensor:
    """[h, w, dim] fixed 2-D sin-cos table (half of the channels for each axis)."""
    def axis(n: int, d: int) -> torch.Tensor:
        omega = 1.0 / (10000 ** (torch.arange(d // 2, dtype=torch.float32) / (d / 2)))
        out = torch.outer(torch.arange(n, dtype=torch.float32), omega)
        return torch.cat([out.sin(), out.cos()], dim=1)
    eh, ew = axis(h, dim // 2), axis(w, dim // 2)
    return torch.cat([ew[None, :, :].expand(h, -1, -1), eh[:, None, :].expand(-1, w, -1)], dim=-1)


class _MHA(nn.Module):
    """Parameter container with nn.MultiheadAttention's names."""

    def __init__(self, dim: int):
        super().__init__()
        self.in_proj_weight, self.in_proj_bias = _param(3 * dim, dim), _param(3 * dim)
        self.out_proj = VLinear(dim, dim)


class Resampler(nn.Module):
    def __init__(self, num_queries: int, embed_dim: int, kv_dim: int, num_heads: Optional[int] = None,
                 max_size: Tuple[int, int] = (70, 70), eps: float = 1e-6):
        super().__init__()
        self.num_queries, self.embed_dim = num_queries, embed_dim
        self.num_heads = num_heads or embed_dim // 128
        self.query = _param(num_queries, embed_dim)
        self.kv_proj = VLinear(kv_dim, embed_dim, bias=False)
        self.attn = _MHA(embed_dim)
        self.ln_q, self.ln_kv, self.ln_post = (VLayerNorm(embed_dim, eps) for _ in range(3))
        self.proj = _param(embed_dim, embed_dim)
        self.max_size = max_size
        self._pos: Optional[torch.Tensor] = None
        self._proj_t: Optional[torch.Tensor] = None

    def _pos_table(self, device, dtype) -> torch.Tensor:
        if self._pos is None or self._pos.device != device:
            self._pos = sincos_2d(self.embed_dim, *self.max_size).to(device=device, dtype=dtype)
        return self._pos

    def forward(self, x: torch.Tensor, tgt_sizes: torch.Tensor, key_mask: Optional[torch.Tensor] = None
                ) -> torch.Tensor:
        """x [B, L, kv_dim] patch features -> [B, num_queries, embed_dim]."""
        B, L, _ = x.shape
        E, H = self.embed_dim, self.num_heads
        kv = self.ln_kv(self.kv_proj(x.reshape(B * L, -1)).view(B, L, E))
        table = self._pos_table(x.device, kv.dtype)
        pos = torch.zeros(B, L, E, dtype=kv.dtype, device=x.device)
        for b, (h, w) in enumerate(tgt_sizes.tolist()):
            pos[b, : h * w] = table[:h, :w].reshape(h * w, E)
        q = self.ln_q(self.query.to(kv.dtype)[None]).expand(B, -1, -1)
        w, bias = self.attn.in_proj_weight, self.attn.in_proj_bias
        Nq = self.num_queries
        qp = ops.linear(q.reshape(B * Nq, E).contiguous(), w[:E], bias[:E]).view(B, Nq, H, E // H)
        kp = ops.linear((kv + pos).reshape(B * L, E), w[E:2 * E], bias[E:2 * E]).view(B, L, H, E // H)
        vp = ops.linear(kv.reshape(B * L, E), w[2 * E:], bias[2 * E:]).view(B, L, H, E // H)
        o = ops.dense_attention(qp, kp, vp, (E // H) ** -0.5, key_mask)
        o = self.ln_post(self.attn.out_proj(o.reshape(B * Nq, E)).view(B, Nq, E))
        if self._proj_t is None:
            self._proj_t = self.proj.t().contiguous()
        return ops.linear(o.reshape(B * Nq, E), self._proj_t).view(B, Nq, E)


def resampler_shapes(embed_dim: int, kv_dim: int, num_queries: int, prefix: str) -> Dict[str, Tuple[int, ...]]:
    e = embed_dim
    s = {prefix + "query": (num_queries, e), prefix + "kv_proj.weight": (e, kv_dim),
         prefix + "attn.in_proj_weight": (3 * e, e), prefix + "attn.in_proj_bias": (3 * e,),
         prefix + "attn.out_proj.weight": (e, e), prefix + "attn.out_proj.bias": (e,), prefix + "proj": (e, e)}
    for ln in ("ln_q", "ln_kv", "ln_post"):
        s[prefix + ln + ".weight"] = (e,)
        s[prefix + ln + ".bias"] = (e,)
    return s


# ---------------------------------------------------------------- preprocessing
def to_chw_float(image: Any) -> torch.Tensor:
    """PIL image / HWC uint8 array / CHW float tensor in [0, 1] -> CHW float32 in [0, 1]."""
    if isinstance(image, torch.Tensor):
        t = image.float()
        if t.dim() == 3 and t.shape[0] not in (1, 3) and t.shape[-1] in (1, 3):
            t = t.permute(2, 0, 1)
        return t / 255.0 if t.max() > 1.5 else t
    arr = np.asarray(image.convert("RGB") if hasattr(image, "convert") else image)
    t = torch.from_numpy(np.ascontiguousarray(arr)).float()
    if t.dim() == 2:
        t = t[:, :, None].expand(-1, -1, 3)
    t = t.permute(2, 0, 1)
    return t / 255.0 if arr.dtype == np.uint8 or t.max() > 1.5 else t


def resize_normalize(chw: torch.Tensor, size: Tuple[int, int], mean, std) -> torch.Tensor:
    x = torch.nn.functional.interpolate(chw[None], size=size, mode="bicubic", align_corners=False,
                                        antialias=True)[0].clamp(0, 1)
    m = torch.tensor(mean)[:, None, None]
    s = torch.tensor(std)[:, None, None]
    return (x - m) / s
