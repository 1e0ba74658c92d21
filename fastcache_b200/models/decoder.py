"""Pre-norm decoder stack shared by the Llama, Qwen2 and Qwen3 families.

Parity: nanovllm/models/llama.py:25-241 and nanovllm/models/qwen3.py:20-235
(attention with packed QKV, optional per-head q/k RMSNorm before rotary,
SwiGLU MLP, residual stream with fused add+norm, tied embeddings optional).

Layout of one layer here (what "fused norm handoff" means): a layer receives
the *already normalised* input and the residual stream, and returns the
normalised input of the next layer.  The two reductions of a tensor-parallel
layer are therefore each followed directly by "add residual + RMSNorm" inside
one call (`row_linear_reduce_add_norm`), which is the unit the fused
communication kernels implement.  Unlike the reference, every family here
reads the tensor-parallel degree from the process group (the reference
hard-codes 1 in Qwen3, nanovllm/models/qwen3.py:36).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..layers.activation import SiluAndMul
from ..layers.attention import Attention
from ..layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..layers.rotary_embedding import get_rope
from ..parallel.fused import get_fused_comm, row_linear_reduce_add_norm


class DecoderAttention(nn.Module):
    def __init__(self, cfg, layer_idx: int, qkv_bias: bool, qk_norm: bool):
        super().__init__()
        hidden = cfg.hidden_size
        heads = cfg.num_attention_heads
        kv_heads = getattr(cfg, "num_key_value_heads", None) or heads
        head_dim = getattr(cfg, "head_dim", None) or hidden // heads
        self.head_dim = head_dim
        self.eps = getattr(cfg, "rms_norm_eps", 1e-6)
        self.qkv_proj = QKVParallelLinear(hidden, head_dim, heads, kv_heads, bias=qkv_bias)
        self.o_proj = RowParallelLinear(heads * head_dim, hidden, bias=False, reduce_results=False)
        self.num_heads = self.qkv_proj.num_heads
        self.num_kv_heads = self.qkv_proj.num_kv_heads
        self.rotary_emb = get_rope(head_dim, head_dim, getattr(cfg, "max_position_embeddings", 4096),
                                   float(getattr(cfg, "rope_theta", 10000.0)),
                                   getattr(cfg, "rope_scaling", None))
        self.attn = Attention(self.num_heads, head_dim, head_dim ** -0.5, self.num_kv_heads, layer_idx)
        if qk_norm:
            self.q_norm = RMSNorm(head_dim, self.eps)
            self.k_norm = RMSNorm(head_dim, self.eps)
        else:
            self.q_norm = self.k_norm = None

    def forward(self, positions: torch.Tensor, normed: torch.Tensor) -> torch.Tensor:
        """Returns this rank's partial attention output rows (before o_proj)."""
        cs = self.rotary_emb.cos_sin_cache
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        if (normed.is_cuda and normed.shape[0] <= 256 and self.head_dim == 128 and self.qkv_proj.bias is None
                and getattr(get_fused_comm(), "_gather", None) is None):
            # decode sizes: the rope / q-k norm / KV store kernel reduces the GEMM's split-K partial sums
            return self.attn(None, positions, cs, qw, kw, self.eps, fused_qkv=(normed, self.qkv_proj.weight))
        return self.attn(self.qkv_proj(normed), positions, cs, qw, kw, self.eps)


class DecoderMLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(cfg.hidden_size, [cfg.intermediate_size] * 2, bias=False)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, bias=False,
                                           reduce_results=False)
        self.act_fn = SiluAndMul()

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        if (normed.is_cuda and normed.shape[0] <= 256 and self.gate_up_proj.bias is None
                and getattr(get_fused_comm(), "_gather", None) is None):
            # decode sizes: the SwiGLU kernel also reduces the GEMM's split-K partial sums.  (Not while `normed`
            # is the gathered buffer that is still filling over NVLink: `ops.linear` below knows how to wait.)
            return ops.linear_silu_mul(normed, self.gate_up_proj.weight)
        if normed.is_cuda and self.gate_up_proj.bias is None:
            # prefill sizes: SwiGLU runs in the GEMM epilogue (gate and up rows share a tile), also in the
            # tensor-parallel GEMM that consumes the gathered activations
            return ops.linear(normed, self.gate_up_proj.weight, None, act="swiglu")
        return self.act_fn(self.gate_up_proj(normed))


class DecoderLayer(nn.Module):
    def __init__(self, cfg, layer_idx: int, qkv_bias: bool, qk_norm: bool):
        super().__init__()
        eps = getattr(cfg, "rms_norm_eps", 1e-6)
        self.eps = eps
        self.self_attn = DecoderAttention(cfg, layer_idx, qkv_bias, qk_norm)
        self.mlp = DecoderMLP(cfg)
        self.input_layernorm = RMSNorm(cfg.hidden_size, eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, eps)

    def forward(self, positions: torch.Tensor, normed: torch.Tensor, residual: torch.Tensor,
                next_norm_weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        attn = self.self_attn(positions, normed)
        o = self.self_attn.o_proj
        normed, residual = row_linear_reduce_add_norm(attn, o.weight, o.bias, residual,
                                                      self.post_attention_layernorm.weight, self.eps)
        act = self.mlp(normed)
        d = self.mlp.down_proj
        return row_linear_reduce_add_norm(act, d.weight, d.bias, residual, next_norm_weight, self.eps)


class DecoderModel(nn.Module):
    def __init__(self, cfg, qkv_bias: bool, qk_norm: bool):
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(DecoderLayer(cfg, i, qkv_bias, qk_norm)
                                    for i in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, getattr(cfg, "rms_norm_eps", 1e-6))

    def forward(self, input_ids: Optional[torch.Tensor], positions: torch.Tensor,
                inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        residual = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        first = self.layers[0].input_layernorm
        normed = ops.rms_norm(residual, first.weight, first.eps)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].input_layernorm.weight if i + 1 < n else self.norm.weight
            normed, residual = layer(positions, normed, residual, nxt)
        comm = get_fused_comm()
        if comm is not None:
            normed = comm.finish_forward(normed)
        return normed


class DecoderForCausalLM(nn.Module):
    """Base of every text model in this package."""
    packed_modules_mapping = {
        "q_proj": ("qkv_proj", "q"),
        "k_proj": ("qkv_proj", "k"),
        "v_proj": ("qkv_proj", "v"),
        "gate_proj": ("gate_up_proj", 0),
        "up_proj": ("gate_up_proj", 1),
    }
    qkv_bias = False
    qk_norm = False

    def __init__(self, cfg):
        super().__init__()
        self.config = cfg
        self.model = DecoderModel(cfg, self.qkv_bias or bool(getattr(cfg, "attention_bias", False)),
                                  self.qk_norm)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size)
        self.tie = bool(getattr(cfg, "tie_word_embeddings", False))
        if self.tie:
            emb = self.model.embed_tokens
            if emb.replicated:
                # the table is whole on every rank: the head multiplies with this rank's rows of it (a view of
                # the same storage, so loading the table loads the head)
                self.lm_head.weight = nn.Parameter(emb.shard_rows(), requires_grad=False)
                self.optional_weight_substrings = ("lm_head.",)
            else:
                self.lm_head.weight = emb.weight

    def get_input_embeddings(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.model.embed_tokens(input_ids)

    def forward(self, input_ids: Optional[torch.Tensor], positions: torch.Tensor,
                inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.model(input_ids, positions, inputs_embeds)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head(hidden)

    # ----------------------------------------------------------- checkpoints
    @classmethod
    def hf_weight_shapes(cls, cfg) -> Dict[str, Tuple[int, ...]]:
        """Tensor names and full shapes of the HuggingFace checkpoint of this model."""
        h = cfg.hidden_size
        heads = cfg.num_attention_heads
        kvh = getattr(cfg, "num_key_value_heads", None) or heads
        d = getattr(cfg, "head_dim", None) or h // heads
        inter = cfg.intermediate_size
        bias = cls.qkv_bias or bool(getattr(cfg, "attention_bias", False))
        shapes: Dict[str, Tuple[int, ...]] = {"model.embed_tokens.weight": (cfg.vocab_size, h)}
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            shapes[p + "self_attn.q_proj.weight"] = (heads * d, h)
            shapes[p + "self_attn.k_proj.weight"] = (kvh * d, h)
            shapes[p + "self_attn.v_proj.weight"] = (kvh * d, h)
            if bias:
                shapes[p + "self_attn.q_proj.bias"] = (heads * d,)
                shapes[p + "self_attn.k_proj.bias"] = (kvh * d,)
                shapes[p + "self_attn.v_proj.bias"] = (kvh * d,)
            if cls.qk_norm:
                shapes[p + "self_attn.q_norm.weight"] = (d,)
                shapes[p + "self_attn.k_norm.weight"] = (d,)
            shapes[p + "self_attn.o_proj.weight"] = (h, heads * d)
            shapes[p + "mlp.gate_proj.weight"] = (inter, h)
            shapes[p + "mlp.up_proj.weight"] = (inter, h)
            shapes[p + "mlp.down_proj.weight"] = (h, inter)
            shapes[p + "input_layernorm.weight"] = (h,)
            shapes[p + "post_attention_layernorm.weight"] = (h,)
        shapes["model.norm.weight"] = (h,)
        if not getattr(cfg, "tie_word_embeddings", False):
            shapes["lm_head.weight"] = (cfg.vocab_size, h)
        return shapes
