"""Engine configuration.

Parity: the reference keeps a small dataclass of engine knobs
(nanovllm/config.py:5-19) and filters constructor kwargs by attribute name
(nanovllm/engine/llm_engine.py:14-18).  This build keeps those field names so
existing call sites keep working, drops the "block size must be a multiple of
256" restriction (that one came from the flash-attn paging constraint,
nanovllm/config.py:19) and adds the three-queue batching caps and the
compression policy fields that the reference scatters over engine kwargs.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any


@dataclass
class Config:
    model: str = ""
    max_num_batched_tokens: int = 32768
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    enforce_eager: bool = False
    hf_config: Any = None
    eos: int = -1
    kvcache_block_size: int = 256
    num_kvcache_blocks: int = -1
    # --- additions of this build -------------------------------------------------
    tensor_parallel_size: int = 1
    dtype: str = "auto"              # "auto" -> bf16 on cuda, fp32 on cpu
    device: str = "auto"             # "auto" -> cuda when available
    # three-queue batching caps (v1 harness semantics: prefill / compress / decode)
    prefill_batch_size: int = 0      # 0 = bounded only by max_num_seqs / max_num_batched_tokens
    compress_batch_size: int = 0
    decode_batch_size: int = 0
    # compression policy
    compression_mode: str = "none"   # none | eager | async | lazy
    lazy_occupancy_threshold: float = 0.9
    # > 0: a prompt that does not fit the rest of a prefill step's token budget is prefetched in pieces of at
    # least this many rows over several steps (text requests only); 0: a prompt is never split
    chunked_prefill_tokens: int = 0
    # position id of a token decoded after compression:
    #   "compressed": kv length after compression (reference engine behaviour)
    #   "original":   number of tokens the request has really seen
    position_mode: str = "compressed"
    prefix_caching: bool = True
    seed: int = 0
    extra: dict = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.kvcache_block_size <= 0:
            raise ValueError("kvcache_block_size must be positive")
        if self.compression_mode not in ("none", "eager", "async", "lazy"):
            raise ValueError(f"unknown compression_mode {self.compression_mode!r}")
        if self.position_mode not in ("compressed", "original"):
            raise ValueError(f"unknown position_mode {self.position_mode!r}")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")

    @classmethod
    def from_kwargs(cls, model: str = "", **kwargs: Any) -> "Config":
        """Build a config, keeping only the kwargs that name a field."""
        names = {f.name for f in fields(cls)}
        known = {k: v for k, v in kwargs.items() if k in names}
        cfg = cls(model=model, **known)
        cfg.extra = {k: v for k, v in kwargs.items() if k not in names}
        return cfg


class ModelConfig:
    """Attribute bag standing in for a HuggingFace config object.

    The engine only reads attributes, so a model directory's ``config.json``
    (or a plain dict for random-init runs) is enough; ``transformers`` is not
    needed to start the engine.  Nested ``text_config`` / ``vision_config``
    dicts become nested ModelConfig objects.
    """

    def __init__(self, **kw: Any) -> None:
        for k, v in kw.items():
            if isinstance(v, dict) and k.endswith("_config"):
                v = ModelConfig(**v)
            setattr(self, k, v)
        # transformers >= 5 writes the rotary settings as one dict, `rope_parameters` = {rope_theta, rope_type,
        # ...}; the models read the 4.x field names, so give both views of the same facts
        rp = kw.get("rope_parameters")
        if isinstance(rp, dict):
            if "rope_theta" not in kw and rp.get("rope_theta") is not None:
                self.rope_theta = float(rp["rope_theta"])
            if "rope_scaling" not in kw:
                kind = rp.get("rope_type", rp.get("type", "default"))
                self.rope_scaling = None if kind in (None, "default") else dict(rp)

    def get(self, name: str, default: Any = None) -> Any:
        return getattr(self, name, default)

    def to_dict(self) -> dict:
        out = {}
        for k, v in self.__dict__.items():
            out[k] = v.to_dict() if isinstance(v, ModelConfig) else v
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as fh:
            return cls(**json.load(fh))

    def __repr__(self) -> str:
        return f"ModelConfig({self.to_dict()})"


def text_config_of(hf_config: Any) -> Any:
    """Return the language-model part of a (possibly multimodal) config."""
    sub = getattr(hf_config, "text_config", None)
    return sub if sub is not None else hf_config
