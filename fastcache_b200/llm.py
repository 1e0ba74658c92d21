"""The user-facing engine class.

`LLM(model_dir_or_config, **settings)` is the engine itself (`engine/llm_engine.py`) under the name the
reference exports from its `llm` module (nanovllm/llm.py:1-4); text and multimodal models, every
compression backend and tensor parallelism go through this one class (`LlavaLLM` and `LlavaLLMEngine` are subclasses of it that add nothing).
"""
from __future__ import annotations

from typing import Any, Dict

from .engine import llm_engine as _engine


class LLM(_engine.LLMEngine):
    """See `LLMEngine` for the constructor arguments."""

    @classmethod
    def from_random_init(cls, architecture: Dict[str, Any], **settings: Any) -> "LLM":
        """An engine over seeded random weights of `architecture` (a HuggingFace `config.json` as a dict):
        what the benchmarks and tests use when no checkpoint is at hand."""
        return cls(dict(architecture), **settings)
