"""Multimodal engine entry points under the reference's names
("kv-cache pipeline"/nanovllm/engine/llava_engine.py:28-49, :52, :617-620)."""
from .llm_engine import LLMEngine, PendingCompression  # noqa: F401
from .sequence import Sequence as LlavaSequence  # noqa: F401


class LlavaLLMEngine(LLMEngine):
    pass


class LlavaLLM(LlavaLLMEngine):
    pass
