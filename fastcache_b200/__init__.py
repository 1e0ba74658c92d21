"""fastcache_b200: KV-cache-compression serving engine for B200 (sm_100a)."""
from .sampling_params import SamplingParams  # noqa: F401
from .config import Config, ModelConfig  # noqa: F401


def __getattr__(name):
    # engine classes import torch-heavy modules; load them on first use
    if name == "LLM":
        from .llm import LLM
        return LLM
    if name in ("LlavaLLM", "LlavaLLMEngine"):
        from .engine import llava_engine
        return getattr(llava_engine, name)
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    raise AttributeError(name)


__all__ = ["LLM", "LlavaLLM", "LLMEngine", "SamplingParams", "Config", "ModelConfig"]
__version__ = "0.1.0"
