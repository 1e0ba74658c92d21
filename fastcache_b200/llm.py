"""`LLM`: the text engine under the reference's name (nanovllm/llm.py:1-4)."""
from .engine.llm_engine import LLMEngine


class LLM(LLMEngine):
    pass
