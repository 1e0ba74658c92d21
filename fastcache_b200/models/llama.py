"""Llama family (reference: nanovllm/models/llama.py:211-241)."""
from .decoder import DecoderForCausalLM


class LlamaForCausalLM(DecoderForCausalLM):
    qkv_bias = False
    qk_norm = False
