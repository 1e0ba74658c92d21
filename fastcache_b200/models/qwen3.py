"""Qwen3 (per-head q/k RMSNorm before rotary; reference: nanovllm/models/qwen3.py:202-235)
and Qwen2 (QKV bias, no q/k norm; the language model of MiniCPM-V-2.6,
nanovllm/models/minicpm.py:33-232)."""
from .decoder import DecoderForCausalLM


class Qwen3ForCausalLM(DecoderForCausalLM):
    qkv_bias = False
    qk_norm = True


class Qwen2ForCausalLM(DecoderForCausalLM):
    qkv_bias = True
    qk_norm = False
