"""Llama family (reference: nanovllm/models/llama.py:25-241)."""
from .decoder import DecoderAttention, DecoderForCausalLM, DecoderLayer, DecoderMLP, DecoderModel


class LlamaForCausalLM(DecoderForCausalLM):
    qkv_bias = False
    qk_norm = False


# The parts of the stack under the reference's class names: the shared decoder classes with
# this family's switches (no QKV bias, no q/k norm) filled in.
class LlamaAttention(DecoderAttention):
    def __init__(self, cfg, layer_idx: int = 0):
        super().__init__(cfg, layer_idx, LlamaForCausalLM.qkv_bias, LlamaForCausalLM.qk_norm)


class LlamaMLP(DecoderMLP):
    pass


class LlamaDecoderLayer(DecoderLayer):
    def __init__(self, cfg, layer_idx: int = 0):
        super().__init__(cfg, layer_idx, LlamaForCausalLM.qkv_bias, LlamaForCausalLM.qk_norm)


class LlamaModel(DecoderModel):
    def __init__(self, cfg):
        super().__init__(cfg, LlamaForCausalLM.qkv_bias, LlamaForCausalLM.qk_norm)
