"""Qwen3 (per-head q/k RMSNorm before rotary; reference: nanovllm/models/qwen3.py:20-235)
and Qwen2 (QKV bias, no q/k norm; the language model of MiniCPM-V-2.6,
nanovllm/models/minicpm.py:33-232)."""
from .decoder import DecoderAttention, DecoderForCausalLM, DecoderLayer, DecoderMLP, DecoderModel


class Qwen3ForCausalLM(DecoderForCausalLM):
    qkv_bias = False
    qk_norm = True


class Qwen2ForCausalLM(DecoderForCausalLM):
    qkv_bias = True
    qk_norm = False


def _family(prefix: str, top):
    """The parts of the stack under the reference's class names (`<prefix>Attention`, `MLP`,
    `DecoderLayer`, `Model`): the shared decoder classes with the family's switches filled in."""
    bias, norm = top.qkv_bias, top.qk_norm

    class Attention(DecoderAttention):
        def __init__(self, cfg, layer_idx: int = 0):
            super().__init__(cfg, layer_idx, bias, norm)

    class MLP(DecoderMLP):
        pass

    class Layer(DecoderLayer):
        def __init__(self, cfg, layer_idx: int = 0):
            super().__init__(cfg, layer_idx, bias, norm)

    class Model(DecoderModel):
        def __init__(self, cfg):
            super().__init__(cfg, bias, norm)

    out = []
    for cls, suffix in ((Attention, "Attention"), (MLP, "MLP"), (Layer, "DecoderLayer"), (Model, "Model")):
        cls.__name__ = cls.__qualname__ = prefix + suffix
        out.append(cls)
    return out


Qwen3Attention, Qwen3MLP, Qwen3DecoderLayer, Qwen3Model = _family("Qwen3", Qwen3ForCausalLM)
Qwen2Attention, Qwen2MLP, Qwen2DecoderLayer, Qwen2Model = _family("Qwen2", Qwen2ForCausalLM)
