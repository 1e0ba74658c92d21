"""Model-type detection and construction.

Parity: "kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:374-398
(minicpm / llava / llama / qwen3 detection from the HuggingFace config).
"""
from __future__ import annotations

from typing import Any, Callable, Dict


def detect_model_type(hf_config: Any) -> str:
    mt = str(getattr(hf_config, "model_type", "")).lower()
    archs = [a.lower() for a in (getattr(hf_config, "architectures", None) or [])]
    joined = " ".join(archs)
    if "minicpm" in mt or "minicpm" in joined:
        return "minicpm"
    if "llava" in mt or "llava" in joined:
        return "llava"
    if "qwen3" in mt or "qwen3" in joined:
        return "qwen3"
    if "qwen2" in mt or "qwen2" in joined:
        return "qwen2"
    if "llama" in mt or "llama" in joined or "mistral" in mt:
        return "llama"
    raise ValueError(f"unsupported model type {mt!r} / architectures {archs}")


def _llama(cfg):
    from .llama import LlamaForCausalLM
    return LlamaForCausalLM(cfg)


def _qwen3(cfg):
    from .qwen3 import Qwen3ForCausalLM
    return Qwen3ForCausalLM(cfg)


def _qwen2(cfg):
    from .qwen3 import Qwen2ForCausalLM
    return Qwen2ForCausalLM(cfg)


def _llava(cfg):
    from .llava import LlavaForConditionalGeneration
    return LlavaForConditionalGeneration(cfg)


def _minicpm(cfg):
    from .minicpm import MiniCPMForConditionalGeneration
    return MiniCPMForConditionalGeneration(cfg)


MODEL_REGISTRY: Dict[str, Callable] = {
    "llama": _llama, "qwen3": _qwen3, "qwen2": _qwen2, "llava": _llava, "minicpm": _minicpm,
}


def build_model(hf_config: Any):
    return MODEL_REGISTRY[detect_model_type(hf_config)](hf_config)
