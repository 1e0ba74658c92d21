"""Checkpoints and numerics against HuggingFace `transformers` models (CPU, fp32).

A tiny Llama and a tiny Qwen3 (per-head q/k RMSNorm) are saved with `save_pretrained(safe_serialization=True)`
and read back through this package's own path (`ModelConfig.from_pretrained`, `load_model`, the shard loaders of
the packed projections); prefill logits and greedy continuations must agree with the HuggingFace forward.
The reference's loader is nanovllm/utils/loader.py:12-62.  A checkpoint whose names do not match is an error.
"""
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")

from fastcache_b200 import LLM, SamplingParams  # noqa: E402


def _save(tmp_path, kind, tie=False):
    torch.manual_seed(0)
    common = dict(hidden_size=64, intermediate_size=160, num_hidden_layers=3, num_attention_heads=4,
                  num_key_value_heads=2, vocab_size=320, max_position_embeddings=512, rms_norm_eps=1e-6,
                  tie_word_embeddings=tie, rope_theta=50000.0)      # not the default base
    if kind == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM
        model = LlamaForCausalLM(LlamaConfig(**common))
    elif kind == "qwen3":
        from transformers import Qwen3Config, Qwen3ForCausalLM
        model = Qwen3ForCausalLM(Qwen3Config(head_dim=32, **common))          # head_dim != hidden / heads
    else:
        from transformers import Qwen2Config, Qwen2ForCausalLM
        model = Qwen2ForCausalLM(Qwen2Config(**common))                      # q/k/v biases
    model = model.eval().float()
    with torch.no_grad():                                    # norm weights away from one, biases away from zero
        for name, p in model.named_parameters():
            if "norm" in name or name.endswith(".bias"):
                p.add_(torch.randn_like(p) * 0.1)
    path = str(tmp_path / kind)
    model.save_pretrained(path, safe_serialization=True)
    return model, path


def _engine(path, **kw):
    return LLM(path, device="cpu", dtype="fp32", enforce_eager=True, kvcache_block_size=16, num_kvcache_blocks=64,
               max_model_len=256, **kw)


def _prompts(vocab, n=3, seed=2):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, vocab, (int(torch.randint(9, 40, (1,), generator=g)),), generator=g).tolist()
            for _ in range(n)]


@pytest.mark.parametrize("kind,tie", [("llama", False), ("llama", True), ("qwen3", False), ("qwen2", False)])
def test_prefill_logits_and_greedy_tokens_match_transformers(tmp_path, kind, tie):
    hf, path = _save(tmp_path, kind, tie)
    llm = _engine(path)
    prompts = _prompts(hf.config.vocab_size)
    seqs = [llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)) for p in prompts]
    batch, is_prefill = llm.scheduler.schedule()
    assert is_prefill and len(batch) == len(prompts)
    logits = llm.model_runner.run_prefill(batch).float()
    for i, p in enumerate(prompts):
        with torch.no_grad():
            want = hf(input_ids=torch.tensor([p])).logits[0, -1]
        torch.testing.assert_close(logits[i], want, rtol=2e-4, atol=2e-4)
    # the whole loop (paged decode included) against HuggingFace greedy generation
    llm2 = _engine(path)
    outs = llm2.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([p]), max_new_tokens=6, do_sample=False, eos_token_id=None,
                               pad_token_id=0)[0, len(p):].tolist()
        assert o["token_ids"] == want


def test_checkpoint_with_other_names_is_refused(tmp_path):
    from safetensors.torch import load_file, save_file
    _, path = _save(tmp_path, "llama")
    file = os.path.join(path, "model.safetensors")
    state = load_file(file)
    save_file({("transformer." + k[len("model."):] if k.startswith("model.layers.1.") else k): v
               for k, v in state.items()}, file)
    with pytest.raises(RuntimeError, match="parameters were not found"):
        _engine(path)
    os.remove(file)
    with pytest.raises(FileNotFoundError):
        _engine(path)


def test_random_init_reaches_every_parameter_of_every_family():
    """The checkpoint-shape tables that drive random initialisation name every parameter of every model family
    (so `load_model`'s missing-parameter check cannot misfire on a complete checkpoint)."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import tiny_llama_config, tiny_qwen3_config
    from test_vision_cpu import _llava_cfg, _minicpm_cfg
    from fastcache_b200.models.registry import build_model
    from fastcache_b200.utils.loader import init_random_weights
    for cfg in (tiny_llama_config(), tiny_qwen3_config(), tiny_llama_config(tie_word_embeddings=True),
                _llava_cfg(), _minicpm_cfg()):
        model = build_model(cfg)
        stats = init_random_weights(model, model.hf_weight_shapes(cfg))
        assert stats["missing"] == [] and stats["unknown"] == 0, (cfg.model_type, stats)
