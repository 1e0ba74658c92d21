"""Shared builders for the test-suite: tiny seeded models and compressors."""
import torch

from fastcache_b200.config import ModelConfig


def tiny_llama_config(**over):
    cfg = dict(model_type="llama", architectures=["LlamaForCausalLM"], hidden_size=256,
               num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
               intermediate_size=512, vocab_size=1024, rope_theta=10000.0, rms_norm_eps=1e-6,
               max_position_embeddings=2048, tie_word_embeddings=False, eos_token_id=2)
    cfg.update(over)
    return ModelConfig(**cfg)


def tiny_qwen3_config(**over):
    return tiny_llama_config(model_type="qwen3", architectures=["Qwen3ForCausalLM"], **over)


def random_compressor(cls, n_layer, head_dim, factor, seed=0, **kw):
    torch.manual_seed(seed)
    m = cls(None, factor, kw.pop("min_seq_len", 1), n_layer=n_layer, nhead=2, head_dim=head_dim)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    return m.eval()
