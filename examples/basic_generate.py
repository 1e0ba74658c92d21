"""Smallest use of the engine: build, generate, print.

    python examples/basic_generate.py /path/to/Qwen3-8B        # a HuggingFace checkpoint directory
    python examples/basic_generate.py                          # no checkpoint: tiny random-weight model

(Reference counterpart: example.py.)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fastcache_b200 import LLM, SamplingParams  # noqa: E402


def main() -> None:
    if len(sys.argv) > 1:
        llm = LLM(sys.argv[1], enable_compression=True, compression_backend="kvpress", kvpress_method="knorm",
                  compression_factor=2)
        prompts = ["Introduce yourself.", "List all prime numbers within 100."]
    else:
        cfg = dict(model_type="llama", architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512,
                   vocab_size=1024, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=2048,
                   tie_word_embeddings=False, eos_token_id=2)
        llm = LLM(cfg, kvcache_block_size=16, num_kvcache_blocks=128, max_model_len=512,
                  enable_compression=True, compression_backend="kvpress", kvpress_method="knorm",
                  compression_factor=2)
        prompts = [list(range(10, 90)), list(range(200, 260))]          # token ids instead of text
    outs = llm.generate(prompts, SamplingParams(temperature=0.6, max_tokens=32), use_tqdm=False)
    for p, o in zip(prompts, outs):
        print("prompt:", p if isinstance(p, str) else f"{len(p)} token ids")
        print("output:", o["text"] or o["token_ids"])
    llm.exit()


if __name__ == "__main__":
    main()
