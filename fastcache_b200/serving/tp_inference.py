"""SPMD tensor-parallel driver (reference: tp_inference.py:34-123).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m fastcache_b200.serving.tp_inference --model DIR --tp-size N [--prompt-len 128 ...]

Every rank builds the same engine and runs the same step loop on the same requests; the
schedulers are deterministic replicas, the model is sharded, and the sampled tokens agree on all
ranks because the LM-head logits are gathered before sampling.  Rank 0 prints the results.
"""
from __future__ import annotations

import argparse
import json
import os
import time


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, help="HF directory, or a JSON file with an HF config for random init")
    ap.add_argument("--tp-size", type=int, default=int(os.environ.get("WORLD_SIZE", 1)))
    ap.add_argument("--num-prompts", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--compressor", default=None)
    ap.add_argument("--compression-backend", default="kvpress", choices=["kvpress", "mlp"])
    ap.add_argument("--kvpress-method", default="knorm")
    ap.add_argument("--compression-factor", type=int, default=2)
    ap.add_argument("--enable-compression", action="store_true")
    ap.add_argument("--backend", default=None, help="nccl (default on GPUs) or gloo")
    a = ap.parse_args(argv)

    import torch
    from .. import LLM, SamplingParams
    from ..parallel import tp as tpmod
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if a.tp_size > 1:
        tpmod.init_tensor_parallel(a.tp_size, rank, backend=a.backend)
    device = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
    model = a.model
    if os.path.isfile(model):
        model = json.load(open(model))
    llm = LLM(model, tensor_parallel_size=a.tp_size, device=device, compressor_path=a.compressor,
              enable_compression=a.enable_compression, compression_backend=a.compression_backend,
              kvpress_method=a.kvpress_method, compression_factor=a.compression_factor)
    vocab = llm.model_runner.text_config.vocab_size
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.num_prompts)]
    t0 = time.perf_counter()
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=a.max_tokens, ignore_eos=True))
    dt = time.perf_counter() - t0
    if rank == 0:
        n = sum(len(o["token_ids"]) for o in out)
        print(json.dumps({"tp": a.tp_size, "output_tokens": n, "seconds": round(dt, 3),
                          "tok_per_s": round(n / dt, 1), "first": out[0]["token_ids"][:8]}))
    llm.exit()
    if a.tp_size > 1:
        tpmod.cleanup_tensor_parallel()


if __name__ == "__main__":
    main()
