"""One engine step of each kind on a shallow copy of the benchmark model, for launch lists.

    python benchmarks/step_profile.py --layers 4
    ncu --metrics gpu__time_duration.sum --clock-control none --nvtx --nvtx-include "decode/" \
        --csv --log-file launches.csv python benchmarks/step_profile.py --layers 4

The model is the Qwen3-8B shape cut to `--layers` layers (every layer launches the same
kernels, so shares per layer carry over); the batch shapes are those of the headline job:
a decode step of 128 requests at 2304 rows of context each and a prefill step of 8 prompts
of 4096 tokens.  The two steps sit in NVTX ranges "decode" and "prefill".  Without a profiler
the script prints the CUDA-event time of each step.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from bench import QWEN3_8B, prompts_for  # noqa: E402
from fastcache_b200 import LLM, SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--decode-batch", type=int, default=128)
    ap.add_argument("--context", type=int, default=2304)
    ap.add_argument("--graphs", action="store_true", help="decode through CUDA graphs (one launch per step)")
    ap.add_argument("--shard", type=int, default=1,
                    help="run the per-rank shapes of a tensor-parallel shard of this degree (heads, KV heads and "
                         "ffn width divided; no communication)")
    args = ap.parse_args()
    hf = dict(QWEN3_8B, num_hidden_layers=args.layers)
    if args.shard > 1:
        hf.update(num_attention_heads=hf["num_attention_heads"] // args.shard,
                  num_key_value_heads=max(1, hf["num_key_value_heads"] // args.shard),
                  intermediate_size=hf["intermediate_size"] // args.shard)
    blocks = args.decode_batch * (-(-(args.context + 16) // 256)) + 8 * 17 + 8
    llm = LLM(hf, device="cuda:0", kvcache_block_size=256, max_model_len=8192, max_num_seqs=args.decode_batch + 32,
              max_num_batched_tokens=32768, num_kvcache_blocks=blocks, enforce_eager=not args.graphs,
              prefix_caching=False)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    for p in prompts_for(args.decode_batch, args.context, hf["vocab_size"], 1):
        llm.add_request(p, sp)
    while llm.scheduler.waiting:
        llm.step()
    llm.step()
    llm.step()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    torch.cuda.nvtx.range_push("decode")
    ev[0].record()
    llm.step()
    ev[1].record()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    # the same prefill step once untimed (one output token, so the requests leave at once): the first step of a
    # new shape grows the caching allocator, which is not part of a steady-state step
    for p in prompts_for(8, 4096, hf["vocab_size"], 3):
        llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
    llm.step()
    torch.cuda.synchronize()
    for p in prompts_for(8, 4096, hf["vocab_size"], 2):
        llm.add_request(p, sp)
    torch.cuda.nvtx.range_push("prefill")
    ev[2].record()
    llm.step()
    ev[3].record()
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    print({"layers": args.layers, "decode_step_ms": round(ev[0].elapsed_time(ev[1]), 3),
           "prefill_step_ms": round(ev[2].elapsed_time(ev[3]), 3), "decode_batch": args.decode_batch,
           "context": args.context, "prefill_tokens": 8 * 4096})


if __name__ == "__main__":
    main()
