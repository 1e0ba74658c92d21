"""Worker for the tensor-parallel tests: launched with torch.distributed.run (any world size,
including 1) on CPU (gloo) or CUDA (nccl).  Writes its results as JSON on rank 0."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from fastcache_b200 import LLM, SamplingParams  # noqa: E402
from fastcache_b200.parallel import tp as tpmod  # noqa: E402
from helpers import tiny_qwen3_config  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--out", required=True)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--one-shot-tokens", type=int, default=512)
    ap.add_argument("--chunk", type=int, default=0, help="chunked_prefill_tokens (with a 64-token step budget)")
    ap.add_argument("--shard-embedding", action="store_true", help="vocabulary-parallel embedding table + all-reduce")
    ap.add_argument("--decode-steps", type=int, default=1, help="decode steps launched back to back per engine step")
    a = ap.parse_args()
    if a.shard_embedding:
        from fastcache_b200.layers import embed_head
        embed_head.REPLICATE_EMBEDDING_BYTES = 0
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    res = {}
    if world > 1:
        tpmod.init_tensor_parallel(world, rank, backend="nccl" if a.device == "cuda" else "gloo", timeout_s=120)
    device = f"cuda:{local}" if a.device == "cuda" else "cpu"

    if a.device == "cuda" and world > 1:
        # fused all-reduce + residual + RMSNorm against the library all-reduce
        from fastcache_b200 import ops
        from fastcache_b200.ops import reference as ref
        from fastcache_b200.parallel import symm
        torch.cuda.set_device(local)
        comm = symm.enable(512, 1024, torch.device(device), max_tokens=4096)
        # GEMM + reduce-scatter + add + norm, then all-gather + GEMM, against the library all-reduce
        fused_errs = []
        for it, T in enumerate([600, 1000, 4096, 777]):
            gx = torch.Generator(device="cpu").manual_seed(1000 + 10 * it + rank)
            x = (torch.randn(T, 256, generator=gx) * 0.5).to(torch.bfloat16).to(device)
            wr = (torch.randn(1024, 256, generator=gx) * 0.05).to(torch.bfloat16).to(device)
            gs = torch.Generator(device="cpu").manual_seed(2000 + it)
            resid = torch.randn(T, 1024, generator=gs).to(torch.bfloat16).to(device)
            nw = (1.0 + 0.1 * torch.randn(1024, generator=gs)).to(torch.bfloat16).to(device)
            wc = (torch.randn(768, 1024, generator=gs) * 0.05).to(torch.bfloat16).to(device)
            total = x.float() @ wr.float().T
            torch.distributed.all_reduce(total)
            want_n, want_r = ref.add_rms_norm(total.to(torch.bfloat16), resid.clone(), nw, 1e-6)
            want_y = want_n.float() @ wc.float().T
            comm.begin_forward()
            normed, shard = comm.row_linear_reduce_add_norm(x, wr, None, resid.clone(), nw, 1e-6)
            y = ops.linear(normed, wc)                      # all-gather + GEMM path
            normed = comm.finish_forward(normed)
            torch.cuda.synchronize()
            chunk = comm.chunk_rows_for(T)
            lo, hi = min(T, rank * chunk), min(T, rank * chunk + chunk)
            fused_errs.append(float((normed.float() - want_n.float()).abs().max()))
            fused_errs.append(float((shard.float() - want_r[lo:hi].float()).abs().max()) if hi > lo else 0.0)
            fused_errs.append(float((y.float() - want_y).abs().max()) / max(1.0, float(want_y.abs().max())))
            torch.distributed.barrier()
        res["fused_prefill_max_err"] = max(fused_errs)
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        errs = []
        for it, T in enumerate([1, 7, 128, 300]):
            part = (torch.randn(T, 1024, generator=g) * 0.5).to(torch.bfloat16).to(device)
            gres = torch.Generator(device="cpu").manual_seed(7 + it)
            resid = torch.randn(T, 1024, generator=gres).to(torch.bfloat16).to(device)
            w = torch.ones(1024, dtype=torch.bfloat16, device=device)
            total = part.float().clone()
            torch.distributed.all_reduce(total)
            want_n, want_r = ref.add_rms_norm(total.to(torch.bfloat16), resid.clone(), w, 1e-6)
            for mm in ([False, True] if comm.use_multimem or os.environ.get("FC_MULTIMEM") == "1" else [False]):
                buf = it % 2
                comm.own_rows(buf, T).copy_(part)
                r2 = resid.clone()
                y = ops.ext().allreduce_add_rmsnorm(buf, r2, w, 1e-6, mm, comm.status)
                torch.cuda.synchronize()
                errs.append(float((y.float() - want_n.float()).abs().max()))
                errs.append(float((r2.float() - want_r.float()).abs().max()))
                torch.distributed.barrier()
        res["allreduce_max_err"] = max(errs)
        res["status"] = int(ops.ext().read_status(local))

    cfg = tiny_qwen3_config(hidden_size=512, num_attention_heads=8, num_key_value_heads=a.kv_heads, head_dim=64,
                            intermediate_size=1024, vocab_size=2000)
    llm = LLM(cfg, device=device, dtype="bf16" if a.device == "cuda" else "fp32", tensor_parallel_size=world,
              kvcache_block_size=16, num_kvcache_blocks=128, max_model_len=256, max_num_seqs=8,
              enforce_eager=False, init_device="cpu", fused_comm_tokens=a.one_shot_tokens,
              decode_steps_per_call=a.decode_steps, prefix_caching=a.decode_steps < 2,
              **({"chunked_prefill_tokens": a.chunk, "max_num_batched_tokens": 64} if a.chunk else {}))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 2000, (n,), generator=g).tolist() for n in (9, 40, 77, 120)]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    res["tokens"] = [o["token_ids"] for o in out]
    # sampled (not greedy) tokens: every rank must draw the same ones, from its own vocabulary shard
    warm = llm.generate(prompts, SamplingParams(temperature=0.8, max_tokens=6, ignore_eos=True))
    res["sampled"] = [o["token_ids"] for o in warm]
    res["decode_steps"] = int(llm.stats.decode_steps)
    res["prefill_steps"] = int(llm.stats.prefill_steps)
    res["engine_steps"] = int(llm.stats.steps)
    if world > 1:
        mine = {"tokens": res["tokens"], "sampled": res["sampled"]}
        everyone = [None] * world
        torch.distributed.all_gather_object(everyone, mine)
        res["ranks_agree"] = all(e == everyone[0] for e in everyone)
    if a.device == "cuda":
        from fastcache_b200 import ops as _ops
        res["engine_status"] = int(_ops.ext().read_status(local))
        res["local_logits"] = bool(llm.model_runner.local_logits)
        res["embedding_replicated"] = bool(llm.model_runner.model.model.embed_tokens.replicated)
    llm.exit()
    if rank == 0:
        with open(a.out, "w") as fh:
            json.dump(res, fh)
    if world > 1:
        if a.device == "cuda":
            from fastcache_b200.parallel import symm
            symm.disable()
        tpmod.cleanup_tensor_parallel()


if __name__ == "__main__":
    main()
