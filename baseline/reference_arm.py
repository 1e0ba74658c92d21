"""Runs the reference engine (installed unmodified under baseline/_ref) on the
benchmark workload through its own public API: `LlavaLLM(...)`, `add_request`,
`step(apply_compression=True)`.  Nothing of fastcache_b200 is imported here.

The reference can only load weights from a HuggingFace directory, so a seeded
random-init checkpoint (safetensors + config.json + a minimal tokenizer) is
written to a scratch directory first.  Two packages the reference imports are
absent from this environment (`xxhash`, `kvpress`); baseline/shims provides
stand-ins that only satisfy the imports (see their docstrings).
"""
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def _write_checkpoint(path, hf, seed=0):
    import torch
    from safetensors.torch import save_file
    if os.path.exists(os.path.join(path, "DONE")):
        return
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(hf, fh, indent=1)
    h, L = hf["hidden_size"], hf["num_hidden_layers"]
    heads, kvh, d = hf["num_attention_heads"], hf["num_key_value_heads"], hf["head_dim"]
    inter, vocab = hf["intermediate_size"], hf["vocab_size"]
    g = torch.Generator(device="cuda").manual_seed(seed)

    def rnd(*shape):
        return (torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16)

    index = {}
    def save(tensors, name):
        save_file(tensors, os.path.join(path, name))
        for k in tensors:
            index[k] = name

    save({"model.embed_tokens.weight": rnd(vocab, h), "model.norm.weight": ones(h),
          "lm_head.weight": rnd(vocab, h)}, "model-embed.safetensors")
    for i in range(L):
        p = f"model.layers.{i}."
        layer = {p + "self_attn.q_proj.weight": rnd(heads * d, h), p + "self_attn.k_proj.weight": rnd(kvh * d, h),
                 p + "self_attn.v_proj.weight": rnd(kvh * d, h), p + "self_attn.o_proj.weight": rnd(h, heads * d),
                 p + "mlp.gate_proj.weight": rnd(inter, h), p + "mlp.up_proj.weight": rnd(inter, h),
                 p + "mlp.down_proj.weight": rnd(h, inter), p + "input_layernorm.weight": ones(h),
                 p + "post_attention_layernorm.weight": ones(h)}
        if hf.get("model_type") == "qwen3":
            layer[p + "self_attn.q_norm.weight"] = ones(d)
            layer[p + "self_attn.k_norm.weight"] = ones(d)
        save(layer, f"model-layer{i:03d}.safetensors")
    # minimal tokenizer: the engine only needs eos_token_id and encode() for string prompts
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab_map = {"<unk>": 0, "<eos>": 1, "hello": 2}
    tok = Tokenizer(models.WordLevel(vocab_map, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as fh:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "unk_token": "<unk>"}, fh)
    with open(os.path.join(path, "special_tokens_map.json"), "w") as fh:
        json.dump({"eos_token": "<eos>", "unk_token": "<unk>"}, fh)
    open(os.path.join(path, "DONE"), "w").close()




def _transformers_4x_config_view():
    """The reference was written against transformers 4.x, where a config without rope scaling has
    `rope_scaling = None` and a top-level `rope_theta`.  transformers 5.x folds both into a
    `rope_parameters` dict, which the reference's `get_rope` (nanovllm/layers/rotary_embedding.py:63-73,
    an lru_cache over its arguments plus `assert rope_scaling is None`) cannot take.  This wraps
    `AutoConfig.from_pretrained` so that the object the reference receives reads as it did under 4.x.
    Nothing of the reference is changed."""
    import transformers
    orig = transformers.AutoConfig.from_pretrained

    def from_pretrained(path, *a, **kw):
        cfg = orig(path, *a, **kw)
        try:
            with open(os.path.join(str(path), "config.json")) as fh:
                raw = json.load(fh)
        except OSError:
            raw = {}
        targets = [cfg] + ([cfg.text_config] if getattr(cfg, "text_config", None) is not None else [])
        for c, r in zip(targets, [raw, raw.get("text_config", raw)]):
            params = getattr(c, "rope_parameters", None) or {}
            if params.get("rope_type", "default") == "default":
                theta = r.get("rope_theta", params.get("rope_theta"))
                c.rope_scaling = None
                if theta is not None:
                    c.rope_theta = float(theta)
        return cfg

    transformers.AutoConfig.from_pretrained = staticmethod(from_pretrained)


def run(args, workload, model_label, ClockSampler, prompts_for, percentile, rank=0, local_rank=0, world=1):
    """One rank of the reference arm.  world == 1: the copy installed under baseline/_ref.  world > 1: the
    reference's newer "kv-cache pipeline" copy (baseline/_ref_p, an unmodified copy of that directory), whose
    linear layers shard full checkpoint tensors, driven the way the reference's own tp_inference.py:34-123 drives
    it: every torchrun rank calls `init_tensor_parallel` and then builds and steps an identical `LlavaLLM`.
    Only the Llama family reads the tensor-parallel degree there (nanovllm/models/llama.py:39-44)."""
    import torch
    from bench import COMPRESSION_LABEL, SAMPLING_TEMPERATURE, job_config
    hf, n_req, p_len, o_len = workload[:4]
    n_req = args.requests or n_req
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, os.path.join(HERE, "_ref_p" if world > 1 else "_ref"))
    torch.cuda.set_device(local_rank)
    ckpt = os.path.join(os.environ.get("FC_REF_CKPT_DIR", "/tmp"), f"fc_ref_{args.config}")
    if world > 1:
        from nanovllm.utils.tp import init_tensor_parallel, tp_barrier
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        init_tensor_parallel(tp_size=world, rank=local_rank)
        if rank == 0:
            _write_checkpoint(ckpt, dict(hf))
        tp_barrier()
    else:
        _write_checkpoint(ckpt, dict(hf))
    _transformers_4x_config_view()

    from nanovllm.engine.llava_engine import LlavaLLM          # the reference's engine
    from nanovllm.sampling_params import SamplingParams

    compress = not args.no_compression
    method = "knorm" if args.method in ("knorm", "knorm_ref") else args.method
    llm = LlavaLLM(ckpt, enable_compression=compress, compression_backend="kvpress", kvpress_method=method,
                   compression_factor=2, async_compression=False, max_model_len=p_len + o_len + 256,
                   max_num_seqs=max(n_req, 8), max_num_batched_tokens=32768, kvcache_block_size=256,
                   gpu_memory_utilization=args.mem_util, enforce_eager=False)
    sp = SamplingParams(temperature=SAMPLING_TEMPERATURE, max_tokens=o_len, ignore_eos=True)
    wsp = SamplingParams(temperature=SAMPLING_TEMPERATURE, max_tokens=4, ignore_eos=True)
    for w in range(args.warmup):                    # the same reduced waves as the other arm
        for p in prompts_for(min(8, n_req), p_len, hf["vocab_size"], 1000 + w):
            llm.add_request(p, wsp)
        while not llm.is_finished():
            llm.step(apply_compression=compress)

    sampler = ClockSampler(local_rank)
    torch.cuda.synchronize()
    if world > 1:
        tp_barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.perf_counter()
    engine_steps = out_tokens = 0
    ttft = []
    for job in range(args.steps):
        for p in prompts_for(n_req, p_len, hf["vocab_size"], 1 + job):
            llm.add_request(p, sp)
        t_arrival = time.perf_counter()
        while not llm.is_finished():
            _, n = llm.step(apply_compression=compress)
            engine_steps += 1
            if n > 0:                               # a prefill step: each request in it got its first token
                now = time.perf_counter() - t_arrival
                batch = sum(1 for s in llm.scheduler.running if s.num_completion_tokens == 1)
                ttft.extend([now] * batch)
                out_tokens += batch
            else:
                out_tokens += -n
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        tp_barrier()
        torch.cuda.synchronize()
    t1 = time.perf_counter()
    clocks = sampler.stop()
    ms = max(ev0.elapsed_time(ev1), (t1 - t0) * 1e3)
    if world > 1:                                   # the slowest rank's time
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = out_tokens / (ms / 1e3)
    return {
        "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / max(1, args.steps), 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights",
        "config": job_config(model_label, n_req, p_len, o_len, world,
                             COMPRESSION_LABEL["knorm_ref"] if (compress and method == "knorm") else
                             (f"{method} keep 50%" if compress else "none"), engine_steps),
        "p50_ttft_s": round(percentile(ttft, 0.5), 4) if ttft else None,
        "p99_ttft_s": round(percentile(ttft, 0.99), 4) if ttft else None,
        "output_tokens": out_tokens,
        "e2e": {"value": round(value, 2), "unit": "tok/s", "ms_total": round(ms, 2),
                "note": "the reference exposes no device-only timer; its single number is end to end"},
        "clocks": clocks, "impl": "reference",
        "shims": ["xxhash", "kvpress", "transformers 4.x view of the config's rope fields"],
        "reference_copy": "kv-cache pipeline/nanovllm" if world > 1 else "nanovllm",
    }
