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


# ------------------------------------------------------------------ multimodal serving job (LLaVA-1.5 shape)
def _write_llava_checkpoint(path, hf, seed=0):
    """Random-init LLaVA-1.5 directory in the HuggingFace layout the reference loads
    (nanovllm/models/llava.py:440-464): safetensors, config.json, a tokenizer that knows `<image>` = 32000 and the
    processor files `AutoProcessor` needs for a `LlavaProcessor` with a CLIP image processor."""
    import torch
    from safetensors.torch import save_file
    if os.path.exists(os.path.join(path, "DONE")):
        return
    os.makedirs(path, exist_ok=True)
    cfg = dict(hf)
    cfg["vision_config"] = dict(cfg["vision_config"], model_type="clip_vision_model", projection_dim=768,
                                layer_norm_eps=1e-5, hidden_act="quick_gelu")
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(cfg, fh, indent=1)
    t, v = cfg["text_config"], cfg["vision_config"]
    h, L, heads, kvh, d = t["hidden_size"], t["num_hidden_layers"], t["num_attention_heads"], \
        t["num_key_value_heads"], t["head_dim"]
    inter, vocab = t["intermediate_size"], t["vocab_size"]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev).manual_seed(seed)

    def rnd(*shape):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16)

    def zeros(n):
        return torch.zeros(n, dtype=torch.bfloat16)

    lm = "language_model."
    save_file({lm + "model.embed_tokens.weight": rnd(vocab, h), lm + "model.norm.weight": ones(h),
               lm + "lm_head.weight": rnd(vocab, h)}, os.path.join(path, "model-embed.safetensors"))
    for i in range(L):
        p = f"{lm}model.layers.{i}."
        save_file({p + "self_attn.q_proj.weight": rnd(heads * d, h), p + "self_attn.k_proj.weight": rnd(kvh * d, h),
                   p + "self_attn.v_proj.weight": rnd(kvh * d, h), p + "self_attn.o_proj.weight": rnd(h, heads * d),
                   p + "mlp.gate_proj.weight": rnd(inter, h), p + "mlp.up_proj.weight": rnd(inter, h),
                   p + "mlp.down_proj.weight": rnd(h, inter), p + "input_layernorm.weight": ones(h),
                   p + "post_attention_layernorm.weight": ones(h)}, os.path.join(path, f"model-layer{i:03d}.safetensors"))
    vh, vi, vl, ps = v["hidden_size"], v["intermediate_size"], v["num_hidden_layers"], v["patch_size"]
    npos = (v["image_size"] // ps) ** 2 + 1
    vm = "vision_tower.vision_model."
    vis = {vm + "embeddings.class_embedding": rnd(vh), vm + "embeddings.patch_embedding.weight": rnd(vh, 3, ps, ps),
           vm + "embeddings.position_embedding.weight": rnd(npos, vh),
           vm + "pre_layrnorm.weight": ones(vh), vm + "pre_layrnorm.bias": zeros(vh),
           vm + "post_layernorm.weight": ones(vh), vm + "post_layernorm.bias": zeros(vh),
           "multi_modal_projector.linear_1.weight": rnd(h, vh), "multi_modal_projector.linear_1.bias": zeros(h),
           "multi_modal_projector.linear_2.weight": rnd(h, h), "multi_modal_projector.linear_2.bias": zeros(h)}
    for i in range(vl):
        p = f"{vm}encoder.layers.{i}."
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            vis[p + f"self_attn.{proj}.weight"] = rnd(vh, vh)
            vis[p + f"self_attn.{proj}.bias"] = zeros(vh)
        for ln in ("layer_norm1", "layer_norm2"):
            vis[p + ln + ".weight"], vis[p + ln + ".bias"] = ones(vh), zeros(vh)
        vis[p + "mlp.fc1.weight"], vis[p + "mlp.fc1.bias"] = rnd(vi, vh), zeros(vi)
        vis[p + "mlp.fc2.weight"], vis[p + "mlp.fc2.bias"] = rnd(vh, vi), zeros(vh)
    save_file(vis, os.path.join(path, "model-vision.safetensors"))
    # tokenizer with a dense vocabulary up to the image token, and the processor files
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab_map = {"<unk>": 0, "<s>": 1, "</s>": 2, "<image>": 32000}
    vocab_map.update({f"t{i}": i for i in range(3, 32000)})
    tok = Tokenizer(models.WordLevel(vocab_map, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(path, "tokenizer.json"))
    dump = lambda name, obj: json.dump(obj, open(os.path.join(path, name), "w"))      # noqa: E731
    dump("tokenizer_config.json", {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "</s>",
                                   "unk_token": "<unk>", "bos_token": "<s>", "processor_class": "LlavaProcessor"})
    dump("special_tokens_map.json", {"eos_token": "</s>", "unk_token": "<unk>", "bos_token": "<s>"})
    dump("preprocessor_config.json", {
        "image_processor_type": "CLIPImageProcessor", "processor_class": "LlavaProcessor",
        "crop_size": {"height": v["image_size"], "width": v["image_size"]}, "size": {"shortest_edge": v["image_size"]},
        "do_resize": True, "do_center_crop": True, "do_normalize": True, "do_rescale": True, "rescale_factor": 1 / 255,
        "do_convert_rgb": True, "resample": 3, "image_mean": [0.48145466, 0.4578275, 0.40821073],
        "image_std": [0.26862954, 0.26130258, 0.27577711]})
    dump("processor_config.json", {"processor_class": "LlavaProcessor", "patch_size": ps,
                                   "vision_feature_select_strategy": "default", "image_token": "<image>",
                                   "num_additional_image_tokens": 1})
    open(os.path.join(path, "DONE"), "w").close()


def run_llava(args, w, ClockSampler, percentile):
    """The reference's `LlavaLLM` on the image serving job: one random 336 x 336 image and 64 random text tokens
    around one `<image>` token per request (the reference's own synthetic multimodal workload,
    bench_llava.py:54-117), Poisson arrivals, CCM merge compression through its `mlp` backend with a random-init
    compressor saved in its own checkpoint layout.  One GPU: the reference's LLaVA attention hard-codes
    tp_size = 1 (nanovllm/models/llava.py:220)."""
    import random

    import numpy as np
    import torch
    from PIL import Image
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, os.path.join(HERE, "_ref_p"))
    torch.cuda.set_device(0)
    hf = w["hf"]
    ckpt = os.path.join(os.environ.get("FC_REF_CKPT_DIR", "/tmp"), f"fc_ref_{args.config}")
    _write_llava_checkpoint(ckpt, dict(hf))
    _transformers_4x_config_view()
    from transformers import AutoConfig

    from nanovllm.engine.llava_engine import LlavaLLM
    from nanovllm.sampling_params import SamplingParams
    from utils_ccm.module_ccm_v11 import KVCacheLinearDecoupleCompressor       # the reference's own module

    pth = os.path.join(ckpt, "compressor_f4.pth")
    if not os.path.exists(pth):
        torch.manual_seed(0)
        comp = KVCacheLinearDecoupleCompressor(AutoConfig.from_pretrained(ckpt), compression_factor=4, min_seq_len=2)
        for prm in comp.parameters():
            torch.nn.init.normal_(prm, std=0.02)
        torch.save({"model_state_dict": {"compressor": comp.state_dict()}}, pth)
        del comp
    n_req = args.requests or w["requests"]
    compress = not args.no_compression
    # the reference captures decode graphs for batch sizes 1, 2, 4, 8, 16, 32, ... up to max_num_seqs in steps of 16
    # and has no bucket for a batch above the last multiple of 16 (llava_model_runner.py:1353-1415, :782): give it a
    # multiple of 16
    llm = LlavaLLM(ckpt, compressor_path=pth, compression_factor=4, enable_compression=compress,
                   async_compression=False, compression_backend="mlp", max_model_len=2048,
                   max_num_seqs=-(-max(n_req, 8) // 16) * 16, max_num_batched_tokens=16384, kvcache_block_size=256,
                   gpu_memory_utilization=min(args.mem_util, 0.6), enforce_eager=False)
    sp = SamplingParams(temperature=0.6, max_tokens=w["out"], ignore_eos=True)
    vocab = 30000
    H, W = w["image"]

    def make_job(n, seed):
        rng, nrng = random.Random(seed), np.random.RandomState(seed)
        prompts, images = [], []
        for _ in range(n):
            toks = [rng.randrange(1000, vocab) for _ in range(w["text"])]
            toks.insert(rng.randrange(10, 30), 32000)
            prompts.append(toks)
            images.append(Image.fromarray(nrng.randint(0, 255, (H, W, 3), dtype=np.uint8), "RGB"))
        return prompts, images

    def serve(prompts, images, rate, max_tokens, seed):
        """Open loop: a request joins the engine at its arrival time; returns per-request records."""
        rng = random.Random(seed)
        arrivals, t = [], 0.0
        for _ in prompts:
            arrivals.append(t)
            t += rng.expovariate(rate)
        sps = SamplingParams(temperature=0.6, max_tokens=max_tokens, ignore_eos=True)
        live, recs, i = {}, [], 0
        t0 = time.perf_counter()
        while i < len(prompts) or not llm.is_finished():
            now = time.perf_counter() - t0
            while i < len(prompts) and arrivals[i] <= now:
                llm.add_request(prompts[i], sps, image=images[i])
                seq = llm.scheduler.waiting[-1]
                live[seq.seq_id] = {"seq": seq, "arrival": time.perf_counter(), "first": None, "done": None}
                i += 1
            if llm.is_finished():
                time.sleep(max(0.0, arrivals[i] - (time.perf_counter() - t0)))
                continue
            outputs, _ = llm.step(apply_compression=compress)
            now_abs = time.perf_counter()
            for r in live.values():
                if r["first"] is None and r["seq"].num_completion_tokens >= 1:
                    r["first"] = now_abs
            for sid, toks in outputs:
                r = live.pop(sid)
                r["done"], r["tokens"] = now_abs, len(toks)
                recs.append(r)
        return recs, time.perf_counter() - t0

    for k in range(args.warmup):                           # reduced waves, untimed
        p, im = make_job(4, 1000 + k)
        serve(p, im, 1e9, 4, k)
    sampler = ClockSampler(0)
    torch.cuda.synchronize()
    sampler.start()
    t0 = time.perf_counter()
    out_tokens, recs = 0, []
    for job in range(args.steps):
        p, im = make_job(n_req, 1 + job)
        recs, wall = serve(p, im, 1e9 if getattr(args, "closed_loop", False) else w["rate"], w["out"], job)
        out_tokens += sum(r["tokens"] for r in recs)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    ttft = [r["first"] - r["arrival"] for r in recs if r["first"] is not None]
    lat = [r["done"] - r["arrival"] for r in recs]
    tpot = [(r["done"] - r["first"]) / max(1, r["tokens"] - 1) for r in recs if r["first"] is not None]
    value = out_tokens / (ms / 1e3)
    return {
        "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / max(1, args.steps), 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform-random images and token ids, random-init weights and compressor",
        "config": {"model": w["label"], "global_batch": n_req, "text_tokens": w["text"], "image": f"{W}x{H}",
                   "output_len": w["out"],
                   "arrivals": "closed loop (all at once)" if getattr(args, "closed_loop", False)
                   else f"Poisson {w['rate']} req/s", "parallelism": "tp1",
                   "compression": "CCM merge, ratio 4 (reference mlp backend)" if compress else "none",
                   "temperature": 0.6, "cuda_graph_decode": True},
        "p50_ttft_s": round(percentile(ttft, 0.5), 4) if ttft else None,
        "p99_ttft_s": round(percentile(ttft, 0.99), 4) if ttft else None,
        "serving": {"completed": len(recs), "wall_s": round(ms / 1e3 / max(1, args.steps), 3),
                    "tpot_p50_s": round(percentile(tpot, 0.5), 5) if tpot else None,
                    "latency_p50_s": round(percentile(lat, 0.5), 4) if lat else None,
                    "latency_p99_s": round(percentile(lat, 0.99), 4) if lat else None},
        "output_tokens": out_tokens,
        "e2e": {"value": round(value, 2), "unit": "tok/s", "ms_total": round(ms, 2),
                "note": "the reference exposes no device-only timer; its single number is end to end"},
        "clocks": clocks, "impl": "reference", "reference_copy": "kv-cache pipeline/nanovllm",
        "shims": ["xxhash", "kvpress", "transformers 4.x view of the config's rope fields"],
        "known_reference_defects": "block tables of image requests are padded with indices the block manager never "
                                   "allocated and decode uses the text length as KV length "
                                   "(llava_model_runner.py:675-679, :733): the run is timed, its tokens are not meaningful",
    }
