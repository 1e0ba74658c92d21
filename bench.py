"""Headline benchmark: output tokens/s (and p50 TTFT) of the serving engine.

    python bench.py --gpus N --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (the reference's text benchmark shape): Qwen3-8B architecture, bf16,
random-init weights, synthetic token ids; 128 concurrent requests of 4096
prompt tokens and 512 output tokens each, sampled at temperature 0.6; KV eviction
by key norm (default: the variant of the reference's engine, so both arms do the
same work; --method knorm scores per head) or SnapKV (--method snapkv, window 64,
pooling kernel 5) keeping 50 % of the prompt rows; CUDA-graph decode; tensor
parallel over the N GPUs.

A "step" is one complete serving job: all requests of the workload submitted at
once and served to their last output token (the unit the reference's benchmark
times; output tokens/s and TTFT are only defined over a whole job).  W warm-up
steps are reduced waves (8 prompts of the job's prompt length, 4 output tokens)
that run every kernel at the job's prefill batch shape.  Then exactly K jobs are
timed between a barrier + synchronize on both sides (default K = 1).  Two numbers
come out of the same run:
  value      output tokens / device time, where device time is the sum of CUDA
             event intervals around the model and compression kernels of each
             step (max over ranks)
  e2e.value  output tokens / elapsed time of the whole step loop through the
             public `LLM.step()` API, including scheduling, the per-step copy of
             the step's inputs from pinned host memory and the read-back of the
             sampled tokens (max over ranks)
`--impl reference` runs the reference engine installed under baseline/_ref on the
same workload through its own API.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
                tie_word_embeddings=False, eos_token_id=151645, torch_dtype="bfloat16", hidden_act="silu",
                attention_bias=False, bos_token_id=151643)

LLAMA2_7B = dict(model_type="llama", architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=32, head_dim=128, intermediate_size=11008,
                 vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=4096,
                 tie_word_embeddings=False, eos_token_id=2, bos_token_id=1, torch_dtype="bfloat16",
                 hidden_act="silu", attention_bias=False)

QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)

# Long prompts under memory pressure: lazy CCM merge (ratio 4) fires when the paged pool passes 90 %
LAZY_CCM = dict(mode="lazy", threshold=0.9, factor=4, compressor="KVCacheLinearCompressor")

WORKLOADS = {
    # name: (hf config, requests, prompt tokens, output tokens[, compression override])
    "qwen3-8b": (QWEN3_8B, 128, 4096, 512),
    # 8 GPUs: 256 x 32768-token prompts do not fit the pool uncompressed (262 KB of KV per token)
    "qwen3-32b": (QWEN3_32B, 256, 32768, 256, LAZY_CCM),
    "qwen3-32b-small": (dict(QWEN3_32B, num_hidden_layers=4), 24, 32768, 32, LAZY_CCM),
    # the language model of the LLaVA-1.5-7B config, text only (MHA: 4x the KV bytes per token of Qwen3-8B)
    "llama2-7b": (LLAMA2_7B, 64, 2048, 256),
    # shrunken variants for quick functional checks; never reported as the headline
    "qwen3-8b-small": (dict(QWEN3_8B, num_hidden_layers=4), 16, 1024, 32),
    "llama2-7b-small": (dict(LLAMA2_7B, num_hidden_layers=4), 16, 1024, 32),
}
MODEL_LABEL = {
    "qwen3-8b": "Qwen3-8B shape (36L, h4096, 32q/8kv, d128, ffn12288, vocab151936)",
    "llama2-7b": "Llama-2-7B shape (32L, h4096, 32 MHA heads, d128, ffn11008, vocab32000)",
    "qwen3-8b-small": "Qwen3-8B shape cut to 4 layers (functional check only)",
    "qwen3-32b": "Qwen3-32B shape (64L, h5120, 64q/8kv, d128, ffn25600, vocab151936)",
    "qwen3-32b-small": "Qwen3-32B shape cut to 4 layers (functional check only)",
    "llama2-7b-small": "Llama-2-7B shape cut to 4 layers (functional check only)",
}


# decode steps per engine step while no request is waiting or being compressed (tokens are the same as with 1;
# the host then synchronises once per group: end-to-end +0.6 % on one GPU, +1.9 % on four, device time unchanged)
DECODE_STEPS_PER_CALL = 4
SAMPLING_TEMPERATURE = 0.6          # the reference's benchmarks sample at 0.6 (bench_llava.py:54-117)
COMPRESSION_LABEL = {
    "knorm_ref": "knorm keep 50% (reference engine-native variant)",
    "knorm": "knorm keep 50% (per-head scores, smallest norms kept)",
    "snapkv": "snapkv keep 50% (window 64, kernel 5)",
    "streaming_llm": "streaming_llm keep 50%",
}


def job_config(model_label, n_req, p_len, o_len, world, compression, engine_steps):
    """The part of the `config` entry that both arms (this build and the reference) fill identically."""
    return {"model": model_label, "global_batch": n_req, "seq_len": p_len, "output_len": o_len,
            "parallelism": f"tp{world}", "compression": compression, "temperature": SAMPLING_TEMPERATURE,
            "cuda_graph_decode": True, "kv_block": 256,
            "l2": "working set per step (weights 16 GB + KV) far exceeds the 126 MB L2; no flush needed",
            "step": "one whole job (all requests submitted at once, served to completion)",
            "warmup_step": "wave of 8 prompts of the same length, 4 output tokens",
            "engine_steps": engine_steps}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(vis.split(",")[self.index]) if vis else self.index
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                     "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                     "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                     "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
            get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = get(h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
                self._stop_evt.wait(self.period)
        except Exception as exc:                       # NVML missing: report that instead of numbers
            self.reasons.add(f"nvml_unavailable:{type(exc).__name__}")

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


_RESULT_OUT = None


def claim_stdout() -> None:
    """Keeps the process's standard output for the one result line.  Libraries write to file descriptor 1 as well
    (NCCL prints "NCCL version ..." there when a communicator is created): from here on descriptor 1 is stderr,
    and `emit` writes the JSON line to the original standard output."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def max_over_ranks(x: float, world: int) -> float:
    if world <= 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def prompts_for(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(1000, vocab - 1000, (length,), generator=g).tolist() for _ in range(n)]


def percentile(xs, q):
    xs = sorted(xs)
    if not xs:
        return None
    i = min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))
    return xs[i]


# ----------------------------------------------------------------------- ours
def run_ours(args):
    import torch
    rank, local_rank, world = dist_env()
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    from fastcache_b200 import LLM, SamplingParams, ops
    from fastcache_b200.engine.model_runner import DeviceTimer
    from fastcache_b200.parallel import tp as tpmod
    if world > 1:
        tpmod.init_tensor_parallel(world, rank)
    hf, n_req, p_len, o_len = WORKLOADS[args.config][:4]
    override = WORKLOADS[args.config][4] if len(WORKLOADS[args.config]) > 4 else None
    n_req = args.requests or n_req
    method = args.method
    kv_params = {"window": 64, "kernel_size": 5} if method == "snapkv" else {}
    if override is None:
        comp_kw = dict(enable_compression=not args.no_compression, compression_backend="kvpress",
                       kvpress_method=method, compression_factor=2, compression_pipeline="prefill",
                       kvpress_params=kv_params)
        comp_label = COMPRESSION_LABEL.get(method, f"{method} keep 50%")
    else:
        from fastcache_b200 import compress as compress_mod
        head_dim = hf.get("head_dim") or hf["hidden_size"] // hf["num_attention_heads"]
        torch.manual_seed(0)
        comp = getattr(compress_mod, override["compressor"])(None, override["factor"], 2,
                                                             n_layer=hf["num_hidden_layers"], nhead=2,
                                                             head_dim=head_dim)
        for prm in comp.parameters():
            torch.nn.init.normal_(prm, std=0.02)
        comp_kw = dict(compression_mode=override["mode"], lazy_occupancy_threshold=override["threshold"],
                       compression_backend="mlp", compressor=comp.eval(), compression_factor=override["factor"],
                       compression_pipeline="prefill")
        if args.no_compression:
            comp_kw = dict(enable_compression=False)
        comp_label = f"{override['mode']} CCM merge ratio {override['factor']} above {override['threshold']:.0%} pool occupancy"
    llm = LLM(dict(hf), tensor_parallel_size=world, device=f"cuda:{local_rank}", kvcache_block_size=256,
              max_model_len=p_len + o_len + 256, max_num_seqs=max(n_req, 8), max_num_batched_tokens=32768,
              gpu_memory_utilization=args.mem_util, seed=0, prefix_caching=False,
              decode_steps_per_call=args.decode_steps,
              **({"num_kvcache_blocks": args.kv_blocks} if args.kv_blocks > 0 else {}), **comp_kw)
    runner = llm.model_runner
    sp = SamplingParams(temperature=SAMPLING_TEMPERATURE, max_tokens=o_len, ignore_eos=True)

    # ---- warm-up (untimed): W reduced waves that run every kernel of the job at its full
    # prefill batch shape (8 prompts of the job's length), compression and graph decode included
    wsp = SamplingParams(temperature=SAMPLING_TEMPERATURE, max_tokens=4, ignore_eos=True)
    for w in range(args.warmup):
        for p in prompts_for(min(8, n_req), p_len, hf["vocab_size"], 1000 + w):
            llm.add_request(p, wsp)
        while not llm.is_finished():
            llm.step()

    # ---- K timed jobs
    runner.timer = DeviceTimer(runner.main_stream)
    runner.io["h2d_bytes"] = runner.io["d2h_bytes"] = 0
    ops.COUNTERS["launches"] = 0
    sampler = ClockSampler(local_rank)
    seqs = []
    engine_steps = 0
    barrier(world)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(runner.main_stream)
    t0 = time.perf_counter()
    for job in range(args.steps):
        batch = [llm.add_request(p, sp) for p in prompts_for(n_req, p_len, hf["vocab_size"], 1 + job)]
        t_arrival = time.perf_counter()
        for s in batch:
            s.arrival_time = t_arrival
        seqs.extend(batch)
        while not llm.is_finished():
            llm.step()
            engine_steps += 1
    steps = args.steps
    ev1.record(runner.main_stream)
    barrier(world)
    t1 = time.perf_counter()
    clocks = sampler.stop()
    e2e_ms = max(ev0.elapsed_time(ev1), 0.0)
    wall_ms = (t1 - t0) * 1e3
    dev_ms = runner.timer.total_ms()
    runner.timer = None
    out_tokens = sum(s.num_completion_tokens for s in seqs)
    ttft = [s.first_token_time - s.arrival_time for s in seqs if s.first_token_time is not None]
    status = ops.ext().read_status(local_rank)

    dev_ms = max_over_ranks(dev_ms, world)
    e2e_ms = max_over_ranks(max(e2e_ms, wall_ms), world)
    if rank == 0:
        base = None
        value = out_tokens / (dev_ms / 1e3)
        line = {
            "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / max(1, steps), 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": base, "dtype": "bf16",
            "data": "synthetic token ids, random-init weights",
            "config": dict(job_config(MODEL_LABEL[args.config], n_req, p_len, o_len, world,
                                      comp_label if not args.no_compression else "none", engine_steps),
                           compressions=llm.stats.compressions, lazy_triggers=llm.stats.lazy_triggers,
                           preemptions=llm.stats.preemptions, blocks_freed=llm.stats.blocks_freed,
                           prefill_steps=llm.stats.prefill_steps, decode_steps=llm.stats.decode_steps,
                           decode_steps_per_call=args.decode_steps,
                           **({"symmetric_memory": runner.fused_comm.runtime, "allreduce_form": runner.fused_comm.ar_form}
                              if runner.fused_comm is not None else {})),
            "p50_ttft_s": round(percentile(ttft, 0.5), 4) if ttft else None,
            "p99_ttft_s": round(percentile(ttft, 0.99), 4) if ttft else None,
            "output_tokens": out_tokens,
            "e2e": {"value": round(out_tokens / (e2e_ms / 1e3), 2), "unit": "tok/s",
                    "ms_total": round(e2e_ms, 2),
                    "h2d_bytes_per_step": int(runner.io["h2d_bytes"] / max(1, steps)),
                    "d2h_bytes_per_step": int(runner.io["d2h_bytes"] / max(1, steps))},
            "gpu_launches": int(ops.COUNTERS["launches"]),
            "clocks": clocks, "device_status": int(status), "impl": "fastcache_b200",
        }
        emit(line)
    llm.exit()
    if world > 1:
        tpmod.cleanup_tensor_parallel()



# ------------------------------------------------------- correctness check of the tensor-parallel path
def compare_first_tokens(got, want):
    """(agreeing, total) over the requests' first sampled tokens."""
    n = min(len(got), len(want))
    return sum(int(a == b) for a, b in zip(got[:n], want[:n])), max(len(got), len(want))


def run_check(args):
    """`--check`: greedy first tokens of every request of a shrunken job under tensor parallelism against the same
    prompts on one GPU.  Rank 0 first runs the one-GPU job as a child process (before it touches the device
    itself), then all ranks run the N-GPU job; one JSON line says how many first tokens agree.  Random-init
    weights give nearly flat logits, so a few near-ties may flip between reduction orders: "ok" means at least
    90 % agree, a broken collective gives about 0 %."""
    import json
    import subprocess
    import tempfile
    rank, local_rank, world = dist_env()
    cfg = args.config if args.config.endswith("-small") else "qwen3-8b-small"
    want = None
    if world > 1 and rank == 0:
        out = os.path.join(tempfile.gettempdir(), f"fc_check_{os.getpid()}.json")
        env = {k: v for k, v in os.environ.items()
               if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "GROUP_RANK",
                            "LOCAL_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE") and not k.startswith("TORCHELASTIC")}
        subprocess.run([sys.executable, os.path.abspath(__file__), "--check", "--gpus", "1", "--config", cfg,
                        "--check-out", out], env=env, check=True, timeout=1200, stdout=subprocess.DEVNULL)
        with open(out) as f:
            want = json.load(f)["first_tokens"]
        os.unlink(out)
    import torch
    torch.cuda.set_device(local_rank)
    from fastcache_b200 import LLM, SamplingParams, ops
    from fastcache_b200.parallel import tp as tpmod
    if world > 1:
        tpmod.init_tensor_parallel(world, rank)
    hf, n_req, p_len, o_len = WORKLOADS[cfg][:4]
    llm = LLM(dict(hf), tensor_parallel_size=world, device=f"cuda:{local_rank}", kvcache_block_size=256,
              max_model_len=p_len + o_len + 256, max_num_seqs=max(n_req, 8), max_num_batched_tokens=32768,
              gpu_memory_utilization=args.mem_util, seed=0, prefix_caching=False, enable_compression=True,
              compression_backend="kvpress", kvpress_method=args.method, compression_factor=2,
              compression_pipeline="prefill")
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    seqs = [llm.add_request(p, sp) for p in prompts_for(n_req, p_len, hf["vocab_size"], 1)]
    while not llm.is_finished():
        llm.step()
    got = [int(s.completion_token_ids[0]) for s in seqs]
    status = ops.ext().read_status(local_rank)
    if rank == 0:
        if args.check_out:
            with open(args.check_out, "w") as f:
                json.dump({"first_tokens": got}, f)
        line = {"check": "first sampled token of every request", "config": MODEL_LABEL[cfg], "n_gpus": world,
                "requests": n_req, "device_status": int(status)}
        if want is not None:
            agree, total = compare_first_tokens(got, want)
            line.update(agree=agree, of=total, result="ok" if agree >= 0.9 * total and status == 0 else "MISMATCH")
        else:
            line.update(result="reference tokens written" if args.check_out else "one GPU: nothing to compare with")
        emit(line)
    llm.exit()
    if world > 1:
        tpmod.cleanup_tensor_parallel()
    if rank == 0 and want is not None and line["result"] != "ok":
        raise SystemExit(1)


# ------------------------------------------------------- multimodal serving jobs
LLAVA_15_7B = dict(
    model_type="llava", architectures=["LlavaForConditionalGeneration"], image_token_index=32000,
    vision_feature_layer=-2, vision_feature_select_strategy="default", torch_dtype="bfloat16",
    text_config=dict(model_type="llama", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                     num_key_value_heads=32, head_dim=128, intermediate_size=11008, vocab_size=32064,
                     rms_norm_eps=1e-5, max_position_embeddings=4096, rope_theta=10000.0, eos_token_id=2),
    vision_config=dict(hidden_size=1024, intermediate_size=4096, num_hidden_layers=24, num_attention_heads=16,
                       image_size=336, patch_size=14))
MINICPM_V_26 = dict(
    model_type="minicpmv", architectures=["MiniCPMV"], hidden_size=3584, num_hidden_layers=28,
    num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=151666, rms_norm_eps=1e-6,
    max_position_embeddings=32768, rope_theta=1000000.0, query_num=64, max_slice_nums=9, scale_resolution=448,
    image_token_id=151646, eos_token_id=151645, torch_dtype="bfloat16",
    vision_config=dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16,
                       image_size=980, patch_size=14))


def _shrunk(cfg, layers, vision_layers):
    c = dict(cfg)
    if "text_config" in c:
        c["text_config"] = dict(c["text_config"], num_hidden_layers=layers)
    else:
        c["num_hidden_layers"] = layers
    c["vision_config"] = dict(c["vision_config"], num_hidden_layers=vision_layers)
    return c


SERVING = {
    # name: model config, image (H, W), text tokens, output tokens, requests, req/s, [prefill, compress, decode]
    # caps, compressor class, green-context (main, compress) SM counts or None
    "llava-1.5-7b": dict(hf=LLAVA_15_7B, image=(336, 336), text=64, out=128, requests=90, rate=10.0,
                         batching=(15, 45, 90), compressor="KVCacheLinearDecoupleCompressor", greenctx=None,
                         label="LLaVA-1.5-7B shape (CLIP ViT-L/14-336 + 2-layer MLP projector + Llama-2-7B)"),
    "minicpm-v-2.6": dict(hf=MINICPM_V_26, image=(896, 1344), text=64, out=128, requests=90, rate=10.0,
                          batching=(15, 45, 90), compressor="KVCacheHybridCompressor", greenctx=(112, 36),
                          label="MiniCPM-V-2.6 shape (SigLIP-400M + resampler, 64 queries per slice, + Qwen2-7B)"),
    "llava-small": dict(hf=_shrunk(LLAVA_15_7B, 2, 2), image=(336, 336), text=64, out=16, requests=12, rate=50.0,
                        batching=(4, 8, 12), compressor="KVCacheLinearDecoupleCompressor", greenctx=None,
                        label="LLaVA-1.5-7B shape cut to 2 + 2 layers (functional check only)"),
    "minicpm-small": dict(hf=_shrunk(MINICPM_V_26, 2, 2), image=(896, 1344), text=64, out=16, requests=12,
                          rate=50.0, batching=(4, 8, 12), compressor="KVCacheHybridCompressor", greenctx=(112, 36),
                          label="MiniCPM-V-2.6 shape cut to 2 + 2 layers (functional check only)"),
}


def run_serving(args):
    """Open-loop serving job: one synthetic image + text tokens per request, Poisson arrivals, CCM
    merge compression at ratio 4, three-stage batching.  A "step" is one whole arrival process served to
    its last token; `value` counts output tokens over the device-busy time of the engine steps, `e2e`
    over the elapsed time of the job (which an open-loop job cannot finish before its last arrival)."""
    import torch
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    from fastcache_b200 import LLM, ops
    from fastcache_b200 import compress as compress_mod
    from fastcache_b200.engine.model_runner import DeviceTimer
    from fastcache_b200.parallel import tp as tpmod
    from fastcache_b200.serving.harness import ConcurrentTester
    if world > 1:
        tpmod.init_tensor_parallel(world, rank)
    w = SERVING[args.config]
    hf = w["hf"]
    text_cfg = hf.get("text_config", hf)
    n_layer, head_dim = text_cfg["num_hidden_layers"], text_cfg.get("head_dim") or \
        text_cfg["hidden_size"] // text_cfg["num_attention_heads"]
    torch.manual_seed(0)
    comp = getattr(compress_mod, w["compressor"])(None, 4, 2, n_layer=n_layer, nhead=2, head_dim=head_dim)
    for p in comp.parameters():
        torch.nn.init.normal_(p, std=0.02)
    green = {}
    split = w["greenctx"] if args.greenctx == "config" else \
        ((112, 36) if args.greenctx == "on" else None)
    if split is not None:
        main_sms, comp_sms = split
        green = dict(greenctx_enabled=True, greenctx_main_ratio=main_sms / 148.0,
                     greenctx_compress_ratio=comp_sms / 148.0, greenctx_main_stream=args.greenctx_main)
    rate = 1e9 if args.closed_loop else w["rate"]          # closed loop: every request is there at the start
    if args.pipeline == "auto":
        args.pipeline = "async" if split is not None else "prefill"
    pipeline_kw = dict(compression_pipeline=args.pipeline, decode_overlap=args.decode_overlap)
    if args.pipeline == "async":
        pipeline_kw = dict(compression_pipeline="prefill", async_compression=True)
    n_req = args.requests or w["requests"]
    llm = LLM(dict(hf), tensor_parallel_size=world, device=f"cuda:{local_rank}", kvcache_block_size=64,
              max_model_len=2048, max_num_seqs=max(n_req, 8), max_num_batched_tokens=16384,
              gpu_memory_utilization=min(args.mem_util, 0.6), enable_compression=not args.no_compression,
              compression_backend="mlp", compressor=comp.eval(), compression_factor=4,
              seed=0, prefix_caching=False, **pipeline_kw, **green)
    runner = llm.model_runner
    vocab = text_cfg["vocab_size"]
    g = torch.Generator().manual_seed(3)
    H, W = w["image"]

    def make_job(n, seed):
        gg = torch.Generator().manual_seed(seed)
        prompts = [torch.randint(1000, min(vocab, 30000) - 1000, (w["text"],), generator=gg).tolist() for _ in range(n)]
        images = [torch.rand(3, H, W, generator=gg) for _ in range(n)]
        return prompts, images

    agree = None
    if world > 1:
        import torch.distributed as dist
        box = torch.zeros(1, dtype=torch.int64, device="cuda")

        def agree(n):
            box.fill_(int(n))
            dist.broadcast(box, src=0)
            return int(box.item())

    # warm-up: W short arrival processes (a prefill batch, its compression, a few decode steps each)
    for i in range(args.warmup):
        prompts, images = make_job(min(8, n_req), 100 + i)
        ConcurrentTester(llm, batching=w["batching"], req_per_sec=1000.0, poisson=False).run(
            prompts, max_tokens=4, images=images, agree=agree)

    runner.timer = DeviceTimer(runner.main_stream)
    runner.io["h2d_bytes"] = runner.io["d2h_bytes"] = 0
    ops.COUNTERS["launches"] = 0
    steps0 = llm.stats.steps
    sampler = ClockSampler(local_rank)
    barrier(world)
    sampler.start()
    t0 = time.perf_counter()
    results = []
    for job in range(args.steps):
        prompts, images = make_job(n_req, 1 + job)
        tester = ConcurrentTester(llm, batching=w["batching"], req_per_sec=rate, poisson=not args.closed_loop, seed=job)
        results.append(tester.run(prompts, max_tokens=w["out"], images=images, agree=agree))
    barrier(world)
    wall_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    dev_ms = max_over_ranks(runner.timer.total_ms(), world)
    wall_ms = max_over_ranks(wall_ms, world)
    runner.timer = None
    status = ops.ext().read_status(local_rank)
    if rank == 0:
        res = [r.to_dict() for r in results]
        out_tokens = sum(int(r["output_tokens"]) for r in res)
        engine_steps = llm.stats.steps - steps0
        line = {
            "metric": "output_tokens_per_s", "value": round(out_tokens / (dev_ms / 1e3), 2), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random images and token ids, random-init weights and compressor",
            "config": {"model": w["label"], "global_batch": n_req, "seq_len": None, "text_tokens": w["text"],
                       "image": f"{W}x{H}", "output_len": w["out"],
                       "arrivals": "closed loop (all at once)" if args.closed_loop else f"Poisson {w['rate']} req/s",
                       "pipeline": args.pipeline,
                       "batching": list(w["batching"]), "parallelism": f"tp{world}",
                       "compression": "CCM merge, ratio 4 (" + w["compressor"] + ")" if not args.no_compression else "none",
                       "greenctx_sms": list(split) if split else None,
                       "greenctx_active": bool(runner.greenctx_enabled),
                       "greenctx_sms_actual": [runner._greenctx_info.get("main_sms"),
                                               runner._greenctx_info.get("compress_sms")]
                       if runner.greenctx_enabled else None, "cuda_graph_decode": True,
                       "l2": "weights (13-16 GB) stream every step: far larger than the 126 MB L2; no flush needed",
                       "step": "one whole arrival process (all requests, served to completion)",
                       "value_is": "output tokens / device-busy time of the engine steps",
                       "engine_steps": engine_steps, "compressions": llm.stats.compressions},
            "p50_ttft_s": round(res[-1]["ttft"].get("p50", 0.0), 4), "p99_ttft_s": round(res[-1]["ttft"].get("p99", 0.0), 4),
            "serving": {k: res[-1][k] for k in ("completed", "failed", "wall_s", "ttft", "tpot", "latency", "compression")},
            "output_tokens": out_tokens,
            "e2e": {"value": round(out_tokens / (wall_ms / 1e3), 2), "unit": "tok/s", "ms_total": round(wall_ms, 2),
                    "h2d_bytes_per_step": int(runner.io["h2d_bytes"] / args.steps),
                    "d2h_bytes_per_step": int(runner.io["d2h_bytes"] / args.steps)},
            "gpu_launches": int(ops.COUNTERS["launches"]), "clocks": clocks, "device_status": int(status),
            "impl": "fastcache_b200",
        }
        emit(line)
    llm.exit()
    if world > 1:
        tpmod.cleanup_tensor_parallel()


# ------------------------------------------------------------------ reference
def unavailable(why: str):
    emit({"impl": "reference", "unavailable": why})
    sys.exit(0)


def run_reference(args):
    rank, local_rank, world = dist_env()
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "nanovllm", "engine")):
        if rank == 0:
            unavailable("reference is not installed under baseline/_ref")
        sys.exit(0)
    if args.config in SERVING:
        if not args.config.startswith("llava") or world > 1:
            if rank == 0:
                unavailable("no reference run of this image config: the reference's MiniCPM engine borrows its "
                            "vision modules from a HuggingFace remote-code checkpoint (nanovllm/models/minicpm.py:"
                            "329-340), which random weights cannot stand in for, and its LLaVA attention hard-codes "
                            "tp_size = 1 (nanovllm/models/llava.py:220), so only --config llava-1.5-7b on one GPU has one")
            sys.exit(0)
        if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref_p", "nanovllm", "engine")):
            unavailable("the reference's pipeline copy is not present under baseline/_ref_p")
        from baseline.reference_arm import run_llava
        try:
            line = run_llava(args, SERVING[args.config], ClockSampler, percentile)
        except SystemExit:
            raise
        except Exception as exc:
            import traceback
            traceback.print_exc()
            unavailable(f"reference failed: {type(exc).__name__}: {str(exc)[:200]}")
        emit(line)
        return
    if world > 1:
        family = WORKLOADS[args.config][0].get("model_type")
        if family != "llama":
            if rank == 0:
                unavailable("the reference cannot run this model tensor-parallel: its Qwen3 attention hard-codes "
                            "tp_size = 1 (nanovllm/models/qwen3.py:36); only its Llama family reads the degree "
                            "(--config llama2-7b has a reference arm at every N)")
            sys.exit(0)
        if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref_p", "nanovllm", "engine")):
            if rank == 0:
                unavailable("the reference's tensor-parallel copy is not present under baseline/_ref_p")
            sys.exit(0)
    from baseline.reference_arm import run as ref_run
    try:
        line = ref_run(args, WORKLOADS[args.config], MODEL_LABEL[args.config], ClockSampler, prompts_for,
                       percentile, rank, local_rank, world)
    except SystemExit:
        raise
    except Exception as exc:                       # import/runtime failure of the reference itself
        import traceback
        traceback.print_exc()
        if rank == 0:
            unavailable(f"reference failed: {type(exc).__name__}: {str(exc)[:200]}")
        sys.exit(0)
    if rank == 0:
        emit(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1, help="whole jobs to time")
    ap.add_argument("--warmup", type=int, default=3, help="reduced warm-up waves (at least 3)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen3-8b", choices=sorted(WORKLOADS) + sorted(SERVING))
    ap.add_argument("--method", default="knorm_ref", choices=["knorm", "snapkv", "knorm_ref", "streaming_llm"],
                    help="knorm_ref: the key-norm variant of the reference's engine (head-mean norms, one index set for "
                         "all heads, largest kept), the one both arms run; knorm: per-head scores, smallest norms kept")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--no-compression", action="store_true")
    ap.add_argument("--mem-util", type=float, default=0.85)
    ap.add_argument("--kv-blocks", type=int, default=0, help="size of the paged pool in blocks (0 = from free memory)")
    # serving configs only
    ap.add_argument("--greenctx", default="config", choices=["config", "on", "off"],
                    help="SM split between decode and compression: as the config says, 112 / 36, or none (priority streams)")
    ap.add_argument("--greenctx-main", action="store_true", help="run the main stream on its green context too")
    ap.add_argument("--closed-loop", action="store_true", help="all requests at once instead of Poisson arrivals")
    ap.add_argument("--decode-overlap", default="shadow", choices=["shadow", "hold"],
                    help="decode pipeline: compress into shadow blocks while the request keeps decoding, or in place "
                         "with the request held out of the decode batches")
    ap.add_argument("--pipeline", default="auto", choices=["auto", "prefill", "async", "decode"],
                    help="compression right after prefill on the main stream, on a compression stream, or a few "
                         "layers per decode step beside decode; auto: a compression stream when the SMs are split "
                         "(measured best: the split only pays when compression runs beside the main stream), else prefill")
    ap.add_argument("--decode-steps", type=int, default=DECODE_STEPS_PER_CALL,
                    help="decode steps launched back to back per engine step while nothing is waiting (one host "
                         "synchronisation per launch group); 1 = one step at a time")
    ap.add_argument("--check", action="store_true",
                    help="instead of timing: first tokens under --gpus N against the same prompts on one GPU "
                         "(shrunken config, greedy)")
    ap.add_argument("--check-out", default="", help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    args.steps = max(1, args.steps)
    claim_stdout()
    if args.check:
        run_check(args)
        return
    if args.impl == "reference":
        run_reference(args)
    elif args.config in SERVING:
        run_serving(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
