"""Models x workloads x engine variants, one JSON row per cell, resumable.

The same experiment grid as the reference's matrix script ("kv-cache pipeline"/bench/
bench_kvcache_matrix.py:336-474, :585-599):

  workloads  heavy-trace     prompts / outputs drawn from a request-trace CSV (columns with the
                             context and generated token counts, Azure LLM inference trace layout);
                             without a file, a seeded stand-in with the same length filters
             light-dataset   short prompts (32-128 tokens), 64 output tokens
             synthetic-long  fixed long context, fixed output length
  variants   baseline            no compression
             compression-only    compression on, fixed policy
             greenctx-only       + compression streams on their own SM group (green context)
             auto-tune+greenctx  + the online controller chooses pipeline, streams and SM split
             triad               + the controller also alternates prefill and decode batches

Every finished cell is appended to the output file at once; `--resume` skips cells the file
already has; a cell that raises is recorded with its error and the sweep goes on.  Models are
random-initialised from their architecture (no checkpoints are needed); `--scale tiny` swaps in
two-layer models and short lengths so the whole grid also runs on a CPU.

    python benchmarks/matrix_bench.py --models qwen3-8b --workloads synthetic-long --output m.json
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import random
import sys
import time
import zlib
from dataclasses import asdict, dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from fastcache_b200 import LLM, SamplingParams  # noqa: E402
from fastcache_b200 import compress as compress_mod  # noqa: E402

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
                tie_word_embeddings=False, eos_token_id=151645)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, intermediate_size=25600)
LLAMA2_7B = dict(model_type="llama", architectures=["LlamaForCausalLM"], hidden_size=4096, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=32, head_dim=128, intermediate_size=11008,
                 vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=4096,
                 tie_word_embeddings=False, eos_token_id=2)
TINY = dict(model_type="llama", architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1024,
            rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=False,
            eos_token_id=2)

# name -> (architecture, compression backend, eviction method or None)
MODELS: Dict[str, Tuple[dict, str, Optional[str]]] = {
    "qwen3-8b": (QWEN3_8B, "kvpress", "knorm"),
    "qwen3-32b": (QWEN3_32B, "kvpress", "knorm"),
    "llava-mlp": (LLAMA2_7B, "mlp", None),          # the language model of LLaVA-1.5-7B with the merge compressor
}


@dataclass
class WorkloadSpec:
    name: str
    mode: str                       # trace | dataset | synthetic
    num_batches: int = 1
    max_output_tokens: int = 64
    min_prompt_tokens: int = 32
    max_prompt_tokens: int = 128
    trace_path: str = ""
    trace_min_context: int = 1024
    trace_min_output: int = 256
    trace_max_output: int = 512
    synthetic_context: int = 3072
    synthetic_output: int = 512
    batch_sizes: Tuple[int, ...] = (8,)


@dataclass
class ConfigVariant:
    label: str
    compression: bool = True
    auto_tune: bool = False
    greenctx: bool = False
    auto_dual: bool = False


VARIANTS = [ConfigVariant("baseline", compression=False),
            ConfigVariant("compression-only"),
            ConfigVariant("greenctx-only", greenctx=True),
            ConfigVariant("auto-tune+greenctx", auto_tune=True, greenctx=True),
            ConfigVariant("triad", auto_tune=True, greenctx=True, auto_dual=True)]


# ------------------------------------------------------------------- workloads
def read_trace(path: str, min_context: int, min_output: int, max_output: int, limit: int
               ) -> List[Tuple[int, int]]:
    """(context tokens, output tokens) of the trace rows that pass the filters, in file order."""
    rows: List[Tuple[int, int]] = []
    with open(path, newline="") as fh:
        reader = csv.DictReader(fh)
        cols = {c.lower(): c for c in reader.fieldnames or []}
        c_ctx = cols.get("contexttokens") or cols.get("context_tokens")
        c_out = cols.get("generatedtokens") or cols.get("generated_tokens")
        if c_ctx is None or c_out is None:
            raise ValueError(f"{path}: need ContextTokens and GeneratedTokens columns, have {reader.fieldnames}")
        for r in reader:
            ctx, out = int(float(r[c_ctx])), int(float(r[c_out]))
            if ctx >= min_context and min_output <= out:
                rows.append((ctx, min(out, max_output)))
                if len(rows) >= limit:
                    break
    return rows


def requests_for(spec: WorkloadSpec, batch: int, vocab: int, max_len: int, seed: int
                 ) -> List[Tuple[List[int], int]]:
    """`batch * num_batches` (prompt token ids, output length) pairs."""
    rng = random.Random(seed)
    n = batch * spec.num_batches
    if spec.mode == "trace":
        if spec.trace_path and os.path.exists(spec.trace_path):
            shapes = read_trace(spec.trace_path, spec.trace_min_context, spec.trace_min_output,
                                spec.trace_max_output, n)
        else:                       # seeded stand-in with the same filters (long-tailed context lengths)
            shapes = [(int(min(8 * spec.trace_min_context, spec.trace_min_context * (1.0 + rng.expovariate(1.5)))),
                       rng.randint(spec.trace_min_output, spec.trace_max_output)) for _ in range(n)]
        shapes = (shapes * (n // max(1, len(shapes)) + 1))[:n]
    elif spec.mode == "dataset":
        shapes = [(rng.randint(spec.min_prompt_tokens, spec.max_prompt_tokens), spec.max_output_tokens)
                  for _ in range(n)]
    else:
        shapes = [(spec.synthetic_context, spec.synthetic_output)] * n
    out = []
    for ctx, gen in shapes:
        gen = min(gen, spec.max_output_tokens)
        ctx = max(4, min(ctx, max_len - gen - 8))
        out.append(([rng.randrange(3, vocab) for _ in range(ctx)], gen))
    return out


# ---------------------------------------------------------------------- a cell
def build_engine(arch: dict, backend: str, method: Optional[str], variant: ConfigVariant, factor: int,
                 device: str, max_len: int, max_seqs: int, args) -> LLM:
    kw: Dict[str, Any] = dict(device=device, kvcache_block_size=args.block_size, max_model_len=max_len,
                              max_num_seqs=max_seqs, max_num_batched_tokens=args.max_batched_tokens, seed=0,
                              prefix_caching=False, enforce_eager=device == "cpu")
    if args.kv_blocks > 0:
        kw["num_kvcache_blocks"] = args.kv_blocks
    else:
        kw["gpu_memory_utilization"] = args.gpu_mem_util
    if variant.compression:
        kw.update(enable_compression=True, compression_factor=factor, compression_backend=backend,
                  compression_pipeline="auto" if variant.auto_tune else "prefill",
                  greenctx_enabled=variant.greenctx, greenctx_compress_ratio=args.greenctx_compress_ratio,
                  greenctx_main_ratio=args.greenctx_main_ratio, greenctx_main_stream=args.greenctx_main_stream,
                  auto_tune=variant.auto_tune, auto_dual_batch=variant.auto_dual)
        if backend == "mlp":
            head_dim = arch.get("head_dim") or arch["hidden_size"] // arch["num_attention_heads"]
            torch.manual_seed(0)
            comp = compress_mod.KVCacheLinearDecoupleCompressor(None, factor, 2, n_layer=arch["num_hidden_layers"],
                                                                nhead=2, head_dim=head_dim)
            for p in comp.parameters():
                torch.nn.init.normal_(p, std=0.02)
            kw["compressor"] = comp.eval()
        else:
            kw["kvpress_method"] = method
    return LLM(dict(arch), **kw)


def run_cell(llm: LLM, reqs: Sequence[Tuple[List[int], int]], batch: int, warmup_waves: int = 1
             ) -> Dict[str, Any]:
    """Feeds the requests in waves of `batch`; throughput counts generated tokens over wall time
    bracketed by device synchronisation.  `warmup_waves` untimed waves of the same prompts with four
    output tokens run first, so every kernel shape of the cell (compression included) has been used."""
    cuda = llm.model_runner.device.type == "cuda"
    sync = (lambda: torch.cuda.synchronize(llm.model_runner.device)) if cuda else (lambda: None)
    for _ in range(warmup_waves):
        for ids, _n in reqs[:batch]:
            llm.add_request(ids, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
        while not llm.is_finished():
            llm.step()
    base_stats = (llm.stats.compressions, llm.stats.blocks_freed, llm.stats.preemptions)
    bm = llm.scheduler.block_manager
    gen = prompt = steps = 0
    min_free = bm.num_free_blocks
    first: Dict[int, float] = {}
    arrive: Dict[int, float] = {}
    sync()
    t0 = time.perf_counter()
    for i in range(0, len(reqs), batch):
        for ids, n_out in reqs[i:i + batch]:
            s = llm.add_request(ids, SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True))
            arrive[s.seq_id] = time.perf_counter()
            prompt += len(ids)
        live = list(llm.scheduler.waiting)
        while not llm.is_finished():
            llm.step()
            steps += 1
            min_free = min(min_free, bm.num_free_blocks)
            now = None
            for s in live:
                if s.seq_id not in first and s.num_completion_tokens > 0:
                    if now is None:
                        sync()
                        now = time.perf_counter()
                    first[s.seq_id] = now - arrive[s.seq_id]
        gen += sum(n for _, n in reqs[i:i + batch])
    sync()
    dt = time.perf_counter() - t0
    ttft = sorted(first.values())
    st = llm.stats
    return {"throughput_tok_s": gen / dt, "total_time_s": dt, "generated_tokens": gen, "prompt_tokens": prompt,
            "engine_steps": steps, "ttft_p50_s": ttft[len(ttft) // 2] if ttft else None,
            "ttft_p99_s": ttft[min(len(ttft) - 1, int(0.99 * len(ttft)))] if ttft else None,
            "compressions": st.compressions - base_stats[0], "blocks_freed": st.blocks_freed - base_stats[1],
            "preemptions": st.preemptions - base_stats[2],
            "min_free_blocks": min_free, "total_blocks": bm.num_blocks}


def run_cell_here(args, arch: dict, backend: str, method: Optional[str], variant: ConfigVariant,
                  reqs: Sequence[Tuple[List[int], int]], batch: int, max_len: int) -> Dict[str, Any]:
    """Build the engine, run the cell, free the engine.  A failure comes back as {"error": ...}."""
    llm = None
    out: Dict[str, Any] = {}
    try:
        llm = build_engine(arch, backend, method, variant, args.compression_factor, args.device, max_len,
                           max(batch, 8), args)
        out["greenctx_active"] = bool(llm.model_runner.greenctx_enabled)
        out.update(run_cell(llm, reqs, batch, args.warmup_waves))
    except Exception as exc:                            # one broken cell must not end the sweep
        out["error"] = f"{type(exc).__name__}: {exc}"
    try:
        if llm is not None:
            llm.exit()
    except Exception as exc:                            # a device error is sticky: report it, do not mask the first
        out.setdefault("error", f"{type(exc).__name__}: {exc}")
    del llm
    if torch.cuda.is_available() and "error" not in out:
        torch.cuda.empty_cache()
    return out


def run_cell_in_child(args, model: str, spec: WorkloadSpec, batch: int, variant: ConfigVariant, max_len: int
                      ) -> Dict[str, Any]:
    """The cell in a process of its own: a fresh device context per cell, so a device error (which
    is sticky for the process that hit it) or memory left behind by one engine cannot reach the next
    cell.  The child prints its result as one JSON line."""
    import subprocess
    cell = {"model": model, "spec": asdict(spec), "batch": batch, "variant": asdict(variant), "max_len": max_len,
            "args": {k: v for k, v in vars(args).items() if k not in ("cell",)}}
    try:
        proc = subprocess.run([sys.executable, os.path.abspath(__file__), "--cell", json.dumps(cell)],
                              capture_output=True, text=True, timeout=args.cell_timeout)
    except subprocess.TimeoutExpired:
        return {"error": f"cell exceeded {args.cell_timeout} s"}
    for line in reversed(proc.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    tail = (proc.stderr or "").strip().splitlines()[-1:] or [""]
    return {"error": f"child exited {proc.returncode}: {tail[0][:300]}"}


def child_main(cell: Dict[str, Any]) -> None:
    args = argparse.Namespace(**cell["args"])
    spec = WorkloadSpec(**{**cell["spec"], "batch_sizes": tuple(cell["spec"]["batch_sizes"])})
    variant = ConfigVariant(**cell["variant"])
    arch, backend, method = MODELS[cell["model"]]
    if args.scale == "tiny":
        arch = dict(TINY)
    reqs = requests_for(spec, cell["batch"], arch["vocab_size"], cell["max_len"], cell_seed(cell["model"], spec.name))
    out = run_cell_here(args, arch, backend, method, variant, reqs, cell["batch"], cell["max_len"])
    sys.stdout.write(json.dumps(out) + "\n")
    sys.stdout.flush()
    if "error" in out:
        os._exit(1)                  # skip interpreter teardown after a device error


def cell_seed(model: str, workload: str) -> int:
    return zlib.crc32(f"{model}/{workload}".encode()) & 0xffff


# ------------------------------------------------------------------------ main
def load_done(path: str) -> Tuple[List[Dict[str, Any]], set]:
    try:
        with open(path, "r", encoding="utf-8") as fh:
            rows = json.load(fh)
    except (OSError, ValueError):
        return [], set()
    done = {(r.get("model"), r.get("workload"), r.get("batch_size"), r.get("variant"))
            for r in rows if "error" not in r}
    return [r for r in rows if "error" not in r], done


def save(path: str, rows: List[Dict[str, Any]]) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as fh:
        json.dump(rows, fh, indent=1)
    os.replace(tmp, path)


def main(argv: Optional[Sequence[str]] = None) -> List[Dict[str, Any]]:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--output", default="kvcache_matrix_results.json")
    ap.add_argument("--models", default="qwen3-8b,qwen3-32b,llava-mlp")
    ap.add_argument("--workloads", default="")
    ap.add_argument("--variants", default="")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--trace-conv", default="", help="request-trace CSV (ContextTokens, GeneratedTokens)")
    ap.add_argument("--synthetic-context", type=int, default=3072)
    ap.add_argument("--synthetic-output", type=int, default=512)
    ap.add_argument("--synthetic-num-batches", type=int, default=2)
    ap.add_argument("--batch-sizes", default="8", help="comma list; every workload runs at each")
    ap.add_argument("--compression-factor", type=int, default=2)
    ap.add_argument("--gpu-mem-util", type=float, default=0.9)
    ap.add_argument("--kv-blocks", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--max-batched-tokens", type=int, default=32768)
    ap.add_argument("--greenctx-compress-ratio", type=float, default=0.25)
    ap.add_argument("--greenctx-main-ratio", type=float, default=None)
    ap.add_argument("--greenctx-main-stream", action="store_true")
    ap.add_argument("--warmup-waves", type=int, default=1)
    ap.add_argument("--isolate", default="auto", choices=["auto", "on", "off"],
                    help="one process per cell (auto: on a CUDA device)")
    ap.add_argument("--cell-timeout", type=float, default=1800.0)
    ap.add_argument("--cell", default="", help=argparse.SUPPRESS)
    ap.add_argument("--scale", default="full", choices=["full", "tiny"])
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    if args.cell:
        child_main(json.loads(args.cell))
        return []
    args.isolate = args.isolate == "on" or (args.isolate == "auto" and args.device.startswith("cuda"))
    if args.greenctx_main_ratio is None:
        args.greenctx_main_ratio = max(0.05, 1.0 - args.greenctx_compress_ratio)
    tiny = args.scale == "tiny"
    if tiny:
        args.block_size = min(args.block_size, 16)
        args.kv_blocks = args.kv_blocks or 512
        args.max_batched_tokens = min(args.max_batched_tokens, 4096)

    batches = tuple(int(x) for x in args.batch_sizes.split(",") if x.strip())
    div = 16 if tiny else 1
    workloads = [WorkloadSpec("heavy-trace", "trace", 4 if not tiny else 1, 512 // div, trace_path=args.trace_conv,
                              trace_min_context=1024 // div, trace_min_output=256 // div,
                              trace_max_output=512 // div, batch_sizes=batches),
                 WorkloadSpec("light-dataset", "dataset", 1, 64 // div, 32 // (2 if tiny else 1),
                              128 // (2 if tiny else 1), batch_sizes=batches),
                 WorkloadSpec("synthetic-long", "synthetic", max(1, args.synthetic_num_batches if not tiny else 1),
                              args.synthetic_output // div, synthetic_context=args.synthetic_context // div,
                              synthetic_output=args.synthetic_output // div, batch_sizes=batches)]
    pick = {w.strip() for w in args.workloads.split(",") if w.strip()}
    workloads = [w for w in workloads if not pick or w.name in pick]
    pick = {v.strip() for v in args.variants.split(",") if v.strip()}
    variants = [v for v in VARIANTS if not pick or v.label in pick]

    rows, done = load_done(args.output) if args.resume else ([], set())
    if args.resume:
        print(f"resume: {len(rows)} finished cells in {args.output}", file=sys.stderr)
    for name in [m.strip() for m in args.models.split(",") if m.strip()]:
        arch, backend, method = MODELS[name]
        if tiny:
            arch = dict(TINY)
        for spec in workloads:
            for batch in spec.batch_sizes:
                max_len = 8 * max(spec.trace_min_context, spec.synthetic_context, spec.max_prompt_tokens) \
                    + spec.max_output_tokens + 64
                max_len = min(max_len, arch["max_position_embeddings"])
                reqs = requests_for(spec, batch, arch["vocab_size"], max_len, seed=cell_seed(name, spec.name))
                base: Optional[float] = next((r["throughput_tok_s"] for r in rows if
                                              (r["model"], r["workload"], r["batch_size"], r["variant"]) ==
                                              (name, spec.name, batch, "baseline")), None)
                for variant in variants:
                    key = (name, spec.name, batch, variant.label)
                    if key in done:
                        continue
                    row: Dict[str, Any] = {"model": name, "workload": spec.name, "batch_size": batch,
                                           "variant": variant.label,
                                           "backend": (backend if variant.compression else "none"),
                                           "method": method if variant.compression else None,
                                           "compression_factor": args.compression_factor, "scale": args.scale,
                                           "workload_spec": asdict(spec), "device": args.device}
                    if args.isolate:
                        row.update(run_cell_in_child(args, name, spec, batch, variant, max_len))
                    else:
                        row.update(run_cell_here(args, arch, backend, method, variant, reqs, batch, max_len))
                    if "error" not in row:
                        if variant.label == "baseline":
                            base = row["throughput_tok_s"]
                        if base:
                            row["speedup_vs_baseline"] = row["throughput_tok_s"] / base
                        done.add(key)
                    rows.append(row)
                    save(args.output, rows)
                    print(json.dumps({k: row.get(k) for k in ("model", "workload", "batch_size", "variant",
                                                              "throughput_tok_s", "speedup_vs_baseline", "error")}),
                          file=sys.stderr)
    return rows


if __name__ == "__main__":
    main()
