"""Concurrent serving test from the command line: open-loop arrivals, three-stage batching, one
compression method per run, or a YAML batch of runs.

Same job as the reference's two harness scripts (scripts/llava_testcon2.6.py:2351-2419 and
scripts/minicpm_testcon2.6.py: argument parser, single run or `--config experiments.yaml`, results
file per run, optional GPU CSV), with their argument names.  Differences: the engine of this
package serves the requests (the reference drives HuggingFace `generate` and moves KV tensors
through a pool of its own), `--model_path` may be omitted to serve a seeded random-weight model of
the chosen architecture (`--arch`), and `--datasets_name synthetic` needs no files.

    python -m fastcache_b200.serving.testcon --model_mode llava --use_compression --comp_mode ccm \\
        --prefill_batch_size 15 --compress_batch_size 45 --decoding_batch_size 90
    python -m fastcache_b200.serving.testcon --config configs/experiments.yaml
"""
from __future__ import annotations

import argparse
import json
import os
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .datasets import load_image_data, load_image_data_milebench, synthetic_samples
from .experiments import Experiment, load_experiments
from .harness import ConcurrentTester

ARCHS: Dict[str, dict] = {
    "llava-1.5-7b": dict(
        model_type="llava", architectures=["LlavaForConditionalGeneration"], image_token_index=32000,
        vision_feature_layer=-2,
        text_config=dict(model_type="llama", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                         num_key_value_heads=32, head_dim=128, intermediate_size=11008, vocab_size=32064,
                         rms_norm_eps=1e-5, max_position_embeddings=4096, rope_theta=10000.0, eos_token_id=2),
        vision_config=dict(hidden_size=1024, intermediate_size=4096, num_hidden_layers=24, num_attention_heads=16,
                           image_size=336, patch_size=14)),
    "minicpm-v-2.6": dict(
        model_type="minicpmv", architectures=["MiniCPMV"], hidden_size=3584, num_hidden_layers=28,
        num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=151666,
        rms_norm_eps=1e-6, max_position_embeddings=32768, rope_theta=1000000.0, query_num=64, max_slice_nums=9,
        scale_resolution=448, image_token_id=151646, eos_token_id=151645,
        vision_config=dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16,
                           image_size=980, patch_size=14)),
    # two-layer models for functional runs on a CPU
    "tiny-llava": dict(
        model_type="llava", architectures=["LlavaForConditionalGeneration"], image_token_index=500,
        text_config=dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=4, intermediate_size=256, vocab_size=600, rms_norm_eps=1e-5,
                         max_position_embeddings=1024, rope_theta=10000.0),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           image_size=56, patch_size=14)),
    "tiny-minicpm": dict(
        model_type="minicpmv", architectures=["MiniCPMV"], hidden_size=128, num_hidden_layers=2,
        num_attention_heads=4, num_key_value_heads=2, intermediate_size=256, vocab_size=600, rms_norm_eps=1e-6,
        max_position_embeddings=2048, rope_theta=1e6, query_num=4, max_slice_nums=9, scale_resolution=56,
        image_token_id=501,
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           image_size=140, patch_size=14)),
}
DEFAULT_ARCH = {"llava": "llava-1.5-7b", "minicpm": "minicpm-v-2.6"}


def parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="concurrent serving test (three-stage batching, one compression mode)")
    p.add_argument("--config", default=None, help="YAML with global_settings and experiments; replaces the "
                   "single-run switches below")
    p.add_argument("--model_mode", default="llava", choices=["llava", "minicpm"])
    p.add_argument("--model_path", default="", help="HuggingFace checkpoint directory; empty: random weights")
    p.add_argument("--arch", default="", choices=[""] + sorted(ARCHS), help="architecture when no checkpoint is given")
    p.add_argument("--ckpt_path", default="", help="merge-compressor checkpoint (.pth); empty: random compressor")
    p.add_argument("--folder_path", default="results_log/")
    p.add_argument("--datasets_js_path", default="")
    p.add_argument("--datasets_img_path", default="./datasets")
    p.add_argument("--datasets_name", default="synthetic", choices=["gqa", "milebench", "synthetic"])
    p.add_argument("--use_compression", action="store_true")
    p.add_argument("--comp_mode", default="orig",
                   help="ccm | Knorm | SnapKV | ExpectedAttention | StreamingLLM | Random | TOVA | orig")
    p.add_argument("--prefill_batch_size", type=int, default=15)
    p.add_argument("--compress_batch_size", type=int, default=45)
    p.add_argument("--decoding_batch_size", type=int, default=90)
    p.add_argument("--seed", type=int, default=48)
    p.add_argument("--torch_dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    p.add_argument("--num_samples", type=int, default=90)
    p.add_argument("--max_input_tokens", type=int, default=128)
    p.add_argument("--max_new_tokens", type=int, default=512)
    p.add_argument("--compression_ratio_list", type=float, nargs="+", default=[5.0, 2.0],
                   help="first value: merge compressor; last value: eviction methods")
    p.add_argument("--req_per_sec", type=float, default=10.0)
    p.add_argument("--fixed_spacing", action="store_true", help="arrivals every 1 / rate s instead of Poisson")
    p.add_argument("--no_log", action="store_true")
    p.add_argument("--gpu_info_path", default=None, help="CSV of sampled GPU utilisation / memory")
    p.add_argument("--engine", default="fastcache", choices=["fastcache", "hf"],
                   help="fastcache: this package's engine; hf: the three-stage pipeline over a HuggingFace causal LM "
                   "(text prompts of the dataset; without --model_path a tiny random Llama)")
    p.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    p.add_argument("--kv_blocks", type=int, default=0)
    p.add_argument("--block_size", type=int, default=256)
    p.add_argument("--max_model_len", type=int, default=2048)
    return p.parse_args(argv)


def batching_for(args: argparse.Namespace, exp: Experiment) -> List[int]:
    """[prefill, compress, decode] caps.  A YAML experiment carries its own list; a single MiniCPM run
    with the merge compressor and the default sizes uses the operational-intensity rule of the
    MiniCPM script (decode 135, compress = decode // 3, prefill = compress // 3)."""
    if exp.extra.get("from_yaml"):
        return list(exp.batching)
    sizes = [args.prefill_batch_size, args.compress_batch_size, args.decoding_batch_size]
    if args.model_mode == "minicpm" and exp.use_compression and exp.comp_mode.lower() == "ccm" \
            and sizes == [15, 45, 90]:
        return ConcurrentTester.ccm_intensity_rule(135)
    return sizes


def samples_for(args: argparse.Namespace, g: Dict[str, Any], model: Any, tokenizer: Any
                ) -> Tuple[List[Any], List[Any]]:
    n = int(g["num_samples"])
    if args.datasets_name == "synthetic":
        vis = getattr(model, "vision_config", None)
        side = int(getattr(vis, "image_size", 336)) if args.model_mode == "llava" else \
            int(getattr(model, "scale_resolution", 448))
        vocab = model.text_config.vocab_size
        got = synthetic_samples(n, (side, side), min(int(g["max_input_tokens"]), 64), min(vocab, 32000), int(g["seed"]))
    elif args.datasets_name == "gqa":
        got = load_image_data(args.datasets_js_path, args.datasets_img_path, n, seed=int(g["seed"]))
    else:
        got = load_image_data_milebench(args.datasets_img_path, n, seed=int(g["seed"]))
    image_id = int(model.image_token_id)
    prompts, images = [], []
    for s in got:
        if isinstance(s.prompt, str):
            if tokenizer is None:
                raise ValueError("text prompts need the checkpoint's tokenizer (--model_path)")
            ids = tokenizer.encode(s.prompt)[: int(g["max_input_tokens"])]
        else:
            ids = list(s.prompt)[: int(g["max_input_tokens"])]
        ids = [t for t in ids if t != image_id]
        prompts.append(ids[:1] + [image_id] + ids[1:] if s.image is not None else ids)
        images.append(s.image)
    return prompts, images


def build_engine(args: argparse.Namespace, exp: Experiment):
    from .. import LLM
    from .. import compress as compress_mod
    kw = dict(exp.engine_kwargs())
    arch = ARCHS[args.arch or DEFAULT_ARCH[args.model_mode]]
    model: Any = args.model_path or dict(arch)
    if kw.get("compression_backend") == "mlp":
        if args.ckpt_path:
            kw["compressor_path"] = args.ckpt_path
        else:                                   # seeded random compressor of the model's shape
            text = arch.get("text_config", arch)
            hd = text.get("head_dim") or text["hidden_size"] // text["num_attention_heads"]
            cls = compress_mod.KVCacheHybridCompressor if args.model_mode == "minicpm" else \
                compress_mod.KVCacheLinearDecoupleCompressor
            torch.manual_seed(0)
            comp = cls(None, kw["compression_factor"], 2, n_layer=text["num_hidden_layers"], nhead=2, head_dim=hd)
            for prm in comp.parameters():
                torch.nn.init.normal_(prm, std=0.02)
            kw["compressor"] = comp.eval()
    if args.kv_blocks > 0:
        kw["num_kvcache_blocks"] = args.kv_blocks
    dtype = {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32"}.get(args.torch_dtype, args.torch_dtype)
    cpu = args.device == "cpu"
    return LLM(model, device=args.device, dtype="auto" if cpu else dtype, kvcache_block_size=args.block_size,
               max_model_len=args.max_model_len, max_num_seqs=max(args.decoding_batch_size, 8), seed=args.seed,
               enforce_eager=cpu, prefix_caching=False, compression_pipeline="prefill", **kw)


def run_one_hf(args: argparse.Namespace, g: Dict[str, Any], exp: Experiment) -> Dict[str, Any]:
    """The same run through `serving/hf_pipeline.py`: HuggingFace model, KV pool, dynamic scheduler."""
    import transformers
    from ..compress.ccm import KVCacheLinearDecoupleCompressor, load_compressor
    from ..compress.kvpress_compat import create_kvpress_compressor
    from .hf_pipeline import HFPipelineTester, TransformersBackend
    if args.model_path:
        model = transformers.AutoModelForCausalLM.from_pretrained(args.model_path, trust_remote_code=True)
        tok = transformers.AutoTokenizer.from_pretrained(args.model_path, trust_remote_code=True)
    else:
        cfg = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                       num_attention_heads=4, num_key_value_heads=2, vocab_size=600,
                                       max_position_embeddings=2048)
        torch.manual_seed(args.seed)
        model, tok = transformers.LlamaForCausalLM(cfg), None
    model = model.eval().to(args.device)
    c = model.config
    kw = exp.engine_kwargs()
    comp = None
    if kw.get("compression_backend") == "mlp":
        if args.ckpt_path:
            comp = load_compressor(args.ckpt_path, compression_factor=kw["compression_factor"], min_seq_len=2)
        else:
            torch.manual_seed(0)
            hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
            comp = KVCacheLinearDecoupleCompressor(None, kw["compression_factor"], 2, n_layer=c.num_hidden_layers,
                                                   nhead=2, head_dim=hd)
        comp = comp.to(args.device).eval()
    elif kw.get("compression_backend") == "kvpress":
        comp = create_kvpress_compressor(kw["kvpress_method"], kw["compression_factor"])
    rng = torch.Generator().manual_seed(int(g["seed"]))
    n, length = int(g["num_samples"]), min(int(g["max_input_tokens"]), 64)
    if tok is None or args.datasets_name == "synthetic":
        prompts = [torch.randint(3, c.vocab_size, (length,), generator=rng).tolist() for _ in range(n)]
    else:
        got = load_image_data(args.datasets_js_path, args.datasets_img_path, n, seed=int(g["seed"]))
        prompts = [tok.encode(s_.prompt)[: int(g["max_input_tokens"])] for s_ in got]
    tester = HFPipelineTester(TransformersBackend(model), comp, batching_for(args, exp), float(g["req_per_sec"]),
                              pad_token_id=getattr(c, "pad_token_id", None) or 0, seed=int(g["seed"]),
                              monitor_gpu=bool(args.gpu_info_path))
    res = tester.run_concurrent_test(prompts, int(g["max_new_tokens"]), poisson=not args.fixed_spacing)
    if args.gpu_info_path and tester.monitor is not None:
        tester.monitor.save_stats(args.gpu_info_path)
    summary, _ = tester.timestamps.analyze_timestamps()
    return {"name": exp.name, "comp_mode": exp.comp_mode, "use_compression": exp.use_compression,
            "compression_ratio": exp.compression_ratio, "batching": batching_for(args, exp), "engine": "hf",
            "result": res.to_dict(), "stage_averages": summary["average_times"]}


def run_one(args: argparse.Namespace, g: Dict[str, Any], exp: Experiment) -> Dict[str, Any]:
    if getattr(args, "engine", "fastcache") == "hf":
        return run_one_hf(args, g, exp)
    llm = build_engine(args, exp)
    try:
        prompts, images = samples_for(args, g, llm.model_runner.model, llm.tokenizer)
        tester = ConcurrentTester(llm, batching_for(args, exp), float(g["req_per_sec"]),
                                  poisson=not args.fixed_spacing, seed=int(g["seed"]),
                                  monitor_gpu=bool(args.gpu_info_path))
        res = tester.run(prompts, int(g["max_new_tokens"]), images)
        if args.gpu_info_path and tester.monitor is not None:
            tester.monitor.to_csv(args.gpu_info_path)
        summary, _ = tester.timestamps.analyze_timestamps()
        return {"name": exp.name, "comp_mode": exp.comp_mode, "use_compression": exp.use_compression,
                "compression_ratio": exp.compression_ratio, "batching": batching_for(args, exp),
                "result": res.to_dict(), "stage_averages": summary["average_times"]}
    finally:
        llm.exit()


exec_testit = run_one          # the reference's name for "run one configuration"


def write_result(folder: str, row: Dict[str, Any]) -> str:
    """One text file per run, named for the run (the reference writes `.txt` summaries, :2056-2076)."""
    os.makedirs(folder, exist_ok=True)
    path = os.path.join(folder, f"{row['name']}_{time.strftime('%m%d_%H%M%S')}.txt")
    r = row.get("result", {})
    with open(path, "w") as fh:
        fh.write(f"run: {row['name']}  mode: {row['comp_mode']}  ratio: {row['compression_ratio']}  "
                 f"batching [prefill, compress, decode]: {row['batching']}\n")
        for key in ("num_requests", "completed", "failed", "wall_s", "output_tokens", "throughput_tok_s",
                    "request_rate"):
            fh.write(f"{key}: {r.get(key)}\n")
        for key in ("ttft", "tpot", "latency"):
            fh.write(f"{key}: " + "  ".join(f"{k}={v:.4f}" for k, v in (r.get(key) or {}).items()) + "\n")
        fh.write("compression: " + json.dumps(r.get("compression", {})) + "\n")
        fh.write("stage averages (s): " + json.dumps(row.get("stage_averages", {})) + "\n")
    return path


def main(argv: Optional[Sequence[str]] = None) -> List[Dict[str, Any]]:
    args = parse_args(argv)
    torch.manual_seed(args.seed)
    if args.config:
        g, exps = load_experiments(args.config, {"seed": args.seed})
        for e in exps:
            e.extra["from_yaml"] = True
        defaults = parse_args([])
        for key in ("model_path", "ckpt_path", "datasets_name", "datasets_js_path", "datasets_img_path",
                    "torch_dtype"):                  # file settings fill what the command line left at its default
            if key in g and getattr(args, key) == getattr(defaults, key):
                setattr(args, key, g[key])
    else:
        g = {"num_samples": args.num_samples, "req_per_sec": args.req_per_sec, "seed": args.seed,
             "max_input_tokens": args.max_input_tokens, "max_new_tokens": args.max_new_tokens}
        mode = args.comp_mode
        use = args.use_compression and mode.lower() not in ("orig", "none")
        ratio = args.compression_ratio_list[0] if mode.lower() == "ccm" else args.compression_ratio_list[-1]
        exps = [Experiment(f"{args.model_mode}_{mode}", use, mode, compression_ratio=float(ratio))]
    rows: List[Dict[str, Any]] = []
    for exp in exps:
        try:
            row = run_one(args, g, exp)
        except Exception as exc:                  # a failing run is recorded; the batch goes on
            row = {"name": exp.name, "comp_mode": exp.comp_mode, "compression_ratio": exp.compression_ratio,
                   "batching": list(exp.batching), "error": f"{type(exc).__name__}: {exc}"}
        rows.append(row)
        if not args.no_log:
            row["log"] = write_result(args.folder_path, row) if "error" not in row else None
        print(json.dumps({k: row.get(k) for k in ("name", "error")} |
                         {k: (row.get("result") or {}).get(k) for k in ("completed", "throughput_tok_s")}))
    if not args.no_log:
        os.makedirs(args.folder_path, exist_ok=True)
        with open(os.path.join(args.folder_path, "summary.json"), "w") as fh:
            json.dump(rows, fh, indent=1)
    return rows


if __name__ == "__main__":
    main()
