"""Batch experiments from a YAML file (reference: configs/experiments.yaml:1-38 and the loader in
scripts/llava_testcon2.6.py:2394-2419): `global_settings` plus a list of
`experiments[{name, use_compression, comp_mode, batching}]`; command-line values override the
global settings."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

DEFAULT_GLOBAL = {"num_samples": 90, "req_per_sec": 10.0, "max_input_tokens": 128, "max_new_tokens": 512,
                  "torch_dtype": "bf16", "compression_ratio_list": [5.0, 2.0], "seed": 42}


@dataclass
class Experiment:
    name: str
    use_compression: bool = False
    comp_mode: str = "ccm"              # ccm | Knorm | SnapKV | ExpectedAttention | StreamingLLM | Random | none
    batching: List[int] = field(default_factory=lambda: [15, 45, 90])
    compression_ratio: float = 5.0
    extra: Dict[str, Any] = field(default_factory=dict)

    def engine_kwargs(self) -> Dict[str, Any]:
        """Constructor arguments of the engine for this experiment."""
        if not self.use_compression or self.comp_mode.lower() in ("none", "orig"):
            return {"enable_compression": False}
        mode = self.comp_mode.lower()
        if mode == "ccm":
            return {"enable_compression": True, "compression_backend": "mlp",
                    "compression_factor": int(round(self.compression_ratio))}
        method = {"knorm": "knorm", "snapkv": "snapkv", "expectedattention": "expected_attention",
                  "streamingllm": "streaming_llm", "random": "random", "tova": "tova"}.get(mode, mode)
        return {"enable_compression": True, "compression_backend": "kvpress", "kvpress_method": method,
                "compression_factor": max(1, int(round(self.compression_ratio)))}


def load_experiments(path: str, overrides: Optional[Dict[str, Any]] = None):
    """Returns (global_settings, [Experiment])."""
    import yaml
    with open(path) as fh:
        doc = yaml.safe_load(fh) or {}
    g = dict(DEFAULT_GLOBAL)
    g.update(doc.get("global_settings", {}) or {})
    g.update({k: v for k, v in (overrides or {}).items() if v is not None})
    ratios = g.get("compression_ratio_list", [5.0, 2.0])
    exps = []
    for e in doc.get("experiments", []) or []:
        mode = str(e.get("comp_mode", "ccm"))
        ratio = e.get("compression_ratio", ratios[0] if mode.lower() == "ccm" else ratios[-1])
        known = {"name", "use_compression", "comp_mode", "batching", "compression_ratio"}
        exps.append(Experiment(str(e.get("name", mode)), bool(e.get("use_compression", False)), mode,
                               list(e.get("batching", [15, 45, 90])), float(ratio),
                               {k: v for k, v in e.items() if k not in known}))
    return g, exps


def run_experiments(path: str, make_engine, make_prompts, out_path: Optional[str] = None,
                    overrides: Optional[Dict[str, Any]] = None, resume: bool = False) -> List[Dict[str, Any]]:
    """Runs every experiment with the concurrent tester.  `make_engine(**kwargs)` builds an engine,
    `make_prompts(global_settings)` returns (prompts, images or None).  With `resume`, experiments whose
    name already has a result in `out_path` are skipped (reference: the bench matrix' --resume)."""
    from .harness import ConcurrentTester
    g, exps = load_experiments(path, overrides)
    done: List[Dict[str, Any]] = []
    if resume and out_path and os.path.exists(out_path):
        done = json.load(open(out_path))
    have = {d["name"] for d in done}
    for e in exps:
        if e.name in have:
            continue
        try:
            llm = make_engine(**e.engine_kwargs())
            prompts, images = make_prompts(g)
            res = ConcurrentTester(llm, e.batching, float(g["req_per_sec"]), seed=int(g.get("seed", 0))).run(
                prompts, int(g["max_new_tokens"]), images)
            done.append({"name": e.name, "result": res.to_dict()})
            llm.exit()
        except Exception as exc:                      # one failing variant must not end the matrix
            done.append({"name": e.name, "error": f"{type(exc).__name__}: {exc}"})
        if out_path:
            with open(out_path, "w") as fh:
                json.dump(done, fh, indent=1)
    return done
