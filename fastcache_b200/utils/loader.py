"""Weight loading from HuggingFace safetensors directories.

Parity: nanovllm/utils/loader.py:12-62 — walk every `*.safetensors` file, map
checkpoint names onto packed parameters through the model's
`packed_modules_mapping` (q/k/v -> qkv_proj, gate/up -> gate_up_proj) and call
each parameter's `weight_loader`.  Also here: `save_random_checkpoint`, which
writes a seeded random-init model in the same layout for benchmarks that have
no access to real weights.
"""
from __future__ import annotations

import json
import os
from glob import glob
from typing import Dict, Iterable, Optional, Tuple

import torch
from torch import nn


def default_weight_loader(param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
    if param.data.shape != loaded.shape:
        raise ValueError(f"shape mismatch {tuple(param.data.shape)} vs {tuple(loaded.shape)}")
    param.data.copy_(loaded)


def _resolve(model: nn.Module, name: str, prefix_map: Dict[str, str]) -> Optional[str]:
    for src, dst in prefix_map.items():
        if name.startswith(src):
            return dst + name[len(src):]
    return name


def load_weights(model: nn.Module, named_tensors: Iterable[Tuple[str, torch.Tensor]],
                 strip_prefix: str = "", verbose: bool = False) -> Dict[str, int]:
    """Feed (name, tensor) pairs into `model`.  Returns counters."""
    packed = getattr(model, "packed_modules_mapping", {})
    prefix_map = getattr(model, "checkpoint_prefix_map", {})
    skip = tuple(getattr(model, "skip_weight_substrings", ()))
    params = dict(model.named_parameters())
    buffers = dict(model.named_buffers())
    stats = {"loaded": 0, "skipped": 0, "unknown": 0}
    seen = set()                      # (parameter name, shard id) pairs that received data
    for name, tensor in named_tensors:
        if strip_prefix:
            if not name.startswith(strip_prefix):
                stats["skipped"] += 1
                continue
            name = name[len(strip_prefix):]
        if any(s in name for s in skip):
            stats["skipped"] += 1
            continue
        name = _resolve(model, name, prefix_map)
        target, shard_id = name, None
        for key, (packed_name, sid) in packed.items():
            if f".{key}." in name or name.startswith(key + "."):
                target = name.replace(key, packed_name)
                shard_id = sid
                break
        if target not in params and name in params:
            # the name only looks packed: the vision towers keep separate q / k / v projections under the same
            # leaf names that the language model packs
            target, shard_id = name, None
        param = params.get(target)
        if param is None:
            if target in buffers:
                buffers[target].copy_(tensor)
                stats["loaded"] += 1
                continue
            stats["unknown"] += 1
            if verbose:
                print(f"[loader] no parameter for checkpoint tensor {name}")
            continue
        loader = getattr(param, "weight_loader", default_weight_loader)
        with torch.no_grad():
            loader(param, tensor.to(param.device) if tensor.device != param.device else tensor, shard_id)
        stats["loaded"] += 1
        seen.add((target, shard_id))
    stats["missing"] = missing_parameters(model, seen)
    return stats


def missing_parameters(model: nn.Module, seen) -> list:
    """Parameters of `model` that no checkpoint tensor reached: a plain parameter needs its own tensor, a packed
    one (qkv_proj, gate_up_proj) every shard of its group.  Tied parameters (the LM head sharing the embedding
    table) count once.  Modules listed in `model.optional_weight_substrings` may stay at their initial values."""
    packed = getattr(model, "packed_modules_mapping", {})
    optional = tuple(o for m in model.modules() for o in getattr(m, "optional_weight_substrings", ()))
    groups: Dict[str, set] = {}
    for _key, (packed_name, sid) in packed.items():
        groups.setdefault(packed_name, set()).add(sid)
    got: Dict[str, set] = {}
    for target, sid in seen:
        got.setdefault(target, set()).add(sid)
    by_id: Dict[int, list] = {}
    for name, prm in model.named_parameters(remove_duplicate=False):
        by_id.setdefault(id(prm), []).append(name)
    missing = []
    for names in by_id.values():
        if any(o in n for n in names for o in optional):
            continue
        ok = False
        for n in names:
            sids = got.get(n)
            if not sids:
                continue
            need = next((g for pk, g in groups.items() if f".{pk}." in n or n.startswith(pk + ".")), None)
            if need is None or None in sids or need <= sids:
                ok = True
                break
        if not ok:
            missing.append(names[0])
    return sorted(missing)


def iter_safetensors(path: str) -> Iterable[Tuple[str, torch.Tensor]]:
    from safetensors import safe_open
    for file in sorted(glob(os.path.join(path, "*.safetensors"))):
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                yield name, f.get_tensor(name)


def load_model(model: nn.Module, path: str, strip_prefix: str = "", verbose: bool = False,
               strict: bool = True) -> Dict[str, int]:
    """Load every `*.safetensors` file of `path`.  With `strict` (default) a parameter that no checkpoint tensor
    reached is an error: a checkpoint with another naming prefix or a missing shard file would otherwise leave
    part of the model at its initial values without a word."""
    if not glob(os.path.join(path, "*.safetensors")):
        raise FileNotFoundError(f"no *.safetensors files in {path!r}")
    stats = load_weights(model, iter_safetensors(path), strip_prefix, verbose)
    if stats["missing"]:
        head = ", ".join(stats["missing"][:8]) + (" ..." if len(stats["missing"]) > 8 else "")
        msg = (f"{len(stats['missing'])} parameters were not found in {path!r} ({stats['unknown']} checkpoint "
               f"tensors matched no parameter): {head}")
        if strict:
            raise RuntimeError(msg)
        print(f"[fastcache_b200] warning: {msg}")
    if hasattr(model, "finalize_weights"):
        model.finalize_weights()
    return stats


def random_named_tensors(shapes: Dict[str, Tuple[int, ...]], seed: int = 0, std: float = 0.02,
                         dtype: torch.dtype = torch.float32, device: str = "cpu"
                         ) -> Iterable[Tuple[str, torch.Tensor]]:
    """Seeded random tensors in checkpoint layout: (name, full tensor) pairs.

    Every tensor is drawn from a generator seeded by (seed, crc32(name)), on
    the given device, at its *full* HuggingFace shape.  Feeding the pairs
    through `load_weights` therefore gives every tensor-parallel rank the
    shard of one and the same model, whatever the TP degree.  1-D tensors whose
    name contains "norm" / "ln" and ends in "weight" are set to one.
    """
    import zlib
    for name, shape in shapes.items():
        leaf = name.rsplit(".", 2)
        is_norm_w = name.endswith("weight") and len(shape) == 1 and any(
            k in name for k in ("norm", "layernorm", "ln_", ".ln", "layer_norm"))
        if is_norm_w:
            yield name, torch.ones(shape, dtype=dtype, device=device)
            continue
        g = torch.Generator(device=device)
        g.manual_seed((zlib.crc32(name.encode()) ^ (seed * 2654435761)) & 0x7FFFFFFFFFFF)
        t = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
        yield name, t.to(dtype)


def init_random_weights(model: nn.Module, shapes: Dict[str, Tuple[int, ...]], seed: int = 0,
                        std: float = 0.02, device: str = "cpu") -> Dict[str, int]:
    """Random-init `model` through its checkpoint loaders (see random_named_tensors)."""
    dtype = next(model.parameters()).dtype
    stats = load_weights(model, random_named_tensors(shapes, seed, std, dtype, device))
    if hasattr(model, "finalize_weights"):
        model.finalize_weights()
    return stats


def save_random_checkpoint(path: str, hf_config: dict, state: Dict[str, torch.Tensor]) -> None:
    """Write `config.json` + one safetensors file in HuggingFace layout."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(hf_config, fh, indent=1)
    save_file({k: v.contiguous() for k, v in state.items()}, os.path.join(path, "model.safetensors"))
