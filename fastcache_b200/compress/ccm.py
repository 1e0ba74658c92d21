"""CCM merge compressors: per-layer MLPs that fold f consecutive KV rows into one.

Parity (semantics and state-dict layout):
  * KVCacheLinearDecoupleCompressor  utils_ccm/module_ccm_v11.py:605-729
    four MLP banks per layer (text-K, text-V, image-K, image-V) + an unused
    `attention` Linear(D, 1) that is part of the saved state
  * KVCacheHybridCompressor          utils_ccm/module_ccm_v11.py:805-1060
    text-K / text-V banks only
  * MiniCPMKVCompressor              "kv-cache pipeline"/nanovllm/kernels/minicpm_compressor.py:17-230
    the four-bank layout under the MiniCPM config conventions
  * KVCacheLinearCompressor          utils_ccm/module_ccm_v11.py:525-603
    one K and one V bank, no image/text split
Each bank is Sequential(Linear(D*f, D), ReLU, Dropout, Linear(D, D), ReLU,
Dropout, Linear(D, D)), so parameters are named `<bank>.<layer>.{0,3,6}.*`.

Semantics of one segment (rows [a, b) of one request, one layer, K or V):
S' = (b-a)//f; if S' < min_seq_len the rows are returned unchanged, else row j
of the output is MLP(concat(rows a+j*f .. a+j*f+f-1)) for j < S', followed by
the (b-a) mod f remainder rows unchanged.  Weights are shared over heads and
batch.  The request's output is image-part followed by text-part.

`PackedCCMWeights` stacks all banks as [L, 4, ...] tensors in the layout the
fused in-pool kernel consumes; the nn.Module classes stay the source of truth
for checkpoints.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn

BANKS = ("tk", "tv", "ik", "iv")


def _mlp(d: int, f: int, p: float = 0.4) -> nn.Sequential:
    return nn.Sequential(nn.Linear(d * f, d), nn.ReLU(), nn.Dropout(p), nn.Linear(d, d), nn.ReLU(),
                         nn.Dropout(p), nn.Linear(d, d))


def _dims_from_config(cfg: Any) -> Tuple[int, int, int]:
    """(layers, kv_heads, head_dim) from an HF-style config (plain or with text_config / llm_config)."""
    for attr in ("text_config", "llm_config"):
        sub = getattr(cfg, attr, None)
        if sub is not None:
            cfg = sub
            break
    layers = cfg.num_hidden_layers
    heads = cfg.num_attention_heads
    kv_heads = getattr(cfg, "num_key_value_heads", None) or heads
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // heads
    return layers, kv_heads, head_dim


def ccm_segment_len(n: int, f: int, min_seq_len: int) -> int:
    if n <= 0:
        return 0
    s = n // f
    return n if s < min_seq_len else s + n % f


def ccm_output_len(total: int, image_len: int, f: int, min_seq_len: int = 1) -> int:
    """Rows left after compressing a request with `image_len` leading image rows."""
    image_len = max(0, min(image_len, total))
    return ccm_segment_len(image_len, f, min_seq_len) + ccm_segment_len(total - image_len, f, min_seq_len)


class _CCMBase(nn.Module):
    banks: Tuple[str, ...] = ()
    has_attention = False

    def __init__(self, src_config: Any = None, compression_factor: int = 2, min_seq_len: int = 1, *,
                 n_layer: Optional[int] = None, nhead: Optional[int] = None, head_dim: Optional[int] = None):
        super().__init__()
        if src_config is not None:
            n_layer, nhead, head_dim = _dims_from_config(src_config)
        if None in (n_layer, nhead, head_dim):
            raise ValueError("give src_config or n_layer/nhead/head_dim")
        self.n_layer, self.nhead, self.head_dim = int(n_layer), int(nhead), int(head_dim)
        self.compression_factor = int(compression_factor)
        self.min_seq_len = int(min_seq_len)
        for bank in self.banks:
            setattr(self, f"compress_{bank}", nn.ModuleList(
                _mlp(self.head_dim, self.compression_factor) for _ in range(self.n_layer)))
        if self.has_attention:
            self.attention = nn.ModuleList(nn.Linear(self.head_dim, 1) for _ in range(self.n_layer))
        self.eval()

    # ----------------------------------------------------------------- math
    def compress_segment(self, x: torch.Tensor, layer_idx: int, bank: str) -> torch.Tensor:
        """x: [B, H, S, D] -> [B, H, S_c, D] with the rule in the module docstring."""
        return self._merge(x, getattr(self, f"compress_{bank}")[layer_idx])

    def _merge(self, x: torch.Tensor, mlp: nn.Module) -> torch.Tensor:
        B, H, S, D = x.shape
        f = self.compression_factor
        s = S // f
        if S == 0 or s < self.min_seq_len:
            return x
        w = next(mlp.parameters())
        z = x[:, :, : s * f, :].reshape(B, H, s, D * f)
        y = mlp(z.to(w.dtype)).to(x.dtype)
        if S > s * f:
            y = torch.cat([y, x[:, :, s * f:, :]], dim=2)
        return y

    def _bank_for(self, segment: str, which: str) -> str:
        raise NotImplementedError

    def compress_layer(self, layer_cache: Tuple[torch.Tensor, torch.Tensor], layer_idx: int,
                       compressor_k: nn.ModuleList, compressor_v: nn.ModuleList
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
        """One segment of one layer through an explicit pair of banks, e.g.
        `m.compress_layer((k, v), l, m.compress_tk, m.compress_tv)` (utils_ccm/module_ccm_v11.py:666-694).
        `forward` and `compress_layer_kv` pick the banks from the image / text split themselves."""
        k, v = layer_cache
        return self._merge(k, compressor_k[layer_idx]), self._merge(v, compressor_v[layer_idx])

    def compress_layer_kv(self, k: torch.Tensor, v: torch.Tensor, layer_idx: int, image_len: int):
        outs = []
        for which, x in (("k", k), ("v", v)):
            img = self.compress_segment(x[:, :, :image_len, :], layer_idx, self._bank_for("image", which))
            txt = self.compress_segment(x[:, :, image_len:, :], layer_idx, self._bank_for("text", which))
            outs.append(torch.cat([img, txt], dim=2))
        return outs[0], outs[1]

    @torch.no_grad()
    def forward(self, kv_cache: Sequence[Tuple[torch.Tensor, torch.Tensor]], it_len: Sequence[int] = (0, 0),
                strategy_com: str = "retain") -> List[Tuple[torch.Tensor, torch.Tensor]]:
        """kv_cache: per layer (K, V) each [B, H, S, D]; it_len = [image_len, text_len]."""
        image_len = int(it_len[0]) if len(it_len) else 0
        out = []
        for layer_idx, (k, v) in enumerate(kv_cache):
            ck, cv = self.compress_layer_kv(k, v, layer_idx, image_len)
            out.append((ck.contiguous(), cv.contiguous()))
        return out

    def output_len(self, total: int, image_len: int) -> int:
        return ccm_output_len(total, image_len, self.compression_factor, self.min_seq_len)

    def pack(self, dtype: torch.dtype = torch.float32, device: Any = None) -> "PackedCCMWeights":
        return PackedCCMWeights.from_module(self, dtype, device)


class KVCacheLinearDecoupleCompressor(_CCMBase):
    banks = BANKS
    has_attention = True

    def _bank_for(self, segment, which):
        return ("i" if segment == "image" else "t") + which


class KVCacheHybridCompressor(_CCMBase):
    """Text banks only: image rows go through the text MLPs as well."""
    banks = ("tk", "tv")
    has_attention = False

    def _bank_for(self, segment, which):
        return "t" + which

    def compress_layer_kv(self, k, v, layer_idx, image_len):
        # one segment: the hybrid module treats the whole request as text when
        # there is no separate image bank (utils_ccm/module_ccm_v11.py:940-953)
        return (self.compress_segment(k, layer_idx, "tk"), self.compress_segment(v, layer_idx, "tv"))

    def output_len(self, total, image_len):
        return ccm_segment_len(total, self.compression_factor, self.min_seq_len)


class MiniCPMKVCompressor(KVCacheLinearDecoupleCompressor):
    """Four banks + attention so the shipped MiniCPM checkpoint loads strictly."""


class KVCacheLinearCompressor(_CCMBase):
    """One K bank and one V bank (`compress_k`, `compress_v`), no image/text split."""
    banks = ()

    def __init__(self, src_config=None, compression_factor=2, min_seq_len=8, **kw):
        super().__init__(src_config, compression_factor, min_seq_len, **kw)
        self.compress_k = nn.ModuleList(_mlp(self.head_dim, self.compression_factor)
                                        for _ in range(self.n_layer))
        self.compress_v = nn.ModuleList(_mlp(self.head_dim, self.compression_factor)
                                        for _ in range(self.n_layer))
        self.attention = nn.ModuleList(nn.Linear(self.head_dim, 1) for _ in range(self.n_layer))
        self.compress_tk, self.compress_tv = self.compress_k, self.compress_v
        self.eval()

    def _bank_for(self, segment, which):
        return "t" + which

    def compress_layer_kv(self, k, v, layer_idx, image_len):
        return (self.compress_segment(k, layer_idx, "tk"), self.compress_segment(v, layer_idx, "tv"))

    def output_len(self, total, image_len):
        return ccm_segment_len(total, self.compression_factor, self.min_seq_len)

    def state_dict(self, *a, **kw):
        sd = super().state_dict(*a, **kw)
        return {k: v for k, v in sd.items() if not k.startswith(("compress_tk.", "compress_tv."))}


class PackedCCMWeights:
    """All banks of all layers stacked for batched / fused execution.

    w1: [L, 4, D, D*f]   b1: [L, 4, D]
    w2: [L, 4, D, D]     b2: [L, 4, D]
    w3: [L, 4, D, D]     b3: [L, 4, D]
    bank order (tk, tv, ik, iv); a module without image banks repeats its text
    banks in the image slots.  Weights keep nn.Linear's [out, in] orientation,
    which is the K-major B operand of the tensor-core kernels.
    """

    def __init__(self, w1, b1, w2, b2, w3, b3, factor: int, min_seq_len: int, single_segment: bool):
        self.w1, self.b1, self.w2, self.b2, self.w3, self.b3 = w1, b1, w2, b2, w3, b3
        self.factor = factor
        self.min_seq_len = min_seq_len
        self.single_segment = single_segment

    @property
    def n_layer(self) -> int:
        return self.w1.shape[0]

    @property
    def head_dim(self) -> int:
        return self.w1.shape[2]

    @classmethod
    def from_module(cls, m: _CCMBase, dtype=torch.float32, device=None) -> "PackedCCMWeights":
        def bank(name):
            lst = getattr(m, f"compress_{name}", None)
            if lst is None:
                lst = getattr(m, "compress_t" + name[-1])
            return lst
        tensors: Dict[str, List[torch.Tensor]] = {k: [] for k in ("w1", "b1", "w2", "b2", "w3", "b3")}
        for l in range(m.n_layer):
            per = {k: [] for k in tensors}
            for name in BANKS:
                seq = bank(name)[l]
                for tag, idx in (("1", 0), ("2", 3), ("3", 6)):
                    per["w" + tag].append(seq[idx].weight.detach())
                    per["b" + tag].append(seq[idx].bias.detach())
            for k in tensors:
                tensors[k].append(torch.stack(per[k]))
        out = {k: torch.stack(v).to(dtype=dtype, device=device).contiguous() for k, v in tensors.items()}
        single = not isinstance(m, KVCacheLinearDecoupleCompressor)
        return cls(out["w1"], out["b1"], out["w2"], out["b2"], out["w3"], out["b3"],
                   m.compression_factor, m.min_seq_len, single)

    def to(self, device=None, dtype=None) -> "PackedCCMWeights":
        conv = lambda t: t.to(device=device, dtype=dtype)  # noqa: E731
        return PackedCCMWeights(conv(self.w1), conv(self.b1), conv(self.w2), conv(self.b2), conv(self.w3),
                                conv(self.b3), self.factor, self.min_seq_len, self.single_segment)

    def slice_layers(self, start: int, end: int) -> "PackedCCMWeights":
        s = slice(start, end)
        return PackedCCMWeights(self.w1[s], self.b1[s], self.w2[s], self.b2[s], self.w3[s], self.b3[s],
                                self.factor, self.min_seq_len, self.single_segment)

    def mlp(self, z: torch.Tensor, layer: int, bank: int) -> torch.Tensor:
        """Reference math on packed weights; z [..., D*f] -> [..., D] (fp32 accumulate)."""
        h = torch.relu(z.float() @ self.w1[layer, bank].float().T + self.b1[layer, bank].float())
        h = torch.relu(h @ self.w2[layer, bank].float().T + self.b2[layer, bank].float())
        return h @ self.w3[layer, bank].float().T + self.b3[layer, bank].float()


# ------------------------------------------------------------------ checkpoints
def _extract_state(obj: Any) -> Dict[str, torch.Tensor]:
    """Accept {'model_state_dict': {'compressor': sd}}, {'model_state_dict': sd} or a bare sd
    (scripts/finetune_llava.py:29-47; "kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:516-524)."""
    if isinstance(obj, dict) and "model_state_dict" in obj:
        obj = obj["model_state_dict"]
    if isinstance(obj, dict) and "compressor" in obj and isinstance(obj["compressor"], dict):
        obj = obj["compressor"]
    if not isinstance(obj, dict):
        raise ValueError("not a compressor checkpoint")
    return obj


def infer_layout(sd: Dict[str, torch.Tensor]) -> Dict[str, Any]:
    """Read layer count, head_dim, factor and bank set off a state dict."""
    bank = "compress_tk" if any(k.startswith("compress_tk.") for k in sd) else "compress_k"
    w0 = sd[f"{bank}.0.0.weight"]
    layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith(bank + "."))
    return {"n_layer": layers, "head_dim": w0.shape[0], "factor": w0.shape[1] // w0.shape[0],
            "decoupled": any(k.startswith("compress_ik.") for k in sd),
            "has_attention": any(k.startswith("attention.") for k in sd),
            "single_bank": bank == "compress_k"}


def load_compressor(path_or_state: Any, src_config: Any = None, compression_factor: Optional[int] = None,
                    min_seq_len: int = 1, nhead: int = 1, strict: bool = False,
                    kind: Optional[str] = None) -> _CCMBase:
    """Build the compressor class matching a `.pth` file (or state dict) and load it."""
    if isinstance(path_or_state, (str, os.PathLike)):
        obj = torch.load(path_or_state, map_location="cpu", weights_only=False)
    else:
        obj = path_or_state
    sd = _extract_state(obj)
    lay = infer_layout(sd)
    if compression_factor is not None and compression_factor != lay["factor"]:
        raise ValueError(f"checkpoint was trained for factor {lay['factor']}, asked for {compression_factor}")
    if kind is None:
        kind = "linear" if lay["single_bank"] else ("decouple" if lay["decoupled"] else "hybrid")
    cls = {"linear": KVCacheLinearCompressor, "decouple": KVCacheLinearDecoupleCompressor,
           "hybrid": KVCacheHybridCompressor, "minicpm": MiniCPMKVCompressor}[kind]
    if src_config is not None:
        L, H, D = _dims_from_config(src_config)
        if (L, D) != (lay["n_layer"], lay["head_dim"]):
            raise ValueError(f"checkpoint is for {lay['n_layer']} layers x head_dim {lay['head_dim']}, "
                             f"model has {L} x {D}")
        nhead = H
    m = cls(None, lay["factor"], min_seq_len, n_layer=lay["n_layer"], nhead=nhead, head_dim=lay["head_dim"])
    missing, unexpected = m.load_state_dict(sd, strict=False)
    missing = [k for k in missing if not k.startswith(("compress_tk.", "compress_tv.")) or kind != "linear"]
    if strict and (missing or unexpected):
        raise RuntimeError(f"missing {missing[:4]} unexpected {list(unexpected)[:4]}")
    return m


def load_minicpm_compressor(compressor_path: str, hf_config: Any, compression_factor: int = 5,
                            device: Any = None, dtype: Optional[torch.dtype] = None) -> "MiniCPMKVCompressor":
    """The full (tk / tv / ik / iv + attention) MiniCPM compressor with its `.pth` loaded strictly.

    Same job as "kv-cache pipeline"/nanovllm/kernels/minicpm_compressor.py:195-229; the device is the
    caller's choice here (the reference always moves to the current CUDA device), and a missing file
    is an error instead of a compressor with random weights."""
    if not os.path.exists(compressor_path):
        raise FileNotFoundError(f"compressor checkpoint not found: {compressor_path}")
    m = load_compressor(compressor_path, src_config=hf_config, compression_factor=compression_factor,
                        min_seq_len=2, kind="minicpm")
    if device is not None or dtype is not None:
        m = m.to(device=device, dtype=dtype)
    return m.eval()


def save_compressor(module: _CCMBase, path: str, epoch: int = 0, optimizer: Any = None, scheduler: Any = None,
                    loss: float = 0.0) -> None:
    """Write the training-script checkpoint layout (scripts/finetune_llava.py:29-47)."""
    torch.save({"epoch": epoch,
                "model_state_dict": {"compressor": module.state_dict()},
                "optimizer_state_dict": optimizer.state_dict() if optimizer is not None else {},
                "scheduler_state_dict": scheduler.state_dict() if scheduler is not None else {},
                "loss": loss}, path)
