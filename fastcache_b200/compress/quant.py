"""KV quantisers: per-row INT8 (symmetric / asymmetric), group-wise INT4 (packed two per
byte), FP8 casts and NF4 (nearest entry of the 16-value NormalFloat table).

Parity: nanovllm/autocompress/methods.py:636-757, nanovllm/autocompress/kernels.py:388-422,
utils_ccm/utils_compress.py:51-70, :144-154 (SimpleKVQuantizer / ImprovedKVQuantizer fake-quant).

bf16 tensors on a CUDA device go through the kernels of csrc/quant.cu (one warp per group, one pass, codes and
scales bit-identical to the statements below); everything else runs the PyTorch statements.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

NF4_TABLE = torch.tensor([-1.0, -0.6961928, -0.52507305, -0.39491749, -0.28444138, -0.18477343, -0.09105004, 0.0,
                          0.0795803, 0.1609302, 0.2461123, 0.33791524, 0.44070983, 0.562617, 0.72295684, 1.0])


def _groups(x: torch.Tensor, g: int):
    n = x.shape[-1]
    if n % g:
        g = n
    return x.reshape(*x.shape[:-1], n // g, g), g


_CUDA_MODES = {"int8": 0, "int8_asym": 1, "int4": 2, "nf4": 3, "fp8_e4m3": 4, "fp8_e5m2": 5}


def _cuda_group(x: torch.Tensor, mode: str, group_size: int) -> int:
    """Group size for the CUDA kernels (csrc/quant.cu), or 0 when `x` is not theirs to take: they work on
    contiguous bf16 rows whose groups are multiples of 8 values and at most 1024 long."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() >= 1 and x.numel() > 0):
        return 0
    n = x.shape[-1]
    g = n
    if mode in ("int4", "nf4"):
        g = group_size if n % group_size == 0 else n
    return g if (g % 8 == 0 and g <= 1024 and n % 2 == 0) else 0


def quantize(x: torch.Tensor, mode: str = "int8", group_size: int = 128) -> Dict[str, Any]:
    g = _cuda_group(x, mode, group_size) if mode in _CUDA_MODES else 0
    if g:
        from ..ops.loader import ext
        q, scale, zero = ext().quantize_rows(x.contiguous(), _CUDA_MODES[mode], g)
        meta = {"mode": mode, "shape": tuple(x.shape), "dtype": x.dtype, "scale": scale}
        if mode in ("int4", "nf4"):
            meta.update(q=q, group=g)
        else:
            meta["scale"] = scale.reshape(*x.shape[:-1], 1)
            meta["q"] = q.view({"int8": torch.int8, "int8_asym": torch.uint8, "fp8_e4m3": torch.float8_e4m3fn,
                                "fp8_e5m2": torch.float8_e5m2}[mode])
            if mode == "int8_asym":
                meta["zero"] = zero.reshape(*x.shape[:-1], 1)
        return meta
    xf = x.float()
    meta: Dict[str, Any] = {"mode": mode, "shape": tuple(x.shape), "dtype": x.dtype}
    if mode == "int8":
        scale = xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / 127.0
        meta.update(q=torch.round(xf / scale).clamp(-127, 127).to(torch.int8), scale=scale)
    elif mode == "int8_asym":
        lo, hi = xf.amin(dim=-1, keepdim=True), xf.amax(dim=-1, keepdim=True)
        scale = ((hi - lo) / 255.0).clamp_min(1e-8)
        meta.update(q=torch.round((xf - lo) / scale).clamp(0, 255).to(torch.uint8), scale=scale, zero=lo)
    elif mode in ("int4", "nf4"):
        xg, g = _groups(xf, group_size)
        absmax = xg.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8)
        if mode == "int4":
            q = (torch.round(xg / absmax * 7.0).clamp(-8, 7) + 8).to(torch.uint8)
        else:
            table = NF4_TABLE.to(xg.device)
            q = (xg / absmax).unsqueeze(-1).sub(table).abs().argmin(dim=-1).to(torch.uint8)
        q = q.reshape(*q.shape[:-2], -1)
        if q.shape[-1] % 2:
            q = torch.cat([q, torch.zeros_like(q[..., :1])], dim=-1)
        meta.update(q=(q[..., 0::2] | (q[..., 1::2] << 4)), scale=absmax, group=g)
    elif mode in ("fp8_e4m3", "fp8_e5m2"):
        dt = torch.float8_e4m3fn if mode == "fp8_e4m3" else torch.float8_e5m2
        amax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8)
        scale = amax / (448.0 if mode == "fp8_e4m3" else 57344.0)
        meta.update(q=(xf / scale).to(dt), scale=scale)
    else:
        raise ValueError(mode)
    return meta


def dequantize(p: Dict[str, Any]) -> torch.Tensor:
    mode = p["mode"]
    q = p["q"]
    if q.is_cuda and p["dtype"] == torch.bfloat16 and mode in _CUDA_MODES and q.is_contiguous():
        n = p["shape"][-1]
        g = p.get("group", n)
        if g % 8 == 0 and n % 2 == 0 and p["scale"].dtype == torch.float32:
            from ..ops.loader import ext
            y = ext().dequantize_rows(q.view(torch.uint8), p["scale"].contiguous(),
                                      p["zero"].contiguous() if mode == "int8_asym" else None,
                                      _CUDA_MODES[mode], g)
            return y.reshape(p["shape"])
    if mode == "int8":
        y = p["q"].float() * p["scale"]
    elif mode == "int8_asym":
        y = p["q"].float() * p["scale"] + p["zero"]
    elif mode in ("int4", "nf4"):
        q = p["q"]
        lo, hi = (q & 0xF), (q >> 4)
        u = torch.stack([lo, hi], dim=-1).reshape(*q.shape[:-1], -1)
        n = p["shape"][-1]
        u = u[..., :n]
        g = p["group"]
        ug = u.reshape(*u.shape[:-1], n // g, g)
        if mode == "int4":
            y = (ug.float() - 8.0) / 7.0 * p["scale"]
        else:
            y = NF4_TABLE.to(q.device)[ug.long()] * p["scale"]
        y = y.reshape(p["shape"])
    elif mode in ("fp8_e4m3", "fp8_e5m2"):
        y = p["q"].float() * p["scale"]
    else:
        raise ValueError(mode)
    return y.reshape(p["shape"]).to(p["dtype"])


def fake_quantize(x: torch.Tensor, nbits: int = 4, group_size: int = 128) -> torch.Tensor:
    """Quantise and immediately restore (the HF harness' SimpleKVQuantizer behaviour)."""
    mode = {8: "int8", 4: "int4"}.get(nbits)
    if mode is None:
        raise ValueError("nbits must be 4 or 8")
    g = _cuda_group(x, mode, group_size)
    if g:                                # one pass on the device: no codes are written
        from ..ops.loader import ext
        return ext().fake_quantize_rows(x.contiguous(), _CUDA_MODES[mode], g)
    return dequantize(quantize(x, mode, group_size))


class SimpleKVQuantizer:
    """Quantise-and-restore of a whole cache (utils_ccm/utils_compress.py:118-164).  Called with a
    cache it returns the restored cache; `totalTime` accumulates seconds like the timed presses."""

    def __init__(self, nbits: int = 4, group_size: int = 128):
        self.nbits, self.group_size = nbits, group_size
        self.totalTime = 0.0

    def reset_timeCheck(self) -> None:
        self.totalTime = 0.0

    def quantize_cache(self, past_key_values):
        import time
        t0 = time.perf_counter()
        out = tuple((fake_quantize(k, self.nbits, self.group_size), fake_quantize(v, self.nbits, self.group_size))
                    for k, v in past_key_values)
        if out and out[0][0].is_cuda:
            torch.cuda.synchronize(out[0][0].device)
        self.totalTime += time.perf_counter() - t0
        return out

    def __call__(self, kv_cache):
        return list(self.quantize_cache(kv_cache))


class ImprovedKVQuantizer(SimpleKVQuantizer):
    """Per-row absmax variant that keeps its scales (utils_ccm/utils_compress.py:27-116):
    `quantize_cache` returns integer codes and remembers one scale per row and tensor,
    `dequantize_cache` restores the values from them."""

    def __init__(self, nbits: int = 4):
        super().__init__(nbits)
        self.cache: Dict[str, Dict[str, torch.Tensor]] = {}

    def _codes(self, x: torch.Tensor, key: str) -> torch.Tensor:
        qmax = 2 ** (self.nbits - 1) - 1
        max_val = x.abs().amax(dim=-1, keepdim=True)
        scale = (max_val / qmax).clamp_min(torch.finfo(torch.float32).tiny)
        self.cache[key] = {"scale": scale, "max_val": max_val}
        return torch.round(x / scale).clamp(-qmax - 1, qmax).to(torch.int8)

    def quantize_cache(self, past_key_values):
        return tuple((self._codes(k, f"k_{i}"), self._codes(v, f"v_{i}"))
                     for i, (k, v) in enumerate(past_key_values))

    def dequantize_cache(self, quantized_cache):
        out = []
        for i, (k, v) in enumerate(quantized_cache):
            sk, sv = self.cache[f"k_{i}"]["scale"], self.cache[f"v_{i}"]["scale"]
            out.append((k.to(sk.dtype) * sk, v.to(sv.dtype) * sv))
        return tuple(out)

    def __call__(self, kv_cache):
        return list(self.dequantize_cache(self.quantize_cache(kv_cache)))


class BaseCompressionMethod:
    """`with method(model) as m:` frame that the harness wraps around generation
    (utils_ccm/utils_compress.py:96-116): the base does nothing to the model."""

    def __init__(self, compression_ratio: float = 0.5):
        self.compression_ratio = compression_ratio

    def __call__(self, model):
        return self.CompressionContext(model, self.compression_ratio)

    class CompressionContext:
        def __init__(self, model, compression_ratio: float):
            self.model, self.compression_ratio = model, compression_ratio

        def __enter__(self):
            return self.model

        def __exit__(self, exc_type, exc, tb):
            return False


class QuantizedCacheWrapper:
    """`with QuantizedCacheWrapper(nbits)(model) as m:` switches a HuggingFace model's generation
    cache to its quantised implementation for the block and restores the config afterwards
    (reference: utils_ccm/utils_compress.py:166-197).  `backend` is the HF cache backend name; the
    reference fixes it to "quanto"."""

    def __init__(self, nbits: int = 4, backend: str = "quanto"):
        self.nbits, self.backend = nbits, backend

    def __call__(self, model):
        return self.QuantizedContext(model, self.nbits, self.backend)

    class QuantizedContext:
        _UNSET = object()

        def __init__(self, model, nbits: int, backend: str = "quanto"):
            self.model, self.nbits, self.backend = model, nbits, backend
            self._saved = {}

        def __enter__(self):
            cfg = self.model.config
            for name in ("cache_implementation", "cache_config"):
                self._saved[name] = getattr(cfg, name, self._UNSET)
            cfg.cache_implementation = "quantized"
            cfg.cache_config = {"backend": self.backend, "nbits": self.nbits}
            return self.model

        def __exit__(self, exc_type, exc, tb):
            cfg = self.model.config
            for name, old in self._saved.items():
                if old is self._UNSET:
                    if hasattr(cfg, name):
                        delattr(cfg, name)
                else:
                    setattr(cfg, name, old)
            return False
