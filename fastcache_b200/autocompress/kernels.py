"""Kernel accessors of the planning package.

The reference generates kernels at run time from TileLang / Triton templates with
PyTorch fallbacks (nanovllm/autocompress/kernels.py:66-455).  Here the kernels are
compiled ahead of time for sm_100a, so the "generator" only hands out callables: the
CUDA kernel for CUDA tensors and the PyTorch statement otherwise.  The class and
function names are kept for callers written against the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Tuple

import torch

from .. import ops
from ..compress import quant


@dataclass
class KernelConfig:
    block_m: int = 128
    block_n: int = 128
    block_k: int = 64
    num_stages: int = 4
    dtype: str = "bfloat16"


def _mlp3(x, w1, b1, w2, b2, w3, b3):
    """relu(relu(x W1^T + b1) W2^T + b2) W3^T + b3 with [out, in] weights."""
    h = ops.linear(x, w1, b1, "relu")
    h = ops.linear(h, w2, b2, "relu")
    return ops.linear(h, w3, b3)


def _sparse_gather(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return x.index_select(0, idx.long())


class TileLangKernelGenerator:
    def __init__(self, config: KernelConfig | None = None):
        self.config = config or KernelConfig()

    def get_mlp_kernel(self) -> Callable:
        return _mlp3

    def get_sparse_gather_kernel(self) -> Callable:
        return _sparse_gather

    def get_quantize_kernels(self) -> Tuple[Callable, Callable]:
        return quant.quantize, quant.dequantize

    # `generate_*` names of the reference (kernels.py:99-422): nothing is generated at run time here,
    # each returns the same ahead-of-time kernel as the `get_*` accessor
    def generate_mlp_compress_kernel(self, *shape_hints, **kw) -> Callable:
        return self.get_mlp_kernel()

    def generate_sparse_gather_kernel(self, *shape_hints, **kw) -> Callable:
        return self.get_sparse_gather_kernel()

    def generate_quantize_kernel(self, bits: int = 8, group_size: int = 128, **kw) -> Callable:
        mode = {8: "int8", 4: "int4"}[bits]
        return lambda x: quant.quantize(x, mode, group_size)

    def generate_dequantize_kernel(self, bits: int = 8, **kw) -> Callable:
        return quant.dequantize


_GEN = None


def get_kernel_generator(config: KernelConfig | None = None) -> TileLangKernelGenerator:
    global _GEN
    if _GEN is None or config is not None:
        _GEN = TileLangKernelGenerator(config)
    return _GEN


def get_mlp_kernel() -> Callable:
    return get_kernel_generator().get_mlp_kernel()


def get_sparse_gather_kernel() -> Callable:
    return get_kernel_generator().get_sparse_gather_kernel()


def get_quantize_kernels():
    return get_kernel_generator().get_quantize_kernels()
