"""tcgen05 GEMM entry point for CUDA tensors."""
from __future__ import annotations

from typing import Optional

import torch

from .loader import ext

_ACT = {"none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "quick_gelu": 4, "silu": 5}


def gemm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x @ weight.T + bias) for bf16 CUDA tensors; x may have leading batch dims."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if act == "swiglu":
        if x2.shape[0] > 256 and weight.shape[0] % 256 == 0 and bias is None:
            y = ext().gemm(x2, weight, None, 6, None)        # SwiGLU applied in the GEMM epilogue
        else:
            y = ext().gemm(x2, weight, bias, 0, None)
            y = ext().silu_and_mul(y)
    else:
        y = ext().gemm(x2, weight, bias, _ACT[act], out.reshape(-1, weight.shape[0]) if out is not None else None)
    return y.reshape(*lead, y.shape[-1])
