"""RMSNorm and LayerNorm modules (reference: nanovllm/layers/layernorm.py:5-51)."""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size), requires_grad=False)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None
                ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        if residual is None:
            return ops.rms_norm(x, self.weight, self.eps)
        return ops.add_rms_norm(x, residual, self.weight, self.eps)

    # the two halves of `forward` under the reference's names (nanovllm/layers/layernorm.py:17-41)
    def rms_forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)

    def add_rms_forward(self, x: torch.Tensor, residual: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.add_rms_norm(x, residual, self.weight, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(hidden_size), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)
