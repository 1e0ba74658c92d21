"""Token sampler (reference: nanovllm/layers/sampler.py:5-17).

Greedy for temperature 0, otherwise an exponential-race (Gumbel-max) draw
from the tempered softmax.  Under tensor parallelism the logits passed in are
already gathered over the vocabulary shards, and every rank draws with the
same seed and step counter, so all ranks obtain the same tokens without a
broadcast.
"""
import torch
from torch import nn

from .. import ops


class Sampler(nn.Module):
    def __init__(self, seed: int = 0):
        super().__init__()
        self.seed = seed
        self.step = 0

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor, noise=None) -> torch.Tensor:
        self.step += 1
        return ops.sample(logits, temperatures, noise, seed=self.seed * 1000003 + self.step)
