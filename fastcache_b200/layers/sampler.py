"""Token sampler (reference: nanovllm/layers/sampler.py:5-17).

Greedy for temperature 0, otherwise an exponential-race (Gumbel-max) draw
from the tempered softmax.  Under tensor parallelism every rank draws with the
same seed and step counter: from gathered logits (CPU ranks, library path), or
from its own vocabulary shard with an exchange of one candidate per rank
(`forward_sharded`, CUDA ranks); either way all ranks obtain the same tokens
without a broadcast (the reference samples on rank 0 and broadcasts,
"kv-cache pipeline"/nanovllm/engine/llava_model_runner.py:1058-1066).
"""
import torch
from torch import nn

from .. import ops


class Sampler(nn.Module):
    def __init__(self, seed: int = 0):
        super().__init__()
        self.seed = seed
        self.step = 0

    def _next_seed(self) -> int:
        self.step += 1
        return self.seed * 1000003 + self.step

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor, noise=None,
                with_status: bool = False) -> torch.Tensor:
        return ops.sample(logits, temperatures, noise, seed=self._next_seed(), with_status=with_status)

    def forward_sharded(self, local_logits: torch.Tensor, temperatures: torch.Tensor, comm, vocab_offset: int,
                        vocab_size: int) -> torch.Tensor:
        """Draw from vocabulary-sharded logits without gathering them: every rank finds the best candidate of
        its shard, the candidates are exchanged through symmetric memory inside the same kernel, and every rank
        returns the same [B] tokens followed by its device status code.  The noise depends on the global
        vocabulary index, so the draw equals the one a single GPU would make."""
        return comm.sample(local_logits, temperatures, self._next_seed(), vocab_offset, vocab_size)
