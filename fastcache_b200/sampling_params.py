"""Per-request sampling knobs (reference: nanovllm/sampling_params.py:4-8)."""
from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False
    # accepted for schema compatibility with the HTTP layer; the sampler is
    # temperature-only like the reference's (nanovllm/layers/sampler.py:10-17)
    top_p: float = 1.0

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
