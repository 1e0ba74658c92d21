"""Streams for overlapping compression with the model: green contexts or priorities.

Parity: "kv-cache pipeline"/nanovllm/utils/streams.py:17-123 (`build_streams`,
`StreamPool`, `try_create_greenctx_streams`).  A green context gives the
compression stream its own SM group (e.g. 36 of 148) so compression GEMMs run
beside memory-bound decode without competing for the same SMs; when the driver
refuses (or on request) the pool falls back to plain streams with the
compression stream at lower priority, as the reference does.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


@dataclass
class GreenCtxInfo:
    """Whether green contexts could be set up, and why not (reference streams.py:12-14)."""
    available: bool
    reason: Optional[str] = None


@dataclass
class StreamPool:
    main: Any
    compress: List[Any]
    greenctx: bool = False
    info: Dict[str, Any] = field(default_factory=dict)
    _next: int = 0

    @property
    def streams(self) -> List[Any]:
        return list(self.compress)

    def next_stream(self) -> Any:
        """Compression streams in round-robin order; the current stream when there is none."""
        if not self.compress:
            return torch.cuda.current_stream() if torch.cuda.is_available() else None
        s = self.compress[self._next % len(self.compress)]
        self._next = (self._next + 1) % len(self.compress)
        return s

    @property
    def greenctx_info(self) -> GreenCtxInfo:
        if self.greenctx:
            return GreenCtxInfo(True)
        return GreenCtxInfo(False, str(self.info.get("fallback", "not requested")))


# (device index, compression SMs asked for) -> partition.  A controller that moves the split up and down
# asks for the same few splits again and again; each is created once and lives until the process ends
# (green contexts are not freed while their streams may still be referenced by captured graphs).
_PARTITIONS: Dict[Any, Dict[str, Any]] = {}


def try_create_greenctx_streams(device: torch.device, compress_ratio: float, n_compress: int = 1
                                ) -> Optional[Dict[str, Any]]:
    """Returns {"main", "compress": [...], "main_sms", "compress_sms"} or None."""
    from ..ops.loader import ext, ext_available
    if not ext_available():
        return None
    index = device.index if device.index is not None else torch.cuda.current_device()
    try:
        total = ext().sm_count(index)
        want = max(1, int(round(total * compress_ratio)))
        cached = _PARTITIONS.get((index, want))
        if cached is not None:
            while len(cached["compress"]) < n_compress:
                extra = torch.cuda.ExternalStream(
                    ext().greenctx_extra_stream(cached["compress"][0].cuda_stream, 0), device=device)
                ext().register_stream_sms(extra.cuda_stream, cached["compress_sms"])
                cached["compress"].append(extra)
            return dict(cached, compress=cached["compress"][:n_compress])
        got = ext().greenctx_create(index, want, 0, 0)
        main = torch.cuda.ExternalStream(got["main_stream"], device=device)
        comp = [torch.cuda.ExternalStream(got["compress_stream"], device=device)]
        for _ in range(n_compress - 1):
            comp.append(torch.cuda.ExternalStream(
                ext().greenctx_extra_stream(got["compress_stream"], 0), device=device))
        ext().register_stream_sms(got["main_stream"], got["main_sms"])
        for s in comp:
            ext().register_stream_sms(s.cuda_stream, got["compress_sms"])
        part = {"main": main, "compress": comp, "main_sms": got["main_sms"],
                "compress_sms": got["compress_sms"], "total_sms": got["total_sms"]}
        _PARTITIONS[(index, want)] = part
        return dict(part, compress=list(comp))
    except Exception as exc:                      # driver too old, MIG, resources exhausted ...
        print(f"[fastcache_b200] green contexts unavailable ({exc}); using stream priorities")
        return None


def build_streams(device: torch.device, n_compress: int = 1, use_greenctx: bool = False,
                  compress_ratio: float = 0.25, main_on_greenctx: bool = False,
                  reuse_main: Any = None) -> StreamPool:
    """Main stream + `n_compress` compression streams.

    With green contexts the compression streams own `compress_ratio` of the SMs.
    The main stream moves to the complementary SM group only when
    `main_on_greenctx` is set (CUDA graphs captured on it are tied to that SM
    group); otherwise it keeps the whole device and compression is merely
    confined to its slice.
    """
    if device.type != "cuda":
        return StreamPool(None, [], False, {})
    if use_greenctx:
        got = try_create_greenctx_streams(device, compress_ratio, n_compress)
        if got is not None:
            main = got["main"] if main_on_greenctx else (reuse_main or torch.cuda.Stream(device=device))
            return StreamPool(main, got["compress"], True,
                              {"compress_ratio": compress_ratio, "main_sms": got["main_sms"],
                               "compress_sms": got["compress_sms"], "total_sms": got["total_sms"],
                               "main_on_greenctx": main_on_greenctx})
    low, high = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, "priority_range") else (0, -1)
    main = reuse_main or torch.cuda.Stream(device=device, priority=high)
    comp = [torch.cuda.Stream(device=device, priority=low) for _ in range(n_compress)]
    return StreamPool(main, comp, False, {"compress_ratio": 0.0, "fallback": "priority"})
