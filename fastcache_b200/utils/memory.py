"""Device memory queries (reference: nanovllm/utils/memory.py:6-18, NVML based).

`torch.cuda.mem_get_info` reports the same driver numbers without a second
library; NVML is used only when asked for (it also sees other processes'
usage, which the pool sizing wants on a shared GPU).
"""
from __future__ import annotations

import os
from typing import Tuple

import torch


def get_gpu_memory(device: int | None = None, use_nvml: bool = False) -> Tuple[int, int, int]:
    """(total, used, free) bytes of the current visible device."""
    if not torch.cuda.is_available():
        return 0, 0, 0
    if device is None:
        device = torch.cuda.current_device()
    if use_nvml:
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(visible.split(",")[device]) if visible else device
            info = pynvml.nvmlDeviceGetMemoryInfo(pynvml.nvmlDeviceGetHandleByIndex(idx))
            return int(info.total), int(info.used), int(info.free)
        except Exception:
            pass
    free, total = torch.cuda.mem_get_info(device)
    return int(total), int(total - free), int(free)
