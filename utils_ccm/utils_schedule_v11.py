"""`utils_ccm.utils_schedule_v11` of the reference (dynamic scheduler, timestamps, GPU monitor)."""
from fastcache_b200.serving.harness import (DynamicScheduler, GPUMonitor, PrioritizedRequest,  # noqa: F401
                                            PriorityRequest, TimestampManager)
