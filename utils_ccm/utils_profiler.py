"""`utils_ccm.utils_profiler` of the reference (analytic FLOP / byte models)."""
from fastcache_b200.serving.profiler import (LLaVAIntensityAnalyzer, LLMIntensityAnalyzer,  # noqa: F401
                                             VisionEncoderAnalyzer)
