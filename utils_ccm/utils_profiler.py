"""`utils_ccm.utils_profiler` of the reference (analytic FLOP / byte models)."""
from fastcache_b200.serving.profiler import (ComputeStats, LLaVAConfigWrapper, LLaVAIntensityAnalyzer,  # noqa: F401
                                             LLMConfig, LLMConfigWrapper, LLMIntensityAnalyzer, PhaseCost,
                                             VisionEncoderAnalyzer, format_number)
