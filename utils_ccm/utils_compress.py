"""`utils_ccm.utils_compress` of the reference (timed presses, quantisers, timers)."""
from fastcache_b200.compress.kvpress_compat import (ExpectedAttentionPressWithTime,  # noqa: F401
                                                    KnormPressWithTime, RandomPressWithTime,
                                                    ScorerPressWithTime, SnapKVPressWithTime,
                                                    StreamingLLMPressWithTime, TimeTik, TOVAPressWithTime,
                                                    exec_compression_methods, get_underlying_model,
                                                    press_select)
from fastcache_b200.compress.quant import (BaseCompressionMethod, ImprovedKVQuantizer, QuantizedCacheWrapper,  # noqa: F401
                                           SimpleKVQuantizer)
