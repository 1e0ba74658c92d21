"""`utils_ccm.module_ccm_v11` of the reference (merge compressors, research-path compressors, cache
containers, training loss) -> fastcache_b200.compress."""
from fastcache_b200.compress.ccm import (KVCacheHybridCompressor, KVCacheLinearCompressor,  # noqa: F401
                                         KVCacheLinearDecoupleCompressor, MiniCPMKVCompressor, load_compressor,
                                         save_compressor)
from fastcache_b200.compress.research import (CompressedDecoder, CompressedDecoder_OnlyMLP,  # noqa: F401
                                              CompressedKVCache, CompressibleCache, CrossModelKVCompressor,
                                              CrossModelRealKVCompressor, LLaMAKVCacheSampler, MAEEncoder,
                                              PositionalEncoding, count_true_segments_with_zeros,
                                              logits_to_onehot)
from fastcache_b200.compress.train import KVCacheCompressionLoss  # noqa: F401
from fastcache_b200.compress.train_data import (LLM, CustomDataset, CustomImageTextDataset,  # noqa: F401
                                                CustomImageTextMinicpmDataset)
