from .ccm import (KVCacheLinearCompressor, KVCacheLinearDecoupleCompressor, KVCacheHybridCompressor,
                  MiniCPMKVCompressor, PackedCCMWeights, load_compressor, load_minicpm_compressor, save_compressor,
                  ccm_output_len)  # noqa: F401
from .scorers import score_keys, select_keep, n_kept_for, SCORERS  # noqa: F401
