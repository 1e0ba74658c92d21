"""`utils_ccm.utils_kvcachePool` of the reference."""
from fastcache_b200.serving.harness import KVCacheItem, KVCachePool  # noqa: F401
