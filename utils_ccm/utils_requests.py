"""`utils_ccm.utils_requests` of the reference."""
from fastcache_b200.serving.harness import Request, RequestMetrics, RequestStatus  # noqa: F401
