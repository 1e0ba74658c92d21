"""Top-level module name used by the reference's scripts (`import fastcache_paths`)."""
from fastcache_b200.serving.paths import (CKPT_DIR, DATASETS_DIR, REPO_ROOT, RESULTS_DIR,  # noqa: F401
                                          ensure_sys_paths)
