"""Directory conventions (reference: fastcache_paths.py:8-22): checkpoint, dataset and result
directories default to folders beside the package and can be moved with
FASTCACHE_CKPT_DIR / FASTCACHE_DATASETS_DIR / FASTCACHE_RESULTS_DIR."""
from __future__ import annotations

import os
import sys
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parents[2]
CKPT_DIR = Path(os.environ.get("FASTCACHE_CKPT_DIR", REPO_ROOT / "ckpt")).resolve()
DATASETS_DIR = Path(os.environ.get("FASTCACHE_DATASETS_DIR", REPO_ROOT / "datasets")).resolve()
RESULTS_DIR = Path(os.environ.get("FASTCACHE_RESULTS_DIR", REPO_ROOT / "results")).resolve()


def ensure_sys_paths() -> None:
    root = str(REPO_ROOT)
    if root not in sys.path:
        sys.path.insert(0, root)
