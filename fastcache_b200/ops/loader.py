"""Locates the compiled extension that holds the sm_100a kernels.

The shared object is built in-tree (`python setup.py build_ext --inplace`, or
`build()` in the repository's entry file) as `fastcache_b200/_C*.so`.
"""
from __future__ import annotations

import importlib
from functools import lru_cache


class ExtensionMissing(RuntimeError):
    pass


@lru_cache(maxsize=1)
def _load():
    import torch  # noqa: F401  (registers libc10/libtorch for the extension's loader)
    return importlib.import_module("fastcache_b200._C")


def ext_available() -> bool:
    try:
        _load()
        return True
    except Exception:
        return False


def ext():
    try:
        return _load()
    except Exception as exc:  # pragma: no cover - depends on the build
        raise ExtensionMissing(
            "fastcache_b200._C is not built; CUDA tensors need the sm_100a extension "
            "(run `python setup.py build_ext --inplace` at the repository root)") from exc
