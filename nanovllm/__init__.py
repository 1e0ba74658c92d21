"""Import-compatibility package: `from nanovllm import LLM, SamplingParams` and the sub-module
paths used by scripts written against the reference resolve to fastcache_b200."""
import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys

from fastcache_b200 import LLM, SamplingParams  # noqa: F401

_ALIASES = {
    "nanovllm.llm": "fastcache_b200.llm",
    "nanovllm.config": "fastcache_b200.config",
    "nanovllm.sampling_params": "fastcache_b200.sampling_params",
    "nanovllm.engine": "fastcache_b200.engine",
    "nanovllm.engine.llm_engine": "fastcache_b200.engine.llm_engine",
    "nanovllm.engine.llava_engine": "fastcache_b200.engine.llava_engine",
    "nanovllm.engine.sequence": "fastcache_b200.engine.sequence",
    "nanovllm.engine.scheduler": "fastcache_b200.engine.scheduler",
    "nanovllm.engine.llava_scheduler": "fastcache_b200.engine.scheduler",
    "nanovllm.engine.block_manager": "fastcache_b200.engine.block_manager",
    "nanovllm.engine.model_runner": "fastcache_b200.engine.model_runner",
    "nanovllm.engine.llava_model_runner": "fastcache_b200.engine.model_runner",
    "nanovllm.engine.auto_compress_controller": "fastcache_b200.engine.auto_compress_controller",
    "nanovllm.autocompress": "fastcache_b200.autocompress",
    "nanovllm.utils": "fastcache_b200.utils",
    "nanovllm.utils.tp": "fastcache_b200.parallel.tp",
    "nanovllm.utils.context": "fastcache_b200.utils.context",
    "nanovllm.utils.loader": "fastcache_b200.utils.loader",
    "nanovllm.utils.memory": "fastcache_b200.utils.memory",
    "nanovllm.utils.streams": "fastcache_b200.utils.streams",
    "nanovllm.layers": "fastcache_b200.layers",
    "nanovllm.models": "fastcache_b200.models",
    "nanovllm.kernels": "fastcache_b200.compress",
    "nanovllm.kernels.batched_compress": "fastcache_b200.compress.batched",
    "nanovllm.kernels.kvpress_compressor": "fastcache_b200.compress.kvpress_compat",
    "nanovllm.kernels.minicpm_compressor": "fastcache_b200.compress.ccm",
    "nanovllm.kernels.fused_compress": "fastcache_b200.compress.batched",
    "nanovllm.kernels.zero_overhead_compress": "fastcache_b200.compress.batched",
    "nanovllm.autocompress.kernels": "fastcache_b200.autocompress.kernels",
}


def _resolve(name: str):
    """Real module for an alias name: an exact entry, or the longest aliased package prefix plus the
    rest of the path (`nanovllm.layers.linear` -> `fastcache_b200.layers.linear`)."""
    if name in _ALIASES:
        return _ALIASES[name]
    parts = name.split(".")
    for cut in range(len(parts) - 1, 0, -1):
        head = ".".join(parts[:cut])
        if head in _ALIASES:
            return _ALIASES[head] + "." + ".".join(parts[cut:])
    return None


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Imports below `nanovllm.` hand back the module of this package itself (the same object, so its
    relative imports and its state are those of `fastcache_b200`), not a second copy under another name."""

    def find_spec(self, name, path=None, target=None):
        if not name.startswith("nanovllm."):
            return None
        real = _resolve(name)
        if real is None:
            return None
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        return importlib.machinery.ModuleSpec(name, self)

    def create_module(self, spec):
        return importlib.import_module(_resolve(spec.name))

    def exec_module(self, module):
        pass



if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
for _name, _real in _ALIASES.items():
    try:
        sys.modules.setdefault(_name, importlib.import_module(_real))
    except Exception:          # optional pieces (e.g. CUDA-only helpers) may be absent on a CPU box
        pass
