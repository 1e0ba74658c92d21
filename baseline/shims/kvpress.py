"""Stand-in for the `kvpress` package.  The reference's engine-side compressor
imports it and instantiates a press object before running its own native
key-norm / streaming code (nanovllm/kernels/kvpress_compressor.py:120-160, :188);
the object is never called on that path.  These classes only accept the
constructor arguments."""


class _Press:
    def __init__(self, *args, **kwargs):
        self.args, self.kwargs = args, kwargs
        self.compression_ratio = kwargs.get("compression_ratio", 0.0)


class StreamingLLMPress(_Press):
    pass


class SnapKVPress(_Press):
    pass


class KnormPress(_Press):
    pass


class RandomPress(_Press):
    pass


class ExpectedAttentionPress(_Press):
    pass


class ObservedAttentionPress(_Press):
    pass


class TOVAPress(_Press):
    pass


class ThinKPress(_Press):
    pass


class SimLayerKVPress(_Press):
    pass


class H2OPress(_Press):
    pass
