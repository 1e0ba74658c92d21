"""Persistent stream-K GEMM for decode-size batches (csrc/gemm_streamk.cu): finished outputs with bias / activation
and the gate/up projection with SwiGLU in the epilogue, against fp32 PyTorch and against the split-K + consumer
form it replaces."""
import pytest
import torch

from fastcache_b200 import ops
from fastcache_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.fixture
def forms():
    e = ops.ext()
    before = e.streamk_mode()
    yield e
    e.set_streamk(before)


# (M, I, K): one tile per CTA and less, tiles split over many CTAs, K that is no multiple of 64, one token
SWIGLU = [(128, 12288, 4096), (128, 3072, 4096), (5, 1408, 512), (90, 11008, 4096), (1, 128, 4096), (33, 1536, 136),
          (64, 9472, 3584), (128, 256, 12288)]


@pytest.mark.parametrize("M,I,K", SWIGLU)
def test_gate_up_swiglu_stream_k(forms, M, I, K):
    e = forms
    x, w = _rand(M, K, seed=6), _rand(2 * I, K, scale=0.05, seed=7)
    want = ref.silu_and_mul(ref.linear(x.float(), w.float()).to(torch.bfloat16).float())
    outs = {}
    for on in (True, False):
        e.set_streamk(2 if on else 0)
        y = ops.linear_silu_mul(x, w)
        y2 = ops.linear_silu_mul(x, w)             # the arrival counters must have been left at zero
        torch.cuda.synchronize()
        assert e.read_status(0) == 0 and y.shape == (M, I)
        assert torch.equal(y, y2)
        assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 3e-2
        outs[on] = y
    assert ((outs[True].float() - outs[False].float()).abs() / (want.abs() + 1.0)).max().item() < 3e-2


@pytest.mark.parametrize("M,N,K,bias,act", [(128, 151936, 1024, False, "none"), (7, 40000, 512, True, "gelu"),
                                            (64, 65536, 256, True, "none"), (100, 38000, 4096, False, "relu")])
def test_wide_output_stream_k(forms, M, N, K, bias, act):
    """More 256-row tiles than SMs (the LM head's shape class): ops.linear takes the stream-K kernel."""
    e = forms
    x, w = _rand(M, K, seed=1), _rand(N, K, scale=0.03, seed=2)
    b = _rand(N, seed=3) if bias else None
    want = ref.linear(x.float(), w.float(), None if b is None else b.float(), act)
    outs = {}
    for on in (True, False):
        e.set_streamk(2 if on else 0)
        y = ops.linear(x, w, b, act)
        y2 = ops.linear(x, w, b, act)
        torch.cuda.synchronize()
        assert e.read_status(0) == 0
        assert torch.equal(y, y2)
        assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 2e-2
        outs[on] = y
    assert ((outs[True].float() - outs[False].float()).abs() / (want.abs() + 1.0)).max().item() < 2e-2


def test_stream_k_in_a_cuda_graph_and_on_two_streams(forms):
    """Captured and replayed (programmatic dependent launch inside the graph), and two streams at once, each with
    its own scratch and counters."""
    e = forms
    e.set_streamk(2)
    M, H, F = 128, 2048, 4096
    wgu, wd = _rand(2 * F, H, scale=0.03, seed=13), _rand(H, F, scale=0.03, seed=14)
    x0 = _rand(M, H, seed=16)

    def chain(x):
        return ops.linear(ops.linear_silu_mul(x, wgu), wd)

    want = chain(x0)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(s1):
        chain(x0)
        s1.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s1):
            out = chain(x0)
        for _ in range(3):
            g.replay()
            s1.synchronize()
            assert torch.equal(out, want)
    res = []
    for _ in range(4):
        with torch.cuda.stream(s1):
            a = chain(x0)
        with torch.cuda.stream(s2):
            b = chain(x0)
        res += [a, b]
    torch.cuda.synchronize()
    assert all(torch.equal(r, want) for r in res)
    assert e.read_status(0) == 0
