"""Decode-size GEMMs whose K splits reduce inside a thread-block cluster (distributed shared memory), against
fp32 PyTorch, and against the form that leaves fp32 partial sums for a consumer kernel.  The cluster form is
opt-in (it measured slower); these tests keep it covered."""
import pytest
import torch

from fastcache_b200 import ops
from fastcache_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.fixture
def both_forms():
    e = ops.ext()
    before, streamk = e.cluster_splitk_enabled(), e.streamk_mode()
    e.set_streamk(0)                     # the persistent stream-K form would take these shapes first
    yield e
    e.set_cluster_splitk(before)
    e.set_streamk(streamk)


SHAPES = [(128, 6144, 4096), (128, 4096, 4096), (128, 4096, 12288), (7, 1024, 512), (33, 768, 4096),
          (64, 4096, 1536), (200, 5120, 3200), (256, 4096, 4096), (128, 151936, 1024), (1, 3072, 4096)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bias", [False, True])
def test_linear_cluster_form_matches_fp32_and_the_partial_form(both_forms, M, N, K, bias):
    e = both_forms
    x, w = _rand(M, K, seed=1), _rand(N, K, scale=0.03, seed=2)
    b = _rand(N, seed=3) if bias else None
    want = ref.linear(x.float(), w.float(), None if b is None else b.float())
    outs = {}
    for on in (True, False):
        e.set_cluster_splitk(on)
        y = ops.linear(x, w, b, act="gelu" if bias else "none")
        y2 = ops.linear(x, w, b, act="gelu" if bias else "none")
        torch.cuda.synchronize()
        assert e.read_status(0) == 0
        assert torch.equal(y, y2)
        outs[on] = y
    if bias:
        want = torch.nn.functional.gelu(want)
    for y in outs.values():
        assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 2e-2
    assert ((outs[True].float() - outs[False].float()).abs() / (want.abs() + 1.0)).max().item() < 2e-2


@pytest.mark.parametrize("M,I,K", [(128, 12288, 4096), (128, 1536, 4096), (5, 1408, 512), (256, 2048, 1024),
                                   (40, 3072, 4096), (128, 11008, 4096)])
def test_gate_up_swiglu_in_the_cluster_epilogue(both_forms, M, I, K):
    e = both_forms
    x, w = _rand(M, K, seed=6), _rand(2 * I, K, scale=0.05, seed=7)
    want = ref.silu_and_mul(ref.linear(x.float(), w.float()).to(torch.bfloat16).float())
    for on in (True, False):
        e.set_cluster_splitk(on)
        y = ops.linear_silu_mul(x, w)
        torch.cuda.synchronize()
        assert e.read_status(0) == 0 and y.shape == (M, I)
        assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 3e-2


def test_decode_chain_in_a_cuda_graph_with_clusters(both_forms):
    """qkv -> o + add + norm -> gate/up + SwiGLU -> down + add + norm, captured once and replayed: the cluster
    launches and their programmatic dependencies survive capture."""
    e = both_forms
    e.set_cluster_splitk(True)
    M, H, F = 128, 2048, 4096
    wq, wo = _rand(H + 512, H, scale=0.03, seed=11), _rand(H, H, scale=0.03, seed=12)
    wgu, wd = _rand(2 * F, H, scale=0.03, seed=13), _rand(H, F, scale=0.03, seed=14)
    nw = _rand(H, seed=15)
    x0, res0 = _rand(M, H, seed=16), _rand(M, H, seed=17)
    xs, rs = x0.clone(), res0.clone()

    def chain(x, r):
        q = ops.linear(x, wq)[:, :H].contiguous()
        n1, r = ops.linear_add_rms_norm(q, wo, None, r, nw, 1e-6)
        act = ops.linear_silu_mul(n1, wgu)
        n2, r = ops.linear_add_rms_norm(act, wd, None, r, nw, 1e-6)
        return n2

    want = chain(x0, res0.clone())
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        chain(xs, rs.clone())
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            out = chain(xs, rs)
        for _ in range(3):
            rs.copy_(res0)
            g.replay()
            stream.synchronize()
            assert torch.equal(out, want)
    assert e.read_status(0) == 0
