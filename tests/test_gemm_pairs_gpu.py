"""Prefill-size GEMM on CTA pairs (csrc/gemm_2cta.cu, tcgen05.mma.cta_group::2) against fp32 PyTorch and against the
one-CTA-per-tile kernel."""
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
    before = e.gemm_pairs_mode()
    yield e
    e.set_gemm_pairs(before)


# M, N, K: whole tiles; row / column / K tails; one tile; many tiles per pair
SHAPES = [(512, 512, 256), (1000, 768, 320), (4096, 6144, 4096), (300, 1376, 4096), (257, 256, 8200),
          (2048, 4096, 64), (9000, 1024, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bias,act", [(False, "none"), (True, "gelu")])
def test_linear_on_cta_pairs(forms, M, N, K, bias, act):
    e = forms
    x, w = _rand(M, K, seed=1), _rand(N, K, scale=0.05, seed=2)
    b = _rand(N, seed=3) if bias else None
    want = ref.linear(x.float(), w.float(), None if b is None else b.float(), act)
    outs = {}
    for on in (1, 0):
        e.set_gemm_pairs(on)
        y = ops.linear(x, w, b, act)
        torch.cuda.synchronize()
        assert e.read_status(0) == 0
        assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 2e-2
        outs[on] = y
    # same products, same fp32 accumulation order along K: the two kernels agree to the last bit or nearly so
    assert ((outs[1].float() - outs[0].float()).abs() / (want.abs() + 1.0)).max().item() < 1e-2


@pytest.mark.parametrize("M,I,K", [(1000, 1024, 512), (4096, 12288, 4096), (257, 128, 64), (640, 2432, 1152)])
def test_swiglu_on_cta_pairs(forms, M, I, K):
    e = forms
    x, w = _rand(M, K, seed=8), _rand(2 * I, K, scale=0.05, seed=9)
    want = ref.silu_and_mul(ref.linear(x.float(), w.float()).to(torch.bfloat16).float())
    for on in (1, 0):
        e.set_gemm_pairs(on)
        y = ops.linear(x, w, None, act="swiglu")
        torch.cuda.synchronize()
        assert e.read_status(0) == 0 and y.shape == (M, I)
        assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 3e-2


def test_cta_pairs_on_a_side_stream_and_repeated(forms):
    e = forms
    e.set_gemm_pairs(1)
    x, w = _rand(3000, 1024, seed=4), _rand(2048, 1024, scale=0.05, seed=5)
    y0 = ops.linear(x, w)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        ys = [ops.linear(x, w) for _ in range(5)]
    torch.cuda.synchronize()
    assert all(torch.equal(y, y0) for y in ys) and e.read_status(0) == 0
