"""GEMM + consumer fusions (split-K partial sums reduced by the op that reads the GEMM result)."""
import pytest
import torch

from fastcache_b200 import ops
from fastcache_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("M,N,K,bias", [(128, 4096, 4096, False), (7, 1024, 12288, True), (256, 512, 512, False),
                                        (300, 1024, 2048, True), (64, 3584, 18944, False)])
def test_linear_add_rms_norm(M, N, K, bias):
    x, w = _rand(M, K, seed=1), _rand(N, K, scale=0.03, seed=2)
    b = _rand(N, seed=3) if bias else None
    res, nw = _rand(M, N, seed=4), _rand(N, seed=5)
    want_y, want_r = ref.add_rms_norm(ref.linear(x.float(), w.float(), None if b is None else b.float()).to(torch.bfloat16),
                                      res.clone(), nw, 1e-6)
    r = res.clone()
    y, r_out = ops.linear_add_rms_norm(x, w, b, r, nw, 1e-6)
    torch.cuda.synchronize()
    assert ops.ext().read_status(0) == 0
    assert (r_out.float() - want_r.float()).abs().max().item() < 0.07
    assert (y.float() - want_y.float()).abs().max().item() < 0.07
    y2, _ = ops.linear_add_rms_norm(x, w, b, res.clone(), nw, 1e-6)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M,I,K", [(128, 12288, 4096), (5, 1376, 512), (256, 2048, 1024), (400, 1024, 512)])
def test_linear_silu_mul(M, I, K):
    x, w = _rand(M, K, seed=6), _rand(2 * I, K, scale=0.05, seed=7)
    y = ops.linear_silu_mul(x, w)
    want = ref.silu_and_mul(ref.linear(x.float(), w.float()).to(torch.bfloat16).float())
    torch.cuda.synchronize()
    assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 3e-2


@pytest.mark.parametrize("M,I,K", [(1000, 1024, 512), (4096, 12288, 4096), (257, 128, 64), (640, 2432, 1152)])
def test_gemm_swiglu_epilogue(M, I, K):
    """Prefill-size gate/up projection with SwiGLU applied in the GEMM epilogue."""
    x, w = _rand(M, K, seed=8), _rand(2 * I, K, scale=0.05, seed=9)
    y = ops.linear(x, w, None, act="swiglu")
    assert y.shape == (M, I)
    want = ref.silu_and_mul(ref.linear(x.float(), w.float()))
    torch.cuda.synchronize()
    assert ops.ext().read_status(0) == 0
    assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 3e-2


@pytest.mark.parametrize("T,Hq,Hkv,qk", [(128, 32, 8, True), (5, 8, 2, False), (256, 16, 16, True)])
def test_linear_rope_qknorm_store_matches_unfused(T, Hq, Hkv, qk):
    """qkv projection fused with rope / q-k norm / paged store: same bits as GEMM followed by the rope op."""
    D, K, nb, bs = 128, 1024, 40, 16
    x, w = _rand(T, K, seed=11), _rand((Hq + 2 * Hkv) * D, K, scale=0.05, seed=12)
    pos = torch.randint(0, 500, (T,), device="cuda")
    cs = ref.build_cos_sin_cache(D, 512, 10000.0, "cuda")
    qw = _rand(D, seed=13) if qk else None
    kw = _rand(D, seed=14) if qk else None
    slots = torch.randperm(nb * bs, device="cuda")[:T].int()
    kc, vc = (torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    kc2, vc2 = kc.clone(), vc.clone()
    q = ops.linear_rope_qknorm_store(x, w, pos, cs, Hq, Hkv, D, qw, kw, 1e-6, kc, vc, slots)
    q2 = ops.rope_qknorm_store(ops.linear(x, w), pos, cs, Hq, Hkv, D, qw, kw, 1e-6, kc2, vc2, slots)
    torch.cuda.synchronize()
    assert ops.ext().read_status(0) == 0
    assert torch.equal(q, q2) and torch.equal(kc, kc2) and torch.equal(vc, vc2)
