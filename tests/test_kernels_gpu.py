"""sm_100a kernels against the fp32 PyTorch statement of the same op."""
import math

import pytest
import torch

from fastcache_b200 import ops
from fastcache_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def _check_status():
    assert ops.ext().read_status(torch.cuda.current_device()) == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 128), (1000, 768, 320), (4096, 6144, 4096),
                                   (300, 1376, 4096), (257, 128, 8200)])
def test_gemm_large_m(M, N, K):
    x, w = _rand(M, K, seed=1), _rand(N, K, scale=0.05, seed=2)
    y = ops.linear(x, w)
    want = x.float() @ w.float().T
    torch.cuda.synchronize()
    _check_status()
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (7, 6144, 4096), (33, 4096, 12288), (90, 1024, 512),
                                   (128, 4096, 4096), (200, 512, 4096), (256, 24576, 4096), (128, 1000, 136)])
def test_gemm_small_m_swapped_splitk(M, N, K):
    x, w = _rand(M, K, seed=3), _rand(N, K, scale=0.05, seed=4)
    b = _rand(N, seed=5)
    y = ops.linear(x, w, b)
    want = x.float() @ w.float().T + b.float()
    torch.cuda.synchronize()
    _check_status()
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-2, err
    y2 = ops.linear(x, w, b)           # counters must have been left at zero
    assert torch.equal(y, y2)


@pytest.mark.parametrize("act", ["relu", "gelu", "gelu_tanh", "quick_gelu", "swiglu"])
def test_gemm_activation_bias(act):
    x, w, b = _rand(300, 256, seed=6), _rand(512, 256, scale=0.1, seed=7), _rand(512, seed=8)
    y = ops.linear(x, w, b, act)
    want = ref.linear(x.float(), w.float(), b.float(), act)
    assert ((y.float() - want).abs() / (want.abs() + 1.0)).max().item() < 2e-2


@pytest.mark.parametrize("T,H", [(1, 256), (37, 4096), (128, 5120), (5, 3584), (3, 1152)])
def test_rms_and_layer_norm(T, H):
    x, r, w, b = _rand(T, H, seed=1), _rand(T, H, seed=2), _rand(H, seed=3), _rand(H, seed=4)
    y = ops.rms_norm(x, w, 1e-6)
    assert (y.float() - ref.rms_norm(x, w, 1e-6).float()).abs().max().item() < 3e-2
    r2 = r.clone()
    y2, r_out = ops.add_rms_norm(x, r2, w, 1e-6)
    wy, wr = ref.add_rms_norm(x, r, w, 1e-6)
    assert torch.equal(r_out, wr)
    assert (y2.float() - wy.float()).abs().max().item() < 3e-2
    y3 = ops.layer_norm(x, w, b, 1e-5)
    assert (y3.float() - ref.layer_norm(x.float(), w.float(), b.float(), 1e-5)).abs().max().item() < 5e-2


def test_silu_embedding_sample():
    x = _rand(77, 2 * 1376, seed=1)
    assert (ops.silu_and_mul(x).float() - ref.silu_and_mul(x.float())).abs().max().item() < 5e-2
    w = _rand(1000, 256, seed=2)
    ids = torch.randint(0, 1200, (50,), device=DEV)
    assert torch.equal(ops.embedding(ids, w, 100), ref.embedding(ids, w, 100))
    logits = _rand(9, 5000, seed=3)
    t0 = torch.zeros(9, device=DEV)
    assert torch.equal(ops.sample(logits, t0), logits.float().argmax(-1))
    t1 = torch.full((9,), 0.8, device=DEV)
    s1, s2 = ops.sample(logits, t1, seed=5), ops.sample(logits, t1, seed=5)
    assert torch.equal(s1, s2) and int(s1.max()) < 5000
    # a peaked distribution must be sampled at its peak
    peaked = logits.clone()
    peaked[:, 123] = 200.0
    assert torch.all(ops.sample(peaked, t1, seed=9) == 123)


def _mix32(x):
    m = 0xFFFFFFFF
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    return x ^ (x >> 16)


@pytest.mark.parametrize("B,V,ld,offset,limit", [(9, 5000, 5000, 0, -1), (5, 151936, 151936, 0, -1),
                                                 (7, 4099, 4104, 0, -1), (6, 4096, 4096, 8192, 10000),
                                                 (3, 24, 24, 0, -1)])
def test_sampler_draw_matches_its_statement(B, V, ld, offset, limit):
    """token = argmax_j logit_j / T + Gumbel(seed, row, global index j): the same draw from the PyTorch statement of
    the hash, whichever CTA of the row's cluster holds the winner (rows that are not a multiple of the slice, a row
    stride larger than the row, a vocabulary shard with padding at its end, a row shorter than one slice)."""
    seed = 77
    logits = (_rand(B, ld, seed=11) * 3)[:, :V]
    temps = torch.tensor([0.0, 0.6, 1.0, 0.8, 1.3, 0.0, 0.9, 0.7, 1.1][:B], device=DEV)
    got = ops.sample(logits, temps, seed=seed, vocab_offset=offset, v_limit=limit)
    torch.cuda.synchronize()
    gj = torch.arange(V, device=DEV, dtype=torch.int64) + offset
    for b in range(B):
        row_seed = _mix32(torch.tensor((seed ^ (b * 0x9E3779B9)) & 0xFFFFFFFF, device=DEV, dtype=torch.int64))
        r = _mix32((row_seed + gj) & 0xFFFFFFFF)
        u = ((r >> 9).double() + 0.5) / 8388608.0
        t = float(temps[b])
        v = logits[b].double()
        if t > 0:
            v = v / t - torch.log(-torch.log(u))
        if limit >= 0:
            v = torch.where(gj < limit, v, torch.full_like(v, -float("inf")))
        tok = int(got[b]) - offset
        assert 0 <= tok < V and (limit < 0 or int(got[b]) < limit)
        if t == 0:
            assert tok == int((v == v.max()).nonzero()[0])          # the lowest index among equal logits
        else:
            assert float(v.max() - v[tok]) < 1e-3       # the kernel's fast logarithms may swap a near-tie


def test_sampler_frequencies_follow_the_tempered_softmax():
    """49152 draws of one 12-entry row (rows of a batch and steps differ only in the noise): every entry is drawn
    with its softmax(logits / T) probability, within four standard deviations."""
    B, V, T = 16384, 12, 0.7
    row = torch.tensor([2.0, 1.5, 1.0, 0.5, 0.0, -0.5, -1.0, 3.0, 2.5, -2.0, 0.25, 1.75]).to(torch.bfloat16)
    logits = row.repeat(B, 1).to(DEV)
    temps = torch.full((B,), T, device=DEV)
    counts = torch.zeros(V, dtype=torch.float64)
    seeds = (3, 1000003 + 4, 77777)
    for seed in seeds:
        tok = ops.sample(logits, temps, seed=seed)
        counts += torch.bincount(tok.cpu(), minlength=V).double()
    n = B * len(seeds)
    p = torch.softmax(row.double() / T, dim=0)
    sigma = torch.sqrt(p * (1 - p) / n)
    assert float(counts.sum()) == n
    assert torch.all((counts / n - p).abs() < 4 * sigma + 1e-4), (counts / n, p)


def test_sampler_noise_is_finite_at_the_ends_of_the_hash_range():
    """The entries whose hash gives the largest and the smallest uniform number get noise of about +16.6 and -2.8:
    neither beats (or loses to) a logit that is 40 away.  A uniform number that rounded to 1 would win every time."""
    seed = 5
    row_seed = _mix32(torch.tensor(seed & 0xFFFFFFFF, device=DEV, dtype=torch.int64))      # row 0
    hi = lo = None
    for start in range(0, 1 << 28, 1 << 24):
        gj = torch.arange(start, start + (1 << 24), device=DEV, dtype=torch.int64)
        k = _mix32((row_seed + gj) & 0xFFFFFFFF) >> 9
        if hi is None and bool((k == 0x7FFFFF).any()):
            hi = int(gj[(k == 0x7FFFFF).nonzero()[0]])
        if lo is None and bool((k == 0).any()):
            lo = int(gj[(k == 0).nonzero()[0]])
        if hi is not None and lo is not None:
            break
    assert hi is not None and lo is not None
    t = torch.ones(1, device=DEV)
    for g, other in ((hi, 40.0), (lo, -40.0)):
        off = max(0, g - 11)
        logits = torch.full((1, 32), other, device=DEV, dtype=torch.bfloat16)
        logits[0, g - off] = 0.0
        tok = int(ops.sample(logits, t, seed=seed, vocab_offset=off)[0])
        assert (tok != g) if other > 0 else (tok == g)


@pytest.mark.parametrize("D,Hq,Hkv,qk", [(128, 8, 2, True), (64, 4, 2, False), (128, 4, 4, False)])
def test_rope_qknorm_store(D, Hq, Hkv, qk):
    T, nb, bs = 45, 8, 16
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=1)
    pos = torch.randint(0, 500, (T,), device=DEV)
    cs = ref.build_cos_sin_cache(D, 512, 10000.0, DEV)
    qw = _rand(D, seed=2) if qk else None
    kw = _rand(D, seed=3) if qk else None
    slots = torch.randperm(nb * bs, device=DEV)[:T].int()
    slots[3] = -1
    kc, vc = (torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    kc2, vc2 = kc.clone(), vc.clone()
    q = ops.rope_qknorm_store(qkv, pos, cs, Hq, Hkv, D, qw, kw, 1e-6, kc, vc, slots)
    q2 = ref.rope_qknorm_store(qkv, pos, cs, Hq, Hkv, D, qw, kw, 1e-6, kc2, vc2, slots)
    _check_status()
    assert (q.float() - q2.float()).abs().max().item() < 6e-2
    assert (kc.float() - kc2.float()).abs().max().item() < 6e-2
    assert torch.equal(vc, vc2)


def _paged(B, lens, Hkv, D, bs, seed=0):
    nb_per = [-(-n // bs) for n in lens]
    nb = sum(nb_per) + 3
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(seed)).tolist()
    kc, vc = _rand(nb, Hkv, bs, D, seed=seed + 1), _rand(nb, Hkv, bs, D, seed=seed + 2)
    bt = torch.zeros(B, max(nb_per), dtype=torch.int32)
    k = 0
    for i, n in enumerate(nb_per):
        bt[i, :n] = torch.tensor(perm[k:k + n], dtype=torch.int32)
        k += n
    return kc, vc, bt.to(DEV)


@pytest.mark.parametrize("D,Hq,Hkv,bs,lens", [
    (128, 32, 8, 16, [1, 17, 64, 65, 300]), (128, 8, 8, 256, [1000, 5]), (64, 4, 2, 16, [33, 129]),
    (128, 28, 4, 64, [2049]), (128, 8, 1, 32, [4000, 77, 640])])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_decode_attention(D, Hq, Hkv, bs, lens, splits):
    B = len(lens)
    kc, vc, bt = _paged(B, lens, Hkv, D, bs)
    q = _rand(B, Hq, D, seed=9)
    cl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = D ** -0.5
    o = ops.decode_attention(q, kc, vc, bt, cl, scale, {"splits": splits})
    want = ref.decode_attention(q.float(), kc.float(), vc.float(), bt, cl, scale)
    _check_status()
    assert (o.float() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("D,Hq,Hkv,bs,lens", [
    (128, 32, 8, 16, [1, 17, 64, 65, 300]), (128, 8, 8, 256, [1000, 5]), (64, 4, 2, 16, [33, 129]),
    (128, 8, 1, 32, [4000, 77, 640])])
@pytest.mark.parametrize("splits", [0, 3, 5])
def test_decode_attention_merge_in_the_attention_kernel(D, Hq, Hkv, bs, lens, splits):
    """Split-KV where the last split of a (request, KV head) to arrive merges (no merge kernel): same results as
    the fp32 statement, again on a second call (the arrival counters are back at zero) and from a CUDA graph."""
    e = ops.ext()
    before = e.decode_merge_in_kernel()
    e.set_decode_merge_in_kernel(True)
    try:
        B = len(lens)
        kc, vc, bt = _paged(B, lens, Hkv, D, bs)
        q = _rand(B, Hq, D, seed=9)
        cl = torch.tensor(lens, dtype=torch.int32, device=DEV)
        scale = D ** -0.5
        want = ref.decode_attention(q.float(), kc.float(), vc.float(), bt, cl, scale)
        o1 = ops.decode_attention(q, kc, vc, bt, cl, scale, {"splits": splits})
        o2 = ops.decode_attention(q, kc, vc, bt, cl, scale, {"splits": splits})
        _check_status()
        assert (o1.float() - want).abs().max().item() < 2e-2 and torch.equal(o1, o2)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            ops.decode_attention(q, kc, vc, bt, cl, scale, {"splits": splits})
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                og = ops.decode_attention(q, kc, vc, bt, cl, scale, {"splits": splits})
            for _ in range(3):
                g.replay()
                stream.synchronize()
                assert torch.equal(og, o1)
        _check_status()
    finally:
        e.set_decode_merge_in_kernel(before)


@pytest.mark.parametrize("D,Hq,Hkv,bs,qlens,kvlens", [
    (128, 8, 2, 16, [5, 64, 130], [5, 64, 130]), (128, 4, 4, 256, [300], [300]),
    (64, 4, 2, 16, [128, 128], [128, 128]), (128, 8, 2, 32, [10, 100], [74, 228]),
    (128, 32, 8, 64, [1000], [1000]), (128, 4, 2, 8, [257, 3], [300, 131]),
    (128, 16, 8, 256, [2048, 700], [2048, 1212])])
@pytest.mark.parametrize("impl", [1, 2, 3])
def test_prefill_attention(D, Hq, Hkv, bs, qlens, kvlens, impl):
    if impl >= 2 and D != 128:
        pytest.skip("the tcgen05 kernel is head_dim 128 only")
    B = len(qlens)
    kc, vc, bt = _paged(B, kvlens, Hkv, D, bs, seed=4)
    T = sum(qlens)
    q = _rand(T, Hq, D, seed=11)
    cu = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    kl = torch.tensor(kvlens, dtype=torch.int32, device=DEV)
    scale = D ** -0.5
    o = ops.prefill_attention(q, kc, vc, bt, cu, kl, scale, max(qlens), impl)
    want = ref.prefill_attention(q.float(), kc.float(), vc.float(), bt, cu, kl, scale)
    _check_status()
    assert (o.float() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("B,Sq,Sk,H,D,masked", [(2, 577, 577, 16, 64, False), (3, 1024, 1024, 16, 72, True),
                                                (2, 64, 700, 28, 128, True), (1, 10, 10, 4, 64, False),
                                                (1, 300, 129, 1, 32, False), (2, 257, 256, 3, 96, True)])
@pytest.mark.parametrize("impl", [1, 2])
def test_dense_attention(B, Sq, Sk, H, D, masked, impl):
    """impl 1: the mma.sync kernel; impl 2: the tcgen05 kernel (head_dim padded to 64 / 128 by the TMA copies)."""
    qkv = _rand(B, max(Sq, Sk), 3, H, D, seed=21)
    q, k, v = qkv[:, :Sq, 0], qkv[:, :Sk, 1], qkv[:, :Sk, 2]          # strided views, as the towers pass them
    mask = None
    if masked:
        lens = torch.randint(Sk // 2, Sk + 1, (B,))
        mask = (torch.arange(Sk)[None, :] < lens[:, None])
        mask[:, 3] = False                                             # a hole, not only a length
        mask = mask.to(DEV)
    o = ops.dense_attention(q, k, v, D ** -0.5, mask, impl=impl)
    want = ref.dense_attention(q.float(), k.float(), v.float(), D ** -0.5, mask)
    _check_status()
    assert (o.float() - want).abs().max().item() < 2e-2


def test_dense_attention_contiguous_and_expanded_operands():
    """Separate contiguous q / k / v (the resampler's form) take the tcgen05 kernel; a query expanded over the
    batch (stride 0) cannot be described to TMA and takes the other kernel under impl 0."""
    B, Sq, Sk, H, D = 3, 64, 1024, 28, 128
    q1 = _rand(1, Sq, H, D, seed=5)
    k, v = _rand(B, Sk, H, D, seed=6), _rand(B, Sk, H, D, seed=7)
    q = q1.expand(B, -1, -1, -1)
    want = ref.dense_attention(q.float(), k.float(), v.float(), D ** -0.5, None)
    for qq, impl in ((q.contiguous(), 2), (q, 0)):
        o = ops.dense_attention(qq, k, v, D ** -0.5, None, impl=impl)
        _check_status()
        assert (o.float() - want).abs().max().item() < 2e-2
    with pytest.raises(RuntimeError):
        ops.dense_attention(q, k, v, D ** -0.5, None, impl=2)


@pytest.mark.parametrize("mode", ["int8", "int8_asym", "int4", "nf4", "fp8_e4m3", "fp8_e5m2"])
@pytest.mark.parametrize("shape", [(2, 8, 333, 128), (5, 77, 256), (3, 64)])
def test_quantiser_kernels_match_the_pytorch_statements(mode, shape):
    """Codes, scales and restored values of the CUDA quantisers against the same op stated in PyTorch on fp32
    copies of the data (bit-identical codes; restored values equal after the bf16 rounding of the output)."""
    from fastcache_b200.compress import quant
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(*shape, generator=g) * 3).to(torch.bfloat16)
    x[..., 0] = 0                                                   # exact zeros and ties
    dev = quant.quantize(x.cuda(), mode, 64)
    cpu = quant.quantize(x, mode, 64)                               # the PyTorch statement
    assert dev["q"].dtype == cpu["q"].dtype and tuple(dev["q"].shape) == tuple(cpu["q"].shape)
    torch.testing.assert_close(dev["scale"].cpu(), cpu["scale"], rtol=0, atol=0)
    if mode == "int8_asym":
        torch.testing.assert_close(dev["zero"].cpu(), cpu["zero"], rtol=0, atol=0)
    assert torch.equal(dev["q"].cpu().view(torch.uint8), cpu["q"].view(torch.uint8))
    back_dev, back_cpu = quant.dequantize(dev), quant.dequantize(cpu)
    assert back_dev.dtype == torch.bfloat16 and back_dev.shape == x.shape
    torch.testing.assert_close(back_dev.cpu().float(), back_cpu.float(), rtol=0, atol=0)
    if mode in ("int8", "int4"):
        fake = quant.fake_quantize(x.cuda(), 8 if mode == "int8" else 4, 64)
        torch.testing.assert_close(fake.cpu().float(), back_cpu.float(), rtol=0, atol=0)
