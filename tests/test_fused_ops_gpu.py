"""GEMM + consumer fusions (split-K partial sums reduced by the op that reads the GEMM result)."""
import pytest
import torch

from fastcache_b200 import ops
from fastcache_b200.ops import reference as ref

pytestmark = pytest.mark.gpu



@pytest.fixture(autouse=True)
def _one_kernel_epilogues():
    """The one-kernel form of GEMM + (all-reduce +) add + RMSNorm is opt-in (the pair of kernels is the faster
    default); the tests of this module switch it on so that both forms stay covered."""
    e = ops.ext()
    before = e.fused_epilogues_enabled()
    e.set_fused_epilogues(True)
    yield
    e.set_fused_epilogues(before)


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


def _norm_ref(x, w, b, res, nw):
    y = ref.linear(x.float(), w.float(), None if b is None else b.float()).to(torch.bfloat16)
    return ref.add_rms_norm(y, res.clone(), nw, 1e-6)


@pytest.mark.parametrize("M,N,K", [(128, 4096, 512), (200, 5120, 3200), (1, 4096, 1536), (33, 8192, 1024)])
def test_fused_gemm_add_norm_in_a_cuda_graph(M, N, K):
    """GEMM + grid barrier + split-K sum + residual add + RMSNorm as one kernel: tensor-parallel shard shapes,
    replayed from a CUDA graph (the barrier words reset themselves) with new inputs every time."""
    x, w = _rand(M, K, seed=21), _rand(N, K, scale=0.03, seed=22)
    nw = _rand(N, seed=23)
    res = _rand(M, N, seed=24)
    xs, rs = x.clone(), res.clone()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(2):                               # warm-up: workspace of this stream, lazy init
            ops.linear_add_rms_norm(xs, w, None, rs.clone(), nw, 1e-6)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            y, r = ops.linear_add_rms_norm(xs, w, None, rs, nw, 1e-6)
        for it in range(3):
            xi, ri = _rand(M, K, seed=30 + it), _rand(M, N, seed=40 + it)
            xs.copy_(xi)
            rs.copy_(ri)
            g.replay()
            stream.synchronize()
            want_y, want_r = _norm_ref(xi, w, None, ri, nw)
            assert (rs.float() - want_r.float()).abs().max().item() < 0.07
            assert (y.float() - want_y.float()).abs().max().item() < 0.07
    assert ops.ext().read_status(0) == 0


def test_two_streams_run_decode_size_gemms_at_once():
    """Every stream has its own split-K scratch and barrier words: the same fused op on two streams at the same
    time, many times, gives each stream its own right answer."""
    M, N, K = 128, 4096, 4096
    w, nw = _rand(N, K, scale=0.03, seed=52), _rand(N, seed=53)
    xa, xb = _rand(M, K, seed=54), _rand(M, K, seed=55)
    ra, rb = _rand(M, N, seed=56), _rand(M, N, seed=57)
    want_a, _ = _norm_ref(xa, w, None, ra, nw)
    want_b, _ = _norm_ref(xb, w, None, rb, nw)
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs_a, outs_b = [], []
    for _ in range(20):
        with torch.cuda.stream(sa):
            outs_a.append(ops.linear_add_rms_norm(xa, w, None, ra.clone(), nw, 1e-6)[0])
        with torch.cuda.stream(sb):
            outs_b.append(ops.linear_add_rms_norm(xb, w, None, rb.clone(), nw, 1e-6)[0])
    torch.cuda.synchronize()
    assert ops.ext().read_status(0) == 0
    for ya, yb in zip(outs_a, outs_b):
        assert (ya.float() - want_a.float()).abs().max().item() < 0.07
        assert (yb.float() - want_b.float()).abs().max().item() < 0.07
        assert torch.equal(ya, outs_a[0]) and torch.equal(yb, outs_b[0])


@pytest.mark.parametrize("M,N,K,bias", [(128, 4096, 512, False), (40, 1024, 1536, True)])
def test_fused_gemm_allreduce_add_norm_on_one_gpu(M, N, K, bias):
    """The tensor-parallel epilogue (GEMM, staging, flag exchange, sum over ranks, add, norm) with this GPU as
    rank 0 of 2 and the second rank played by local memory: its contribution is written beforehand and its flag
    words are preset to an epoch far ahead, so nothing waits for anything.  Checks both the one-kernel path and
    the two-kernel path against fp32."""
    import os
    e = ops.ext()
    dev = torch.device("cuda", 0)
    bufs = [torch.zeros(2, 256, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]      # [buf][rank][rows][N]
    flags = torch.zeros(2, 512 * 8, dtype=torch.int32, device=dev)
    flags[0].view(512, 8)[:, 1] = 1 << 20                                 # "rank 1 has arrived" for a long time
    status = e.status_tensor(0)
    e.read_status(0)
    x, w = _rand(M, K, seed=61), _rand(N, K, scale=0.03, seed=62)
    b = _rand(N, seed=63) if bias else None
    nw, res = _rand(N, seed=64), _rand(M, N, seed=65)
    other = _rand(M, N, scale=0.5, seed=66)                               # what rank 1 would have contributed
    mine = ref.linear(x.float(), w.float(), None if b is None else b.float()).to(torch.bfloat16)
    want_y, want_r = ref.add_rms_norm((mine.float() + other.float()).to(torch.bfloat16), res.clone(), nw, 1e-6)
    try:
        e.comm_init(0, 2, [bufs[0][0].data_ptr(), bufs[0][1].data_ptr()],
                    [bufs[1][0].data_ptr(), bufs[1][1].data_ptr()],
                    [flags[0].data_ptr(), flags[1].data_ptr()], 0, 0, 0)
        for buf in (0, 1, 0):
            bufs[buf][1][:M].copy_(other)
            r = res.clone()
            y = e.linear_allreduce_add_rmsnorm(x, w, b, buf, r, nw, 1e-6, False, status)
            torch.cuda.synchronize()
            assert e.read_status(0) == 0
            assert (r.float() - want_r.float()).abs().max().item() < 0.07
            # one bf16 step at the magnitude of the normalised, weighted values
            assert ((y.float() - want_y.float()).abs() / (want_y.float().abs() + 1.0)).max().item() < 2e-2
            assert (bufs[buf][0][:M].float() - mine.float()).abs().max().item() < 0.03   # rank 0's staged rows
    finally:
        e.comm_shutdown()


@pytest.mark.parametrize("M,N,K,bias", [(128, 4096, 512, False), (40, 1024, 1536, True), (3, 2048, 4096, False)])
def test_push_form_of_the_allreduce_on_one_gpu(M, N, K, bias):
    """The push form (every rank stores its finished row into its slot of every peer's buffer before the flag
    exchange, then sums the slots of its own buffer) with this GPU as rank 0 of 2 and the second rank played by
    local memory: what rank 1 would have pushed is written into slot 1 of rank 0's buffer beforehand, its flags
    are preset, and afterwards slot 0 of "rank 1's" buffer must hold rank 0's row."""
    e = ops.ext()
    e.set_fused_epilogues(False)
    dev = torch.device("cuda", 0)
    R = 256                                                               # rows per slot
    bufs = [torch.zeros(2, 2 * R, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]    # [buf][rank][slot rows][N]
    flags = torch.zeros(2, 512 * 8, dtype=torch.int32, device=dev)
    flags[0].view(512, 8)[:, 1] = 1 << 20
    status = e.status_tensor(0)
    e.read_status(0)
    x, w = _rand(M, K, seed=61), _rand(N, K, scale=0.03, seed=62)
    b = _rand(N, seed=63) if bias else None
    nw, res = _rand(N, seed=64), _rand(M, N, seed=65)
    other = _rand(M, N, scale=0.5, seed=66)
    mine = ref.linear(x.float(), w.float(), None if b is None else b.float()).to(torch.bfloat16)
    want_y, want_r = ref.add_rms_norm((mine.float() + other.float()).to(torch.bfloat16), res.clone(), nw, 1e-6)
    try:
        e.comm_init(0, 2, [bufs[0][0].data_ptr(), bufs[0][1].data_ptr()],
                    [bufs[1][0].data_ptr(), bufs[1][1].data_ptr()],
                    [flags[0].data_ptr(), flags[1].data_ptr()], 0, 0, 0, R)
        for buf in (0, 1, 0):
            bufs[buf][0][R:R + M].copy_(other)                            # slot 1 of rank 0's buffer
            bufs[buf][1].zero_()
            r = res.clone()
            y = e.linear_allreduce_add_rmsnorm(x, w, b, buf, r, nw, 1e-6, False, status)
            torch.cuda.synchronize()
            assert e.read_status(0) == 0
            assert (r.float() - want_r.float()).abs().max().item() < 0.07
            assert ((y.float() - want_y.float()).abs() / (want_y.float().abs() + 1.0)).max().item() < 2e-2
            assert (bufs[buf][1][:M].float() - mine.float()).abs().max().item() < 0.03    # pushed to "rank 1", slot 0
            assert int(bufs[buf][1][R:].abs().max()) == 0                                 # and nowhere else
    finally:
        e.comm_shutdown()


@pytest.mark.parametrize("pipelined", [False, True])
@pytest.mark.parametrize("T,K", [(1000, 256), (4096, 512), (300, 1024)])
def test_row_parallel_gemm_reduce_scatter_on_one_gpu(pipelined, T, K):
    """The prefill-size fused GEMM + reduce-scatter + add + RMSNorm + all-gather send with this GPU as rank 0 of 2
    and the second rank played by local memory: what rank 1 would have delivered for rank 0's rows is written into
    the staging buffer beforehand and its flags are preset.  Both forms: one reduction phase after the GEMM, and
    row groups reduced by the extra warps while the GEMM runs.  Checks rank 0's residual rows, the normalised rows
    it sends to both ranks, and the partial sums it delivers for rank 1's rows."""
    e = ops.ext()
    dev = torch.device("cuda", 0)
    H, W = 1024, 8                                                        # hidden, flag words per group
    chunk = -(-(-(-T // 2)) // 128) * 128
    groups = chunk // 128
    stage = [torch.zeros(2 * chunk, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]   # [rank][source slot rows][H]
    xg = [torch.zeros(2 * chunk, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    flags = [torch.zeros(2 * W + groups * W, dtype=torch.int32, device=dev) for _ in range(2)]
    flags[0][1] = 1 << 20                                                 # chunk flag: source 1 delivered
    flags[0][2 * W:].view(groups, W)[:, 1] = 1 << 20                      # group flags: source 1 delivered
    status = e.status_tensor(0)
    e.read_status(0)
    before = e.tp_pipeline_enabled()
    x, w = _rand(T, K, scale=0.5, seed=71), _rand(H, K, scale=0.05, seed=72)
    nw = _rand(H, seed=73)
    own = min(T, chunk)
    res = _rand(own, H, seed=74)
    other = _rand(own, H, scale=0.5, seed=75)                             # rank 1's partial sums for rank 0's rows
    mine = ref.linear(x.float(), w.float()).to(torch.bfloat16)            # [T, H]: rank 0's partial sums
    want_y, want_r = ref.add_rms_norm((mine[:own].float() + other.float()).to(torch.bfloat16), res.clone(), nw, 1e-6)
    try:
        e.set_tp_pipeline(pipelined)
        e.tp_init(0, 2, [t.data_ptr() for t in stage], [t.data_ptr() for t in xg], [t.data_ptr() for t in flags],
                  chunk, 2 * chunk, H, 0, groups)
        for epoch in (1, 2):
            stage[0][chunk:chunk + own].copy_(other)                      # slot of source 1 in rank 0's buffer
            r = res.clone()
            e.gemm_rs_add_norm(x, w, r, nw, 1e-6, chunk, epoch, status, 0)
            torch.cuda.synchronize()
            assert e.read_status(0) == 0
            assert (r.float() - want_r.float()).abs().max().item() < 0.07
            for d in (0, 1):                                              # the all-gather send reached both ranks
                got = xg[d][:own].float()
                assert ((got - want_y.float()).abs() / (want_y.float().abs() + 1.0)).max().item() < 2e-2
            if T > chunk:                                                 # rank 0's partial sums for rank 1's rows
                assert (stage[1][:T - chunk].float() - mine[chunk:].float()).abs().max().item() < 0.03
            delivered = flags[1][2 * W] if pipelined else flags[1][0]        # first row group / whole chunk
            assert int(delivered) == epoch and int(flags[1][W]) == epoch       # delivered to / gathered at rank 1
            assert int(flags[0][W]) == epoch                                   # gathered flag on itself
    finally:
        e.set_tp_pipeline(before)
