"""Device-timed micro-benchmarks of the hot kernels against the measured roofline.

Usage:  python benchmarks/kernel_bench.py [--what gemm,decode_gemm,decode_attn,prefill_attn,norm,elementwise,
                                            dense_attn,vit_gemm,ccm,evict,quant,swiglu_gemm] [--small] [--json out.json]
Timing: CUDA events on the launching stream, >= 3 warm-up iterations, an L2 flush
(write of a 256 MB buffer) before every timed iteration, median of the samples.
Peaks come from MEASURED_PEAKS.json at the repository root when present
("of measured"), else the fallback 6.65 TB/s / 1590 TFLOP/s ("of fallback").
"""
import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from fastcache_b200 import ops  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def timeit(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def bench_gemm(rows, shapes, tag):
    hbm, tf, src = peaks()
    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        ms = timeit(lambda: ops.linear(x, w))
        ms_lib = timeit(lambda: torch.nn.functional.linear(x, w))
        flops = 2.0 * M * N * K
        byts = 2.0 * (M * K + N * K + M * N)
        t_roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3
        other = {}
        if M > 256:                          # the other of the two prefill kernels (one CTA per tile / CTA pairs)
            e = ops.ext()
            mode = e.gemm_pairs_mode()
            e.set_gemm_pairs(0 if mode else 1)
            other = {("one_cta_per_tile_ms" if mode else "cta_pairs_ms"): round(timeit(lambda: ops.linear(x, w)), 4)}
            e.set_gemm_pairs(mode)
        rows.append({"kernel": tag, "M": M, "N": N, "K": K, "ms": round(ms, 4), **other, "cublas_ms": round(ms_lib, 4),
                     "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
                     "frac_of_roofline": round(t_roof / ms, 3), "peaks": src})
        print(rows[-1], flush=True)


def bench_swiglu_gemm(rows):
    """Decode-size gate/up projection + SwiGLU: the persistent stream-K kernel (one launch), the split-K GEMM with
    the consumer kernel that sums its partial sums (two launches), and cuBLAS + an elementwise kernel; then the
    LM head with and without stream-K."""
    hbm, tf, src = peaks()
    e = ops.ext()
    before = e.streamk_mode()
    for M, I, K in [(128, 12288, 4096), (128, 3072, 4096), (128, 1536, 4096), (90, 11008, 4096), (16, 12288, 4096)]:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(2 * I, K, device="cuda", dtype=torch.bfloat16) * 0.02
        t = {}
        for on in (True, False):
            e.set_streamk(2 if on else 0)
            t[on] = timeit(lambda: ops.linear_silu_mul(x, w))
        def lib():
            y = torch.nn.functional.linear(x, w)
            return torch.nn.functional.silu(y[:, :I]) * y[:, I:]
        ms_lib = timeit(lib)
        byts = 2.0 * (M * K + 2 * I * K + M * I)
        rows.append({"kernel": "gate_up_swiglu_decode", "M": M, "I": I, "K": K, "stream_k_ms": round(t[True], 4),
                     "splitk_plus_consumer_ms": round(t[False], 4), "cublas_plus_elementwise_ms": round(ms_lib, 4),
                     "gbs": round(byts / t[True] / 1e6, 1), "frac_of_copy_bw": round(byts / t[True] / 1e6 / hbm, 3),
                     "peaks": src})
        print(rows[-1], flush=True)
    for M, N, K in [(128, 151936, 4096), (128, 37984, 4096)]:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        t = {}
        for on in (True, False):
            e.set_streamk(2 if on else 0)
            t[on] = timeit(lambda: ops.linear(x, w))
        ms_lib = timeit(lambda: torch.nn.functional.linear(x, w))
        byts = 2.0 * (M * K + N * K + M * N)
        rows.append({"kernel": "lm_head_decode", "M": M, "N": N, "K": K, "stream_k_ms": round(t[True], 4),
                     "one_tile_per_cta_ms": round(t[False], 4), "cublas_ms": round(ms_lib, 4),
                     "gbs": round(byts / t[True] / 1e6, 1), "frac_of_copy_bw": round(byts / t[True] / 1e6 / hbm, 3),
                     "peaks": src})
        print(rows[-1], flush=True)
    e.set_streamk(before)


def bench_decode_attn(rows):
    hbm, tf, src = peaks()
    for B, Hq, Hkv, ctx, bs in [(128, 32, 8, 2304, 256), (128, 32, 8, 4352, 256), (90, 32, 32, 320, 64),
                                (16, 32, 8, 8192, 256), (256, 8, 1, 8448, 256)]:
        D = 128
        nb_per = -(-ctx // bs)
        nb = B * nb_per
        kc = torch.randn(nb, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(nb, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.randperm(nb, device="cuda").int().view(B, nb_per)
        cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: ops.decode_attention(q, kc, vc, bt, cl, D ** -0.5))
        byts = 2.0 * B * ctx * Hkv * D * 2
        rows.append({"kernel": "decode_attn", "B": B, "Hq": Hq, "Hkv": Hkv, "ctx": ctx, "block": bs,
                     "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                     "frac_of_hbm": round(byts / ms / 1e6 / hbm, 3), "peaks": src})
        print(rows[-1], flush=True)


def bench_prefill_attn(rows):
    hbm, tf, src = peaks()
    for nseq, S, Hq, Hkv in [(8, 4096, 32, 8), (1, 640, 32, 32), (1, 32768, 8, 1)]:
        D, bs = 128, 256
        nb_per = -(-S // bs)
        nb = nseq * nb_per
        kc = torch.randn(nb, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(nb, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.arange(nb, device="cuda").int().view(nseq, nb_per)
        q = torch.randn(nseq * S, Hq, D, device="cuda", dtype=torch.bfloat16)
        cu = (torch.arange(nseq + 1, device="cuda") * S).int()
        kl = torch.full((nseq,), S, dtype=torch.int32, device="cuda")
        flops = 4.0 * nseq * Hq * D * S * S / 2
        for impl, name in ((1, "mma.sync"), (2, "tcgen05"), (3, "tcgen05 2-tile")):
            ms = timeit(lambda: ops.prefill_attention(q, kc, vc, bt, cu, kl, D ** -0.5, S, impl), iters=5)
            rows.append({"kernel": "prefill_attn", "impl": name, "seqs": nseq, "S": S, "Hq": Hq, "Hkv": Hkv,
                         "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1),
                         "frac_of_bf16_peak": round(flops / ms / 1e9 / tf, 3), "peaks": src})
            print(rows[-1], flush=True)


def bench_norm(rows):
    hbm, tf, src = peaks()
    for T, H in [(32768, 4096), (128, 4096)]:
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: ops.add_rms_norm(x, r, w, 1e-6))
        byts = 2.0 * T * H * 4
        rows.append({"kernel": "add_rms_norm", "T": T, "H": H, "ms": round(ms, 4),
                     "gbs": round(byts / ms / 1e6, 1), "frac_of_hbm": round(byts / ms / 1e6 / hbm, 3), "peaks": src})
        print(rows[-1], flush=True)


def _bw_row(rows, name, ms, byts, extra):
    hbm, _, src = peaks()
    rows.append(dict({"kernel": name}, **extra, ms=round(ms, 4), gbs=round(byts / ms / 1e6, 1),
                     frac_of_hbm=round(byts / ms / 1e6 / hbm, 3), peaks=src))
    print(rows[-1], flush=True)


def bench_elementwise(rows):
    """Rope + q/k norm + paged store, standalone SwiGLU, embedding gather, sampler (prefill and decode sizes)."""
    from fastcache_b200.ops import reference as ref
    Hq, Hkv, D, bs = 32, 8, 128, 256
    cs = ref.build_cos_sin_cache(D, 8192, 1e6, "cuda")
    qw = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    for T in (32768, 128):
        nb = -(-T // bs) + 1
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        pos = torch.arange(T, device="cuda") % 8192
        slots = torch.randperm(nb * bs, device="cuda")[:T].int()
        kc, vc = (torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        ms = timeit(lambda: ops.rope_qknorm_store(qkv, pos, cs, Hq, Hkv, D, qw, qw, 1e-6, kc, vc, slots))
        byts = 2.0 * T * D * ((Hq + 2 * Hkv) + Hq + 2 * Hkv)
        _bw_row(rows, "rope_qknorm_store", ms, byts, {"T": T, "Hq": Hq, "Hkv": Hkv})
    for T, inter in ((32768, 12288), (128, 12288)):
        x = torch.randn(T, 2 * inter, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: ops.silu_and_mul(x))
        _bw_row(rows, "silu_and_mul", ms, 2.0 * T * inter * 3, {"T": T, "I": inter})
    emb = torch.randn(151936, 4096, device="cuda", dtype=torch.bfloat16)
    for T in (32768, 128):
        ids = torch.randint(0, 151936, (T,), device="cuda")
        ms = timeit(lambda: ops.embedding(ids, emb))
        _bw_row(rows, "embedding", ms, 2.0 * T * 4096 * 2, {"T": T, "H": 4096})
    del emb
    logits = torch.randn(128, 151936, device="cuda", dtype=torch.bfloat16)
    temps = torch.full((128,), 0.6, device="cuda")
    ms = timeit(lambda: ops.sample(logits, temps, seed=1))
    _bw_row(rows, "sample", ms, 2.0 * logits.numel(), {"B": 128, "V": 151936})


def bench_quant(rows, small=False):
    """KV quantisers on the K rows of one layer of the headline decode batch (128 requests x 2304 rows x 8 heads x
    128): codes + scales out, restore, and the one-pass round trip, beside the PyTorch statement on the device."""
    from fastcache_b200.compress import quant
    n = (16 if small else 128) * 2304 * 8
    x = torch.randn(n, 128, device="cuda", dtype=torch.bfloat16)
    for mode, out_bytes in (("int8", 1.0), ("int4", 0.5), ("nf4", 0.5), ("fp8_e4m3", 1.0)):
        ms = timeit(lambda: quant.quantize(x, mode, 128))
        _bw_row(rows, f"quantize_{mode}", ms, x.numel() * (2.0 + out_bytes) + 4.0 * n, {"rows": n, "D": 128})
        packed = quant.quantize(x, mode, 128)
        ms = timeit(lambda: quant.dequantize(packed))
        _bw_row(rows, f"dequantize_{mode}", ms, x.numel() * (2.0 + out_bytes) + 4.0 * n, {"rows": n, "D": 128})
    ms = timeit(lambda: quant.fake_quantize(x, 4, 128))
    _bw_row(rows, "fake_quantize_int4", ms, x.numel() * 4.0, {"rows": n, "D": 128})
    xf = x.float()
    ms = timeit(lambda: (torch.round(xf / (xf.abs().amax(-1, keepdim=True).clamp_min(1e-8) / 127.0))
                         .clamp(-127, 127).to(torch.int8)), iters=5)
    rows.append({"kernel": "quantize_int8 (PyTorch statement on the device, fp32 input)", "ms": round(ms, 4)})
    print(rows[-1], flush=True)


def bench_dense_attn(rows):
    """Vision-tower attention (CLIP 577 x 16 x 64, SigLIP 1024 x 16 x 72) beside torch's fused attention."""
    _, tf, src = peaks()
    for B, S, H, D in [(16, 577, 16, 64), (8, 1024, 16, 72)]:
        qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=torch.bfloat16)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        ms = timeit(lambda: ops.dense_attention(q, k, v, D ** -0.5, None))
        ms_mma = timeit(lambda: ops.dense_attention(q, k, v, D ** -0.5, None, impl=1))
        qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
        ms_lib = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt))
        flops = 4.0 * B * H * S * S * D
        rows.append({"kernel": "dense_attn", "B": B, "S": S, "H": H, "D": D, "ms": round(ms, 4),
                     "mma_sync_kernel_ms": round(ms_mma, 4), "torch_sdpa_ms": round(ms_lib, 4), "tflops": round(flops / ms / 1e9, 1),
                     "frac_of_bf16_peak": round(flops / ms / 1e9 / tf, 3), "peaks": src})
        print(rows[-1], flush=True)


def bench_vit_gemm(rows):
    """Vision-tower GEMMs with bias and the activation in the epilogue (16 images of 577 tokens, CLIP ViT-L)."""
    hbm, tf, src = peaks()
    M = 16 * 577
    for N, K, act in [(3072, 1024, "none"), (1024, 1024, "none"), (4096, 1024, "quick_gelu"), (1024, 4096, "none"),
                      (4096, 4096, "gelu")]:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: ops.linear(x, w, b, act=act))
        ms_lib = timeit(lambda: torch.nn.functional.linear(x, w, b))
        flops = 2.0 * M * N * K
        byts = 2.0 * (M * K + N * K + M * N)
        t_roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3
        rows.append({"kernel": "gemm_vit", "M": M, "N": N, "K": K, "act": act, "ms": round(ms, 4),
                     "cublas_no_act_ms": round(ms_lib, 4), "tflops": round(flops / ms / 1e9, 1),
                     "frac_of_roofline": round(t_roof / ms, 3), "peaks": src})
        print(rows[-1], flush=True)


def _tables(nreq, nb_per):
    perm = torch.randperm(nreq * nb_per).view(nreq, nb_per)
    return [perm[i].tolist() for i in range(nreq)]


def bench_ccm(rows, small=False):
    """Fused CCM merge (gather -> 3 GEMMs -> in-place scatter), LLaVA-1.5-7B shape: 32 layers, 32 KV heads,
    15 requests of 576 image + 64 text rows, factor 4; beside the PyTorch statement of the same operation."""
    from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
    from fastcache_b200.compress.inpool import ccm_compress_in_pool, ccm_compress_reference
    hbm, tf, src = peaks()
    L, H, D, bs, f, nreq, n, img = 32, 32, 128, 256, 4, (4 if small else 15), 640, 576
    nb_per = -(-n // bs)
    m = KVCacheLinearDecoupleCompressor(None, f, 1, n_layer=L, nhead=H, head_dim=D).eval()
    w = m.pack(torch.bfloat16, "cuda")
    pool = torch.randn(L, 2, nreq * nb_per, H, bs, D, device="cuda", dtype=torch.bfloat16)
    tables, lens, imgs = _tables(nreq, nb_per), [n] * nreq, [img] * nreq
    new = ccm_compress_in_pool(pool, tables, lens, imgs, w)
    ms = timeit(lambda: ccm_compress_in_pool(pool, tables, lens, imgs, w), iters=5)

    def torch_statement():
        for bt in tables:
            ccm_compress_reference(pool, bt, n, img, w)
    ms_ref = float("nan") if small else timeit(torch_statement, iters=2, warmup=1)
    rows_in, rows_out = nreq * n, sum(new)
    byts = 2.0 * L * 2 * H * D * (rows_in + rows_out)
    flops = 2.0 * L * 2 * H * (rows_in // f) * (D * f * D + 2 * D * D)
    t_roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3
    rows.append({"kernel": "ccm_merge", "layers": L, "kv_heads": H, "requests": nreq, "rows": n, "factor": f,
                 "ms": round(ms, 4), "torch_statement_ms": round(ms_ref, 3), "gbs": round(byts / ms / 1e6, 1),
                 "tflops": round(flops / ms / 1e9, 1), "frac_of_roofline": round(t_roof / ms, 3), "peaks": src})
    print(rows[-1], flush=True)


def bench_evict(rows, small=False):
    """Scoring + top-k + in-pool compaction, Qwen3-8B shape: 36 layers, 8 KV heads, 8 requests of 4096 rows, keep
    half.  Algorithmic bytes: K read once for the scores, kept K and V rows read and written once."""
    from fastcache_b200.compress.inpool import evict_in_pool
    L, H, Hq, D, bs, nreq, n, w = 36, 8, 32, 128, 256, (2 if small else 8), 4096, 64
    nb_per = n // bs
    pool = torch.randn(L, 2, nreq * nb_per, H, bs, D, device="cuda", dtype=torch.bfloat16)
    tables, lens, kept = _tables(nreq, nb_per), [n] * nreq, [n // 2] * nreq
    wq = [{l: torch.randn(w, Hq, D, device="cuda", dtype=torch.bfloat16) for l in range(L)} for _ in range(nreq)]
    for method, params in (("knorm", {}), ("streaming_llm", {"n_sink": 4}),
                           ("snapkv", {"window": w, "kernel_size": 5}), ("expected_attention", {"n_sink": 4})):
        use_q = wq if method in ("snapkv", "expected_attention") else None
        ms = timeit(lambda: evict_in_pool(pool, tables, lens, method, kept, use_q, params), iters=5)
        k_bytes = 2.0 * L * H * D * nreq * n
        byts = (k_bytes if method != "streaming_llm" else 0.0) + 2 * k_bytes      # kept K, V: half read + half written
        if method == "expected_attention":
            byts += k_bytes                                                         # the score needs the value norms
        _bw_row(rows, "evict_" + method, ms, byts, {"layers": L, "kv_heads": H, "requests": nreq, "rows": n,
                                                    "kept": n // 2})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,decode_gemm,decode_attn,prefill_attn,norm")
    ap.add_argument("--json", default="")
    ap.add_argument("--small", action="store_true", help="capture-sized cases (about 1.5 GB on the device)")
    a = ap.parse_args()
    rows = []
    what = a.what.split(",")
    if "gemm" in what:
        bench_gemm(rows, [(32768, 6144, 4096), (32768, 4096, 4096), (32768, 24576, 4096), (32768, 4096, 12288),
                          (8192, 8192, 8192), (640, 12288, 4096)], "gemm_prefill")
    if "decode_gemm" in what:
        bench_gemm(rows, [(128, 6144, 4096), (128, 4096, 4096), (128, 24576, 4096), (128, 4096, 12288),
                          (128, 151936, 4096), (16, 4096, 4096), (256, 4096, 12288)], "gemm_decode")
    if "swiglu_gemm" in what:
        bench_swiglu_gemm(rows)
    if "decode_attn" in what:
        bench_decode_attn(rows)
    if "prefill_attn" in what:
        bench_prefill_attn(rows)
    if "norm" in what:
        bench_norm(rows)
    if "elementwise" in what:
        bench_elementwise(rows)
    if "quant" in what:
        bench_quant(rows, a.small)
    if "dense_attn" in what:
        bench_dense_attn(rows)
    if "vit_gemm" in what:
        bench_vit_gemm(rows)
    if "ccm" in what:
        bench_ccm(rows, a.small)
    if "evict" in what:
        bench_evict(rows, a.small)
    if a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
