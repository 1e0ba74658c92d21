"""Device-timed micro-benchmarks of the hot kernels against the measured roofline.

Usage:  python benchmarks/kernel_bench.py [--what gemm,decode_gemm,decode_attn,prefill_attn,norm] [--json out.json]
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
        rows.append({"kernel": tag, "M": M, "N": N, "K": K, "ms": round(ms, 4), "cublas_ms": round(ms_lib, 4),
                     "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
                     "frac_of_roofline": round(t_roof / ms, 3), "peaks": src})
        print(rows[-1], flush=True)


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,decode_gemm,decode_attn,prefill_attn,norm")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    rows = []
    what = a.what.split(",")
    if "gemm" in what:
        bench_gemm(rows, [(32768, 6144, 4096), (32768, 4096, 4096), (32768, 24576, 4096), (32768, 4096, 12288),
                          (8192, 8192, 8192), (640, 12288, 4096)], "gemm_prefill")
    if "decode_gemm" in what:
        bench_gemm(rows, [(128, 6144, 4096), (128, 4096, 4096), (128, 24576, 4096), (128, 4096, 12288),
                          (128, 151936, 4096), (16, 4096, 4096), (256, 4096, 12288)], "gemm_decode")
    if "decode_attn" in what:
        bench_decode_attn(rows)
    if "prefill_attn" in what:
        bench_prefill_attn(rows)
    if "norm" in what:
        bench_norm(rows)
    if a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
