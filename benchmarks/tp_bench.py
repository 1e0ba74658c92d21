"""Device-timed benchmark of the tensor-parallel hot paths against their roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29520 benchmarks/tp_bench.py [--tokens 32768] [--decode-tokens 128] [--json out.json]

One rank per GPU.  The shapes are those of a Qwen3-8B layer split over N ranks
(hidden 4096, q/kv width 6144, ffn 12288).  For prefill-size inputs the timed sequence is the
non-attention part of one layer as the engine runs it:

    o_proj    : GEMM + reduce-scatter + residual add + RMSNorm + all-gather send   (one kernel)
    gate_up   : all-gather wait + GEMM                                             (one kernel)
    SwiGLU
    down_proj : GEMM + reduce-scatter + residual add + RMSNorm + all-gather send   (one kernel)
    qkv       : all-gather wait + GEMM                                             (one kernel)

and the baseline is the same math with this package's GEMM and norm kernels but NCCL all-reduce
in between.  For decode-size inputs the fused path is GEMM into symmetric memory + the one-shot
all-reduce + add + RMSNorm kernel.  Every number is CUDA-event time on the launching stream,
median over iterations, maximum over ranks.  Roofline of a fused op = the slower of its FLOPs at the
measured bf16 peak and its NVLink bytes per GPU at 770 GB/s per direction.
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from fastcache_b200 import ops  # noqa: E402
from fastcache_b200.parallel import symm, tp as tpmod  # noqa: E402

NVLINK_GBS = 770.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def timed(fn, world, iters=8, warmup=3):
    """fn() returns a list of (label, start_event, end_event); returns {label: ms} (median, max over ranks)."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    acc = {}
    for _ in range(iters):
        _flush.zero_()                 # operands start from HBM, not from the 126 MB L2
        dist.barrier()
        torch.cuda.synchronize()
        marks = fn()
        torch.cuda.synchronize()
        for label, a, b in marks:
            acc.setdefault(label, []).append(a.elapsed_time(b))
    out = {}
    for label, xs in acc.items():
        t = torch.tensor([statistics.median(xs)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[label] = float(t.item())
    return out


def ev():
    return torch.cuda.Event(enable_timing=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--decode-tokens", type=int, default=128)
    ap.add_argument("--decode-layers", type=int, default=8)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    rank, local, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), \
        int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tpmod.init_tensor_parallel(world, rank)
    H, QKV, FFN = 4096, 6144, 12288
    T, Td = args.tokens, args.decode_tokens
    hbm, tf, src = peaks()
    comm = symm.enable(max(Td, 256), H, dev, max_tokens=T) if world > 1 else None
    g = torch.Generator(device="cuda").manual_seed(1 + rank)

    def rnd(*shape, scale=0.02):
        return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)

    w_o, w_down = rnd(H, H // world), rnd(H, FFN // world)
    w_qkv, w_gu = rnd(QKV // world, H), rnd(2 * FFN // world, H)
    norm_w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rows = []

    from fastcache_b200.parallel.fused import row_linear_reduce_add_norm

    # ---- decode size: L layers with their own weights in ONE CUDA graph, as the engine runs decode
    # (eager launches of 10-microsecond kernels would time the host, not the device)
    L = args.decode_layers
    layer_w = [(rnd(H, H // world), rnd(2 * FFN // world, H), rnd(H, FFN // world), rnd(QKV // world, H))
               for _ in range(L)]
    attn_d, res_d = rnd(Td, H // world, scale=1.0), rnd(Td, H, scale=1.0)

    def decode_layers(kind):
        res, x = res_d.clone(), attn_d
        if comm is not None and kind.startswith("fused"):
            comm.begin_forward()
        for wo, wgu, wd, wq in layer_w:
            for w_row in (wo, wd):
                if kind.startswith("fused"):
                    normed, res = row_linear_reduce_add_norm(x, w_row, None, res, norm_w, 1e-6)
                else:
                    y = ops.linear(x, w_row)
                    if kind == "nccl" and world > 1:
                        dist.all_reduce(y)
                    normed, res = ops.add_rms_norm(y, res, norm_w, 1e-6)
                if w_row is wo:
                    x = ops.linear_silu_mul(normed, wgu)
            x = ops.linear(normed, wq)[:, :H // world]
        return x

    def graph_ms(kind):
        # variants of the fused path: the reduction inside the GEMM kernel instead of a second kernel, and
        # multimem.ld_reduce through the switch instead of one peer load per rank
        ops.ext().set_fused_epilogues(kind == "fused_one_kernel")
        if comm is not None:
            comm.use_multimem = kind == "fused_multimem" and comm.has_multicast
            if kind == "fused_multimem" and not comm.has_multicast:
                raise RuntimeError("no multicast address for the staging buffers on this system")
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(3):
                decode_layers(kind)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            decode_layers(kind)
        xs = []
        for _ in range(10):
            _flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            xs.append(a.elapsed_time(b))
        t = torch.tensor([statistics.median(xs[2:])], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / L

    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    w_bytes = 2.0 * (H * H + 2 * FFN * H + H * FFN + QKV * H) / world
    drow = {"phase": "decode (CUDA graph)", "tokens": Td, "world": world, "layers_in_graph": L,
            "op": "layer total (4 GEMMs, SwiGLU, 2 x reduce + add + norm)", "peaks": src,
            "roofline_ms": round(w_bytes / (hbm * 1e9) * 1e3, 4)}
    for kind in ("fused", "fused_one_kernel", "fused_multimem", "gemm_only", "nccl"):
        try:
            drow[kind + "_ms"] = round(graph_ms(kind), 4)
        except Exception as exc:               # e.g. a collective that refuses stream capture
            drow[kind + "_ms"] = None
            drow[kind + "_error"] = f"{type(exc).__name__}: {str(exc)[:120]}"
    ops.ext().set_fused_epilogues(False)
    if comm is not None:
        comm.use_multimem = False
    if drow.get("fused_ms"):
        drow["frac_of_roofline"] = round(drow["roofline_ms"] / drow["fused_ms"], 3)
    rows.append(drow)
    if rank == 0:
        print(drow, flush=True)

    for label, tokens in (("prefill", T),):
        attn = rnd(tokens, H // world, scale=1.0)
        res0 = rnd(tokens, H, scale=1.0)

        def fused():
            if comm is not None:
                comm.begin_forward()
            res = res0.clone()
            marks = []
            e = [ev() for _ in range(6)]
            e[0].record()
            normed, res = row_linear_reduce_add_norm(attn, w_o, None, res, norm_w, 1e-6)
            e[1].record()
            gu = ops.linear(normed, w_gu)
            e[2].record()
            act = ops.silu_and_mul(gu)
            e[3].record()
            normed, res = row_linear_reduce_add_norm(act, w_down, None, res, norm_w, 1e-6)
            e[4].record()
            qkv = ops.linear(normed, w_qkv)
            if comm is not None:
                comm.finish_forward(normed)
            e[5].record()
            names = ["o_proj+reduce+add+norm", "gate_up (gathered GEMM)", "swiglu", "down+reduce+add+norm",
                     "qkv (gathered GEMM)"]
            marks = [(n, e[i], e[i + 1]) for i, n in enumerate(names)]
            marks.append(("layer total", e[0], e[5]))
            return marks

        def library():
            res = res0.clone()
            e = [ev() for _ in range(6)]
            e[0].record()
            y = ops.linear(attn, w_o)
            if world > 1:
                dist.all_reduce(y)
            normed, res = ops.add_rms_norm(y, res, norm_w, 1e-6)
            e[1].record()
            gu = ops.linear(normed, w_gu)
            e[2].record()
            act = ops.silu_and_mul(gu)
            e[3].record()
            y = ops.linear(act, w_down)
            if world > 1:
                dist.all_reduce(y)
            normed, res = ops.add_rms_norm(y, res, norm_w, 1e-6)
            e[4].record()
            qkv = ops.linear(normed, w_qkv)
            e[5].record()
            names = ["o_proj+reduce+add+norm", "gate_up (gathered GEMM)", "swiglu", "down+reduce+add+norm",
                     "qkv (gathered GEMM)"]
            marks = [(n, e[i], e[i + 1]) for i, n in enumerate(names)]
            marks.append(("layer total", e[0], e[5]))
            return marks

        def compute_only():
            e = [ev() for _ in range(5)]
            e[0].record()
            ops.linear(attn, w_o)
            e[1].record()
            ops.linear(res0, w_gu)
            e[2].record()
            ops.linear(rnd_act, w_down)
            e[3].record()
            ops.linear(res0, w_qkv)
            e[4].record()
            names = ["o_proj+reduce+add+norm", "gate_up (gathered GEMM)", "down+reduce+add+norm",
                     "qkv (gathered GEMM)"]
            return [(n, e[i], e[i + 1]) for i, n in enumerate(names)] + [("layer total", e[0], e[4])]

        rnd_act = rnd(tokens, FFN // world, scale=1.0)
        t_f = timed(fused, world)
        t_l = timed(library, world)
        t_c = timed(compute_only, world)
        # NVLink bytes each GPU must send for one reduce-scatter + all-gather of [tokens, H] bf16
        link_ms = 2.0 * (world - 1) / world * tokens * H * 2 / (NVLINK_GBS * 1e9) * 1e3 if world > 1 else 0.0
        flops = {"o_proj+reduce+add+norm": 2.0 * tokens * H * H / world,
                 "down+reduce+add+norm": 2.0 * tokens * H * FFN / world,
                 "gate_up (gathered GEMM)": 2.0 * tokens * 2 * FFN * H / world,
                 "qkv (gathered GEMM)": 2.0 * tokens * QKV * H / world}
        for name in t_f:
            row = {"phase": label, "tokens": tokens, "world": world, "op": name, "fused_ms": round(t_f[name], 4),
                   "nccl_ms": round(t_l[name], 4), "gemm_only_ms": round(t_c.get(name, 0.0), 4), "peaks": src}
            if "reduce" in name and comm is not None:
                from fastcache_b200.ops import ext as _ext
                row["reduce_form"] = ("pipelined, in-switch sums" if _ext().tp_pipeline_enabled() and comm.tp_multicast
                                      and _ext().tp_nvls_enabled() else
                                      "pipelined" if _ext().tp_pipeline_enabled() else "one phase after the GEMM")
            if name in flops:
                # the row-parallel kernel sends both the reduce-scatter partials and the all-gather rows
                # (link_ms); the gathered GEMM that follows only waits for them
                link = link_ms if "reduce" in name else 0.0
                roof = max(flops[name] / (tf * 1e12) * 1e3, link)
                row["roofline_ms"] = round(roof, 4)
                row["frac_of_roofline"] = round(roof / t_f[name], 3)
            elif name == "layer total":
                roof = max(sum(flops.values()) / (tf * 1e12) * 1e3, 2 * link_ms)
                row["roofline_ms"] = round(roof, 4)
                row["frac_of_roofline"] = round(roof / t_f[name], 3)
            rows.append(row)
            if rank == 0:
                print(row, flush=True)
    if rank == 0 and args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        json.dump(rows, open(args.json, "w"), indent=1)
    if comm is not None:
        symm.disable()
    tpmod.cleanup_tensor_parallel()


if __name__ == "__main__":
    main()
