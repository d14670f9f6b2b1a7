"""Per-operator timings on seeded synthetic inputs of the benchmark configurations.

    python -m triton_int_b200.microbench --op linear|lnq|gelu|attention|sweep [--iters N] [--rows R] ...

Every line printed is one JSON object: the operator, its shape, the median CUDA-event
time over `--iters` launches (L2 flushed before each launch; problems of M <= 1024
are timed as CUDA-graph replays), the algorithmic work, the achieved rate and its fraction of the
measured peak (MEASURED_PEAKS.json next to the package's parent, else the
fallback 6650 GB/s / 2 x 1400 TOP/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import _lib, synthetic
from .kernels import bmm as KB
from .kernels import fused as KF
from .kernels import linear as KL


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return d["hbm_gbs"], 2.0 * d["bf16_tflops"], "measured"
    return 6650.0, 2.0 * 1590.0, "fallback"


HBM_GBS, INT8_TOPS_BURST, PEAK_SRC = peaks()
_FLUSH = None


def timeit(fn, iters, warm=3, flush=False):
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.int8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _FLUSH.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def timeit_graph(fn, iters, calls=20):
    """Device time per call with the host out of the picture: `calls` launches are captured
    into one CUDA graph and the graph is replayed (small problems finish faster than Python
    can issue them)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(calls):
                fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) / calls)
    ts.sort()
    return ts[len(ts) // 2]


def emit(op, shape, ms, ops=None, nbytes=None, **extra):
    line = {"op": op, "shape": shape, "ms": round(ms, 5)}
    if ops is not None:
        line.update(tops=round(ops / ms / 1e9, 1), frac_of_int8_peak=round(ops / ms / 1e9 / INT8_TOPS_BURST, 4),
                    frac_of_nominal_4500=round(ops / ms / 1e9 / 4500.0, 4))
    if nbytes is not None:
        line.update(gbs=round(nbytes / ms / 1e6, 1), frac_of_hbm=round(nbytes / ms / 1e6 / HBM_GBS, 4),
                    frac_of_nominal_8000=round(nbytes / ms / 1e6 / 8000.0, 4))
    line["peak_source"] = PEAK_SRC
    line.update(extra)
    print(json.dumps(line), flush=True)


def bench_linear(m, n, k, iters, epilogues=("i32", "b8o8", "f32", "geluq"), cublas=True, graph=False):
    g = synthetic.gen(4)
    x, w = synthetic.int8_normal((m, k), 35, g).cuda(), synthetic.int8_normal((n, k), 35, g).cuda()
    b8, bf = synthetic.int8_normal((n,), 35, g).cuda(), torch.randn((n,), generator=g).cuda()
    a, b = torch.tensor(2e-4).cuda(), torch.tensor(0.02).cuda()
    fns = {"i32": lambda: KL.linear_a8_w8_b32_o32(x, w, None),
           "b8o8": lambda: KL.linear_a8_w8_b8_o8(x, w, b8, a, b),
           "f32": lambda: KL.linear_a8_w8_bfp32_ofp32(x, w, bf, a, b),
           "geluq": lambda: KF.linear_a8_w8_bfp32_ofp32_GeLu_Q(x, w, bf, a, torch.tensor(50.0).cuda())}
    for name in epilogues:
        if graph:
            out_bytes = m * n * (1 if name in ("b8o8", "geluq") else 4)
            emit(f"linear_{name}", [m, n, k], timeit_graph(fns[name], iters), ops=2 * m * n * k,
                 nbytes=m * k + n * k + out_bytes, timing="cuda graph replay (device time per call)")
        else:
            # flushed: operands of the mid-size problems fit the L2, and the flush kernel keeps the GPU
            # busy while the host prepares the launch (an idle GPU would count the host's time)
            emit(f"linear_{name}", [m, n, k], timeit(fns[name], iters, flush=True), ops=2 * m * n * k)
    if cublas and m > 16 and m % 8 == 0 and n % 8 == 0 and k % 8 == 0:
        emit("cublaslt_int_mm (torch._int_mm, for comparison)", [m, n, k],
             timeit(lambda: torch._int_mm(x, w.t()), iters, flush=True), ops=2 * m * n * k)


def bench_lnq(rows, hidden, iters):
    c = synthetic.config2_lnq(1, rows=rows, hidden=hidden)
    acc, res, gam, bet = (c[k].cuda() for k in ("acc", "residual", "gamma", "beta"))
    ms = timeit(lambda: KF.dq_add_layernorm_q(acc, c["dq_scale"], res, gam, bet, c["eps"]), iters, flush=True)
    emit("dq_add_layernorm_q", [rows, hidden], ms, nbytes=acc.numel() * 13 + hidden * 8)
    ms = timeit(lambda: KF.layer_norm_fwd_fused_single_pass_q(res, gam, bet, c["eps"]), iters, flush=True)
    emit("layer_norm_q", [rows, hidden], ms, nbytes=acc.numel() * 5 + hidden * 8)


def bench_gelu(rows, cols, iters):
    c = synthetic.config2_gelu(1, rows=rows, cols=cols)
    x = c["x"].cuda()
    y = torch.empty_like(x)
    ms = timeit(lambda: KF.gelu_q(x, c["in_scale"], 1.0 / c["out_scale"], out=y), iters, flush=True)
    emit("gelu_q", [rows, cols], ms, nbytes=x.numel() * 2)


def bench_attention(bh, seq, d, iters):
    c = synthetic.config3_attention(2, bh=bh, seq=seq, head_dim=d)
    q, k, v = c["q"].cuda(), c["k"].cuda(), c["v"].cuda()
    vt = v.transpose(1, 2).contiguous()
    a1, a2 = c["alpha_qk"].cuda(), c["alpha_pv"].cuda()
    s = torch.empty((bh, seq, seq), dtype=torch.float32, device="cuda")
    p = torch.empty((bh, seq, seq), dtype=torch.int8, device="cuda")
    o = torch.empty((bh, seq, d), dtype=torch.int8, device="cuda")
    ops = 2 * bh * seq * seq * d
    for causal in (False, True):
        ms = timeit(lambda: KB.bmm_s8t_s8n_f32t(q, k, a1, out=s, causal=causal), iters)
        emit("bmm_s8t_s8n_f32t" + ("_causal_skip" if causal else ""), [bh, seq, seq, d], ms, ops=ops,
             nbytes=s.numel() * 4 + 2 * q.numel())
    ms = timeit(lambda: KF.causal_softmax_q(s, 127.0, out=p), iters)
    emit("causal_softmax_q", [bh, seq, seq], ms, nbytes=s.numel() * 5)
    ms = timeit(lambda: KB.bmm_s8t_s8n_s8t(p, vt, a2, out=o), iters)
    emit("bmm_s8t_s8n_s8t", [bh, seq, d, seq], ms, ops=ops, nbytes=p.numel() + 2 * o.numel())
    # the fused kernel on the same problem laid out [B, S, h, D] (heads = 32 when bh allows)
    heads = 32 if bh % 32 == 0 else 1
    b = bh // heads
    q4, k4, v4 = (t.view(b, heads, seq, d).permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
    o4 = torch.empty_like(q4)
    ms = timeit(lambda: KF.attention_i8(q4, k4, v4, a1, a2, 127.0, causal=True, out=o4), iters)
    # causal: about half of the score tiles; scores are computed twice, P V once
    emit("attention_i8_fused_causal", [b, seq, heads, d], ms, ops=int(ops * 1.5 * (seq / 128 + 1) / (2 * seq / 128)),
         nbytes=4 * q.numel())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "linear", "lnq", "gelu", "attention", "sweep"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--gelu-rows", type=int, default=16384)
    ap.add_argument("--bh", type=int, default=256)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--epilogues", default="i32,b8o8,f32,geluq")
    ap.add_argument("--no-cublas", action="store_true")
    args = ap.parse_args()
    _lib.load()
    eps = tuple(args.epilogues.split(","))
    if args.op in ("all", "linear"):
        bench_linear(args.m, args.n, args.k, args.iters, eps, not args.no_cublas)
    if args.op in ("all", "lnq"):
        bench_lnq(args.rows, args.hidden, args.iters)
    if args.op in ("all", "gelu"):
        bench_gelu(args.gelu_rows, 16384, args.iters)
    if args.op in ("all", "attention"):
        bench_attention(args.bh, args.seq, 128, max(3, args.iters // 4))
    if args.op == "sweep":
        # config 5: OPT-66B-shape shards of an 8-way tensor-parallel layer
        for layer in ("fc1", "fc2", "qkv"):
            n, k = {"fc1": (4608, 9216), "fc2": (9216, 4608), "qkv": (3456, 9216)}[layer]
            for m in (1, 16, 128, 1024, 4096, 16384):
                bench_linear(m, n, k, args.iters, ("b8o8", "f32"), cublas=False, graph=(m <= 1024))
    st = _lib.device_status()
    if st:
        raise SystemExit(f"device status {st:#x}")


if __name__ == "__main__":
    main()
