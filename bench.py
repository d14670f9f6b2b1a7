#!/usr/bin/env python
"""Benchmark of the INT8 hot path: one OPT-6.7B-shape SmoothQuant decoder block
(hidden 4096, 32 heads, FFN 16384, batch 8 x seq 2048, seeded synthetic data),
tensor-parallel over N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # CPU arm (oracle port)

Prints ONE JSON line on rank 0.  `value` is whole-job tokens/s with the inputs
resident in HBM; `e2e` is the same block driven from pinned host buffers (host to
device copy of the inputs and device to host copy of the outputs inside the timed
region, pipelined over three streams); `roofline` describes the dominant kernel
(the tcgen05 int8 GEMM of the six linears) timed with CUDA events inside the
timed region; `cpu_baseline` is the CPU oracle on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "opt6.7b_int8_decoder_block_tokens_per_s"
UNIT = "tokens/s"
CFG = dict(hidden=4096, heads=32, ffn=16384, batch=8, seq=2048, seed=3)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced shapes (profiling under ncu)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-groups", type=int, default=4,
                    help="host-buffer run: sequence groups per step moving through the upload/compute/download ring")
    ap.add_argument("--tp-mode", default="fused", choices=["fused", "dma", "push", "nccl"],
                    help="N>1: 'push' = row-parallel GEMMs store their tiles into the owners' buffers from the epilogue, "
                         "owner adds locally inside the LayerNorm kernel; 'fused' = LayerNorm kernel pulls the partial "
                         "sums from every peer; 'dma' = partial sums pushed to their owners by the copy engines "
                         "(overlaps another group of sequences' kernels with --microbatches 2); "
                         "'nccl' = int32 all-reduce then LayerNorm")
    ap.add_argument("--microbatches", type=int, default=1,
                    help="N>1, fused exchange: sequences are split into this many groups that run on their own "
                         "streams so one group's exchange overlaps the other's GEMMs")
    return ap.parse_args()


def block_ops(cfg, world=1):
    """Algorithmic int8 ops (2*M*N*K) of the six linears of one block, per rank."""
    t, h, f = cfg["batch"] * cfg["seq"], cfg["hidden"], cfg["ffn"]
    return (2 * t * h * h * 4 + 2 * t * h * f * 2) // world


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
                for n, v in zip(names, s[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
def cpu_block_tokens_per_s(steps, warmup, budget_s=150.0):
    """Times the CPU oracle's block forward on one sequence (batch 1) of config 4; the
    sequence length is the largest of 2048/1024/512/256/128 that keeps the whole run
    within `budget_s`.  Returns (tokens/s, description, cores)."""
    from oracle import block as OB
    from triton_int_b200 import synthetic
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    small = synthetic.config4_block(seed=CFG["seed"], hidden=CFG["hidden"], heads=CFG["heads"], ffn=CFG["ffn"],
                                    batch=1, seq=128)
    t0 = time.perf_counter()
    OB.block_forward(small, small["residual"], small["prev_acc"], 1, 128)
    probe = time.perf_counter() - t0
    seq = 128
    for cand in (2048, 1024, 512, 256):
        est = probe * (cand / 128.0) * 1.15
        if est * (steps + warmup) <= budget_s:
            seq = cand
            break
    p = small if seq == 128 else synthetic.config4_block(seed=CFG["seed"], hidden=CFG["hidden"], heads=CFG["heads"],
                                                         ffn=CFG["ffn"], batch=1, seq=seq)
    for _ in range(warmup):
        OB.block_forward(p, p["residual"], p["prev_acc"], 1, seq)
    t0 = time.perf_counter()
    for _ in range(steps):
        OB.block_forward(p, p["residual"], p["prev_acc"], 1, seq)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return seq / dt, f"config 4 block, batch 1 x seq {seq} ({seq} tokens per step), float64-matmul int32 emulation", cores, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, sample, cores, dt = cpu_block_tokens_per_s(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "configs[3]: OPT-6.7B-shape int8 decoder block, hidden 4096, 32 heads, FFN 16384, "
                               "batch 8 x seq 2048 (CPU arm runs a bounded sample of it)"},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def run_b200(args):
    import torch.distributed as dist
    from triton_int_b200 import _lib, synthetic
    from triton_int_b200.kernels import _gemm
    from triton_int_b200.nn.decoder import Int8DecoderBlock

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    if not _lib.load().ti_device_supported():
        raise SystemExit("sm_100a device required")

    cfg = dict(CFG)
    if args.small:
        cfg.update(batch=2, seq=1024)
    p = synthetic.config4_block(seed=cfg["seed"], hidden=cfg["hidden"], heads=cfg["heads"], ffn=cfg["ffn"],
                                batch=cfg["batch"], seq=cfg["seq"])
    tokens = cfg["batch"] * cfg["seq"]

    def reduce_fn(t):
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t

    block = Int8DecoderBlock(p, rank=rank, world=world, reduce_fn=reduce_fn).to(dev)
    residual_h = p["residual"].pin_memory()
    acc_h = p["prev_acc"].pin_memory()
    residual, prev_acc = residual_h.to(dev), acc_h.to(dev)
    del p
    tp_mode = "single" if world == 1 else args.tp_mode
    bufs = None
    nmb = 1
    if tp_mode in ("fused", "push", "dma"):
        # residual stream row-sharded; the int32 partial sums and the gathered int8
        # activations live in peer-mapped buffers, one set per group of sequences
        from triton_int_b200 import tp
        nmb = max(1, min(args.microbatches, cfg["batch"]))
        while cfg["batch"] % nmb:
            nmb -= 1
        try:
            bufs = [tp.SymmetricBuffers(dist.group.WORLD, tokens // nmb, cfg["hidden"], dev) for _ in range(nmb)]
        except Exception as exc:  # symmetric memory not available on this box
            if rank == 0:
                print(f"[bench] symmetric memory unavailable ({exc}); using the NCCL all-reduce path", file=sys.stderr)
            tp_mode = "nccl"
    if tp_mode in ("fused", "push", "dma"):
        mb_tokens = tokens // nmb
        r0, rc = bufs[0].rank_rows()
        state = []
        for i in range(nmb):
            lo = i * mb_tokens
            state.append(residual[lo + r0:lo + r0 + rc].contiguous())
            bufs[i].partial[0][0].zero_()
            if tp_mode in ("push", "dma"):
                # receive-buffer layout [world][rows/world][H]: the previous block's slices, all in slot 0
                bufs[i].partial[0][0].view(world, rc, cfg["hidden"])[0].copy_(prev_acc[lo + r0:lo + r0 + rc])
            elif rank == 0:
                bufs[i].partial[0][0].copy_(prev_acc[lo:lo + mb_tokens])   # the previous block's partial sums: all on rank 0 here
        # the first group's stream has priority, so the groups fall out of step and one group's
        # copies run under the other's kernels instead of both copying at the same time
        side = [torch.cuda.Stream(dev, priority=(-1 if (nmb > 1 and i == 0) else 0)) for i in range(nmb)]
        comm = [torch.cuda.Stream(dev, priority=-1) for _ in range(nmb)]
        torch.cuda.synchronize()
        dist.barrier()

    # ---- per-launch timing of the dominant kernel: wrap the GEMM launcher with events
    gemm_events = []
    orig_gemm = _gemm.gemm
    record = {"on": False}

    def timed_gemm(a3, b3, *a, **kw):
        if record["on"] and a3.shape[0] == 1:  # the six linears (batch == 1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = orig_gemm(a3, b3, *a, **kw)
            e.record()
            gemm_events.append((s, e))
            return out
        return orig_gemm(a3, b3, *a, **kw)

    import triton_int_b200.kernels.linear as KL
    import triton_int_b200.kernels.fused as KF
    KL.gemm = timed_gemm
    KF.gemm = timed_gemm

    def step():
        if tp_mode in ("fused", "push", "dma"):
            # chained like a stack of blocks: the fc2 partial sums left in the peer-mapped
            # buffer are the next step's input, the residual shard carries over.  Each group
            # of sequences runs on its own stream.
            main = torch.cuda.current_stream(dev)
            for i in range(nmb):
                side[i].wait_stream(main)
                with torch.cuda.stream(side[i]):
                    if tp_mode == "dma":
                        state[i] = block.forward_tp_dma(state[i], bufs[i], cfg["batch"] // nmb, cfg["seq"], comm[i])
                    else:
                        fwd = block.forward_tp_push if tp_mode == "push" else block.forward_tp_fused
                        state[i] = fwd(state[i], bufs[i], cfg["batch"] // nmb, cfg["seq"])
            for i in range(nmb):
                main.wait_stream(side[i])
                if tp_mode == "dma":
                    main.wait_stream(comm[i])
            return state
        return block(residual, prev_acc, cfg["batch"], cfg["seq"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = _lib.launch_count()
    record["on"] = True
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    record["on"] = False
    launches = _lib.launch_count() - launches0
    ms_total = ev0.elapsed_time(ev1)
    gemm_ms = sum(s.elapsed_time(e) for s, e in gemm_events)
    n_gemm = len(gemm_events)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.device_status()
    if status:
        raise SystemExit(f"device status {status:#x}: a bounded wait expired during the benchmark")

    # ---- end to end from host buffers: H2D inputs, block, D2H outputs, three streams
    e2e = None
    if not args.no_e2e:  # (host-buffer run uses the all-reduce form of the step at every N)
        e2e = run_e2e(block, residual_h, acc_h, cfg, dev, world, dist, max(3, args.steps), barrier, args.e2e_groups)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = measured_peaks()
    ms_per_step = ms_total / args.steps
    value = tokens / (ms_per_step * 1e-3)
    ops_per_launch = block_ops(cfg, world) / 6.0
    achieved = (block_ops(cfg, world) * args.steps) / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "configs[3]: OPT-6.7B-shape int8 decoder block, hidden 4096, 32 heads, FFN 16384, "
                               f"batch {cfg['batch']} x seq {cfg['seq']} = {tokens} tokens per step",
                   "parallelism": f"tp{world}", "tp_exchange": tp_mode, "microbatches": nmb, "global_batch": cfg["batch"], "seq_len": cfg["seq"],
                   "l2": "working set (>= 5 GB of activations, 201 MB of weights) exceeds the 126 MB L2; no flush",
                   "rounding": "rne_sat"},
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "roofline": {
            "bound": "tensor", "kernel": "gemm_i8_tcgen05_pair_kernel (six linears of the block, CTA pairs)",
            "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
            "frac": (achieved / int8_peak) if achieved else None,
            "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}): int8 tensor rate is twice bf16",
            "frac_of_nominal_4500": (achieved / 4500.0) if achieved else None,
            "launches_timed": n_gemm, "avg_launch_ms": gemm_ms / n_gemm if n_gemm else None,
            "ops_per_launch_avg": ops_per_launch,
            # ncu capture of the q/k/v-shape launch (16384 x 4096 x 4096, int8 out): 84.0 MB read +
            # 43.1 MB written to DRAM against 151 MB algorithmic (part of the output was still in L2)
            "traffic": (127.1e6 if (world == 1 and not args.small) else None),
            "traffic_note": "dram__bytes_read+write of one q/k/v-shape launch (profiles/gemm_i8_tcgen05_16384x4096x4096.md); "
                            "algorithmic bytes of that launch: 151 MB",
        },
    }
    if not args.no_cpu_baseline and world == 1 and not args.small:
        tps, sample, cores, _ = cpu_block_tokens_per_s(1, 0, budget_s=25.0)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(block, residual_h, acc_h, cfg, dev, world, dist, steps, barrier, want_groups=4):
    """Same block, inputs in pinned host memory: every step copies both inputs to the
    device, runs the block and copies both outputs back.  A step moves as groups of
    sequences (sequences are independent of one another in a decoder block): uploads,
    kernels and downloads run on three streams over a ring of group-sized buffers, so
    one group's upload and another's download overlap a third's kernels, and the
    pipeline's fill and drain cost one group, not one step."""
    tokens = cfg["batch"] * cfg["seq"]
    groups = max(1, min(want_groups, cfg["batch"]))
    while cfg["batch"] % groups:
        groups -= 1
    gb = cfg["batch"] // groups          # sequences per group
    gt = gb * cfg["seq"]                 # tokens per group
    ring = 3
    h2d, d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    comp = torch.cuda.current_stream(dev)
    hid = residual_h.shape[-1]
    din = [(torch.empty((gt, hid), dtype=residual_h.dtype, device=dev),
            torch.empty((gt, hid), dtype=acc_h.dtype, device=dev)) for _ in range(ring)]
    hout = [(torch.empty((gt, hid), dtype=residual_h.dtype).pin_memory(),
             torch.empty((gt, hid), dtype=acc_h.dtype).pin_memory()) for _ in range(ring)]
    up_done = [torch.cuda.Event() for _ in range(ring)]
    in_free = [torch.cuda.Event() for _ in range(ring)]
    out_ready = [torch.cuda.Event() for _ in range(ring)]
    out_free = [torch.cuda.Event() for _ in range(ring)]

    def upload(j):
        b, g = j % ring, j % groups
        with torch.cuda.stream(h2d):
            h2d.wait_event(in_free[b])
            din[b][0].copy_(residual_h[g * gt:(g + 1) * gt], non_blocking=True)
            din[b][1].copy_(acc_h[g * gt:(g + 1) * gt], non_blocking=True)
            up_done[b].record(h2d)

    def run(n):
        total = n * groups
        for b in range(ring):
            in_free[b].record(comp)
            out_free[b].record(d2h)
        for j in range(min(ring - 1, total)):
            upload(j)
        for j in range(total):
            b = j % ring
            if j + ring - 1 < total:
                upload(j + ring - 1)
            comp.wait_event(up_done[b])
            comp.wait_event(out_free[b])
            r, a = block(din[b][0], din[b][1], gb, cfg["seq"])
            in_free[b].record(comp)
            out_ready[b].record(comp)
            with torch.cuda.stream(d2h):
                d2h.wait_event(out_ready[b])
                hout[b][0].copy_(r, non_blocking=True)
                hout[b][1].copy_(a, non_blocking=True)
                out_free[b].record(d2h)
                r.record_stream(d2h)
                a.record_stream(d2h)

    run(2)
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(comp)
    run(steps)
    comp.wait_stream(d2h)
    t1.record(comp)
    barrier()
    ms = t0.elapsed_time(t1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    nbytes = residual_h.numel() * 4 + acc_h.numel() * 4
    return {"value": tokens / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "steps": steps,
            "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
            "note": "pinned host buffers; upload, kernels and download pipelined on three streams in %d groups "
                    "of %d sequences per step" % (groups, gb)}


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
