#!/usr/bin/env python
"""Benchmark of the packed T2-g128 decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|gemv|gemv-one] [...]

Prints ONE JSON line (rank 0).  Workloads:
  decode    Bonsai-1.7B-architecture hybrid MTP decode, block size 8, forced
            full-block acceptance, 256-token prompt, 512 new tokens, batch 1,
            CUDA-graph replay (the configuration the headline metric is quoted
            on).  A step is one full generation; value = decode tokens/s.
            --model 4b --accept categorical is the 4B configuration (accepted
            length per step drawn from a seeded categorical with mean 4).
  gemv      Width-specialised GEMV sweep over every Qwen3-1.7B-style layer shape
            and W in {1,2,4,8}; a step is one pass over the sweep;
            value = aggregate algorithmic GB/s.
  gemv-one  One shape / width / consumer, the case the ncu captures use.

Under torchrun (N > 1) every rank runs an independent stream over its own
replica (no data-path collective); value is the sum over ranks divided by the
max-over-ranks time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYER_SHAPES = [("q", 2048, 2048), ("k", 1024, 2048), ("v", 1024, 2048), ("o", 2048, 2048),
                ("gate", 6144, 2048), ("up", 6144, 2048), ("down", 2048, 6144)]
SWEEP_W = (1, 2, 4, 8)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["decode", "gemv", "gemv-one", "gemv-nsplit"])
    ap.add_argument("--shape", default="151936x2048", help="gemv-one: NxK")
    ap.add_argument("--w", type=int, default=1, help="gemv-one: width")
    ap.add_argument("--path", default="auto", choices=["auto", "dp4a", "mma", "rowwarp", "direct"])
    ap.add_argument("--calls", type=int, default=0, help="gemv-one: launches per step")
    ap.add_argument("--pdl", action="store_true",
                    help="gemv workloads: programmatic dependent launch between the calls, as in the decode replay")
    ap.add_argument("--tune", type=int, default=0, help="gemv-one: tuning value passed in bits 8.. of the path")
    ap.add_argument("--mode", default="hybrid", choices=["ar", "conf", "spec", "hybrid"])
    ap.add_argument("--accept", default="forced", choices=["forced", "categorical", "free"],
                    help="decode: accepted length per step (forced = whole block; categorical = seeded "
                         "draw over 1..8 with mean 4; free = measured)")
    ap.add_argument("--model", default="1p7b", choices=["1p7b", "4b", "tiny"])
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="bm_clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx = float(f[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=mx, reasons=sorted(reasons),
                       samples=len(sm))
        return out


# ----------------------------------------------------------------------------- dist
def init_dist(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        if args.impl == "reference":
            return world, rank, local, None
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return world, rank, local, dist
    return world, rank, local, None


def barrier(dist):
    import torch
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(dist, value: float, device) -> float:
    import torch
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, value: float, device) -> float:
    import torch
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------- GEMV workloads
class GemvSet:
    """Device-resident GEMV problems whose weights together exceed L2 several times over,
    so that back-to-back calls always stream from HBM."""

    def __init__(self, device, shapes_w, min_bytes=512 << 20, path=0, seed=0, pdl=False):
        import torch
        from bitmtp_b200 import native, ops
        self.ops, self.native, self.path, self.pdl = ops, native, path, pdl
        self.calls = []
        gen = torch.Generator(device="cpu").manual_seed(seed)
        per_pass = sum(n * k // 4 for (_, n, k, _) in shapes_w)
        self.copies = max(2, -(-min_bytes // per_pass))
        for c in range(self.copies):
            for (name, n, k, w) in shapes_w:
                B = torch.randint(0, 256, (n, k // 4), generator=gen, dtype=torch.int32).to(torch.uint8)
                B = ((B & 0x55) + 0x55).to(torch.uint8).view(torch.int8).to(device)   # codes in {1,2}
                ws = (torch.rand(n, k // 128, generator=gen) * 0.04 + 0.01).to(torch.bfloat16).to(device)
                A = torch.randint(-127, 128, (w, k), generator=gen, dtype=torch.int8).to(device)
                s = (torch.rand(w, generator=gen) * 40 + 20).to(device)
                C = torch.empty(w, n, dtype=torch.bfloat16, device=device)
                self.calls.append((A, B, s, ws, C, w, n, k))
        self.bytes_per_pass = sum(ops.gemv_bytes(w, n, k) for (_, _, _, _, _, w, n, k) in self.calls)

    def run_pass(self):
        for (A, B, s, ws, C, w, n, k) in self.calls:
            self.ops.t2_gemv(A, B, s, ws, path=self.path, out=C, ldc=n, pdl=self.pdl)


def capture(fn, device):
    import torch
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream(device)
    s.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream(device).wait_stream(s)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        fn()
    return g


def time_replays(graph, steps, warmup, dist, device, sampler):
    import torch
    for _ in range(warmup):
        graph.replay()
    barrier(dist)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    barrier(dist)
    clocks = sampler.stop()
    ms = max_over_ranks(dist, e0.elapsed_time(e1), device)
    return ms, clocks


def time_cases(gs, launch, device, reps=10):
    """Per (shape, width) GB/s: for each case a graph of its calls over all weight copies (distinct
    buffers, together larger than L2), CUDA events around `reps` replays.  `launch(call)` issues
    one call on the current stream."""
    import torch
    from bitmtp_b200 import ops
    by_case = {}
    for call in gs.calls:
        by_case.setdefault((call[6], call[7], call[5]), []).append(call)
    out = {}
    for (n, k, w), calls in by_case.items():
        graph = capture(lambda: [launch(c) for c in calls], device)
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) * 1e-3 / (reps * len(calls))
        out[f"{n}x{k}:W{w}"] = {"us": round(sec * 1e6, 2), "gbs": round(ops.gemv_bytes(w, n, k) / sec / 1e9, 1)}
    return out


REFERENCE_WIDTHS = (1, 4, 5, 6, 7, 8, 9, 10, 12, 16, 17)      # widths the reference kernel registers
REFERENCE_SHAPES = {(1024, 2048), (2048, 2048), (4096, 2048), (6144, 2048), (12288, 2048), (2048, 6144),
                    (151936, 2048)}                           # (N, K) of its 1.7B table


def reference_cuda_sweep(shapes_w, device_index=0):
    """The reference's own CUDA GEMV (built from its source into oracle/_ref by oracle/build.py) timed
    on the GPU over the cases of the sweep it registers; None when the library or a GPU is absent.
    Reference arm only: none of this package's kernels run here."""
    import ctypes
    import torch
    from oracle.build import reference_kernel_path
    path = reference_kernel_path()
    if not path or not torch.cuda.is_available():
        return None
    lib = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    lib.t2g128_int8xint2_linear.argtypes = [vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp]
    lib.t2g128_int8xint2_linear.restype = None
    device = torch.device("cuda", device_index)
    torch.cuda.set_device(device)
    cases = [c for c in shapes_w if c[3] in REFERENCE_WIDTHS and (c[1], c[2]) in REFERENCE_SHAPES]
    if not cases:
        return None
    gs = GemvSet(device, cases, min_bytes=768 << 20)

    def launch(call):
        A, B, sc, ws, C, w, n, k = call
        lib.t2g128_int8xint2_linear(A.data_ptr(), B.data_ptr(), C.data_ptr(), sc.data_ptr(), ws.data_ptr(), w, n, k,
                                    torch.cuda.current_stream(device).cuda_stream)

    per_case = time_cases(gs, launch, device)
    tot_b = sum(v["gbs"] * v["us"] for v in per_case.values())
    tot_t = sum(v["us"] for v in per_case.values())
    return {"gbs": round(tot_b / tot_t, 1), "per_case": per_case,
            "what": "the reference's t2g128_kernels.cu compiled for sm_100a with its own flags, same buffers "
                    "and timing protocol as the GPU arm; widths it does not register are left out"}


def cpu_gemv_baseline(shapes_w, budget_s=12.0):
    """The CPU oracle timed on this box's host cores over the same sweep (bounded)."""
    import numpy as np
    from oracle import oracle as O
    from bitmtp_b200 import synthetic
    O.lib()
    total_bytes, total_t, done = 0, 0.0, []
    from bitmtp_b200 import ops
    t_start = time.time()
    for (name, n, k, w) in shapes_w:
        case = synthetic.gemv_case(w, n, k, seed=0)
        A, B = case["A"].numpy(), case["B"].numpy().view(np.uint8)
        ws, s = O.torch_to_u16(case["ws"]), case["s"].numpy()
        O.t2_gemv(A, B, ws, s)
        t0 = time.time()
        reps = 3
        for _ in range(reps):
            O.t2_gemv(A, B, ws, s)
        total_t += (time.time() - t0) / reps
        total_bytes += ops.gemv_bytes(w, n, k)
        done.append(f"{name}:W{w}")
        if time.time() - t_start > budget_s:
            break
    return total_bytes / total_t / 1e9, O.lib().bmo_num_threads(), done


def run_gemv(args, world, rank, local, dist):
    import torch
    from bitmtp_b200 import native, ops
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    path = {"auto": 0, "dp4a": 1, "mma": 2, "rowwarp": 3, "direct": 4}[args.path] | (args.tune << 8)
    if args.workload == "gemv-one":
        n, k = (int(x) for x in args.shape.lower().split("x"))
        shapes_w = [("one", n, k, args.w)]
        min_bytes = 384 << 20
        label = f"gemv-one {n}x{k} W={args.w} path={args.path}"
    else:
        shapes_w = [(nm, n, k, w) for w in SWEEP_W for (nm, n, k) in LAYER_SHAPES]
        min_bytes = 768 << 20
        label = "T2-g128 GEMV sweep, Qwen3-1.7B layer shapes, W in {1,2,4,8}"
    gs = GemvSet(device, shapes_w, min_bytes=min_bytes, path=path, pdl=args.pdl)
    if args.calls:
        gs.calls = gs.calls[: args.calls]
        gs.bytes_per_pass = sum(ops.gemv_bytes(w, n, k) for (_, _, _, _, _, w, n, k) in gs.calls)
    steps = args.steps or 20
    warmup = args.warmup if args.warmup is not None else 5
    graph = capture(gs.run_pass, device)
    sampler = ClockSampler(local)
    ms, clocks = time_replays(graph, steps, warmup, dist, device, sampler)
    err = native.lib().bm_device_error()
    if err:
        raise RuntimeError(f"device error word = {err}")
    launches = len(gs.calls) * steps
    gbs_rank = gs.bytes_per_pass * steps / (ms * 1e-3) / 1e9
    value = sum_over_ranks(dist, gs.bytes_per_pass, device) * steps / (ms * 1e-3) / 1e9

    # e2e: the same pass through the public operator with host activations.
    from bitmtp_b200 import model as M
    host = [(A.cpu().pin_memory(), s.cpu().pin_memory()) for (A, _, s, _, _, _, _, _) in gs.calls]
    h2d = sum(a.numel() + 4 * s_.numel() for a, s_ in host)
    d2h = sum(2 * w * n for (_, _, _, _, _, w, n, _) in gs.calls)
    outs = [torch.empty(w, n, dtype=torch.bfloat16).pin_memory() for (_, _, _, _, _, w, n, _) in gs.calls]

    def e2e_pass():
        for (ha, hs), (A, B, s, ws, C, w, n, k), ho in zip(host, gs.calls, outs):
            a = ha.to(device, non_blocking=True)
            sc = hs.to(device, non_blocking=True)
            y = M.packed_int8_linear(a, B, sc.view(w, 1), ws, validate_registry=False)
            ho.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    e2e_pass()
    barrier(dist)
    t0 = time.time()
    e2e_steps = max(1, min(steps, 5))
    for _ in range(e2e_steps):
        e2e_pass()
    barrier(dist)
    e2e_s = max_over_ranks(dist, time.time() - t0, device)
    e2e_val = sum_over_ranks(dist, gs.bytes_per_pass, device) * e2e_steps / e2e_s / 1e9

    peak, peak_kind = peaks()
    out = {
        "metric": "T2-g128 GEMV algorithmic HBM GB/s", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8 x ternary -> s32",
        "data": "synthetic", "config": {"workload": label, "l2": "weights rotate over "
                                        f"{gs.copies} distinct copies ({gs.copies * sum(n * k // 4 for (_, n, k, _) in shapes_w) >> 20} MiB) > L2",
                                        "timing": "CUDA events around graph replays", "pdl": bool(args.pdl)},
        "gpu_launches": launches, "clocks": clocks,
        "e2e": {"value": round(e2e_val, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "roofline": {"bound": "hbm", "achieved": round(gbs_rank, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(gbs_rank / peak, 4), "traffic": None, "peak_kind": peak_kind,
                     "kernel": "t2_gemv (all launches of the pass)",
                     "frac_of_8TBps": round(gbs_rank / 8000.0, 4)},
    }
    if rank == 0 and world == 1 and args.workload == "gemv":
        out["per_case"] = time_cases(
            gs, lambda c: ops.t2_gemv(c[0], c[1], c[2], c[3], path=path, out=c[4], ldc=c[6], pdl=args.pdl), device)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cores, done = cpu_gemv_baseline(shapes_w)
        out["cpu_baseline"] = {"value": round(v, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                               "sample": f"oracle GEMV on {len(done)} of {len(shapes_w)} sweep cases, 3 reps each"}
    return out


def run_reference_gemv(args, rank):
    """CPU arm: the oracle port of the reference GEMV on all host threads."""
    if rank != 0:
        return None
    steps = args.steps or 3
    warmup = args.warmup if args.warmup is not None else 1
    if args.workload == "gemv-one":
        n, k = (int(x) for x in args.shape.lower().split("x"))
        shapes_w = [("one", n, k, args.w)]
    elif args.workload == "gemv-nsplit":
        shapes_w = [("wide", 28672, 8192, 1), ("wide", 28672, 8192, 8)]
    else:
        shapes_w = [(nm, n, k, w) for w in SWEEP_W for (nm, n, k) in LAYER_SHAPES]
    import numpy as np
    from oracle import oracle as O
    from bitmtp_b200 import synthetic
    # every host core, also under a launcher that exports OMP_NUM_THREADS=1 for its ranks
    O.lib().bmo_set_num_threads(len(os.sched_getaffinity(0)))
    cases = []
    for (name, n, k, w) in shapes_w:
        c = synthetic.gemv_case(w, n, k, seed=0)
        cases.append((c["A"].numpy(), c["B"].numpy().view(np.uint8), O.torch_to_u16(c["ws"]), c["s"].numpy(), w, n, k))
    nbytes = sum(n * k // 4 + n * (k // 128) * 2 + w * k + 4 * w + 2 * w * n for (*_, w, n, k) in cases)

    def one():
        for (A, B, ws, s, w, n, k) in cases:
            O.t2_gemv(A, B, ws, s)

    for _ in range(warmup):
        one()
    t0 = time.time()
    for _ in range(steps):
        one()
    dt = time.time() - t0
    v = nbytes * steps / dt / 1e9
    cores = O.lib().bmo_num_threads()
    ref_cuda = reference_cuda_sweep(shapes_w)
    return {"impl": "reference", "reference_cuda_kernel": ref_cuda,
            "metric": "T2-g128 GEMV algorithmic HBM GB/s", "value": round(v, 3),
            "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8 x ternary -> s32", "data": "synthetic",
            "config": {"workload": "same sweep on host cores (CPU oracle port of the reference kernel)"},
            "cpu_baseline": {"value": round(v, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                             "sample": "full sweep per step"},
            "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    args = parse_args()
    if args.workload is None:
        args.workload = "decode" if os.path.exists(os.path.join(ROOT, "bitmtp_b200", "fast_generate.py")) else "gemv"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        if rank != 0:
            return 0
        if args.workload == "decode":
            from bitmtp_b200.benchmarks import run_reference_decode
            out = run_reference_decode(args)
        else:
            out = run_reference_gemv(args, rank)
        print(json.dumps(out), flush=True)
        return 0
    world, rank, local, dist = init_dist(args)
    if args.workload == "decode":
        from bitmtp_b200.benchmarks import run_decode
        out = run_decode(args, world, rank, local, dist)
    elif args.workload == "gemv-nsplit":
        from bitmtp_b200.benchmarks import run_nsplit
        out = run_nsplit(args, world, rank, local, dist)
    else:
        out = run_gemv(args, world, rank, local, dist)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
