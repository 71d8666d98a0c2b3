#!/usr/bin/env python
"""Benchmark of the packed T2-g128 decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|gemv|gemv-one|gemv-nsplit] [...]

Prints ONE JSON line (rank 0).  Workloads:
  decode       Bonsai-1.7B-architecture hybrid MTP decode, block size 8, forced
               full-block acceptance, 256-token prompt, 512 new tokens, batch 1,
               CUDA-graph replay (the configuration the headline metric is quoted
               on).  A step is one full generation; value = decode tokens/s.  The
               line also carries the per-shape GEMV table (`gemv_table`) and, under
               torchrun, the wide-layer N-split (`nsplit`) and the 4B categorical
               configuration (`streams_4b_categorical`).
               --model 4b --accept categorical is that 4B configuration by itself.
  gemv         Width-specialised GEMV sweep over every Qwen3-1.7B-style layer shape
               and W in {1,2,4,8}; value = aggregate algorithmic GB/s.
  gemv-one     One shape / width / consumer, the case the ncu captures use.
  gemv-nsplit  The 8192 -> 28672 layer split by rows over the ranks.

--impl reference times the CPU side of the same workload on the host cores: per step one
full-depth forward of the CPU oracle port at the replay width the workload runs at, with
the reference's own CUDA GEMV (built into oracle/_ref) and, where the reference's Python
is installed under baseline/_ref, its own CPU linear path and its own GPU decode loops
attached as extra keys.

Under torchrun (N > 1) every rank runs an independent request stream over its own
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
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYER_SHAPES = [("q", 2048, 2048), ("k", 1024, 2048), ("v", 1024, 2048), ("o", 2048, 2048),
                ("gate", 6144, 2048), ("up", 6144, 2048), ("down", 2048, 6144)]
SWEEP_W = (1, 2, 4, 8)
# (N, K) of the per-shape table: the layer shapes of the sweep configuration, the merged shapes a
# replay actually launches, the packed head and the wide stress layer
TABLE_SHAPES = [(1024, 2048), (2048, 2048), (4096, 2048), (6144, 2048), (12288, 2048), (2048, 6144),
                (151936, 2048), (28672, 8192)]
TABLE_W = (1, 8)
GEOMETRIES = {"1p7b": "BONSAI_1P7B", "4b": "BONSAI_4B", "tiny": "TINY"}
D8_WIDTHS = (1, 8, 9, 10, 12, 16, 17)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "gemv", "gemv-one", "gemv-nsplit", "attention", "prompt-gemm"])
    ap.add_argument("--shape", default="151936x2048", help="gemv-one: NxK")
    ap.add_argument("--w", type=int, default=1, help="gemv-one, attention: width")
    ap.add_argument("--cache-len", type=int, default=700, help="attention: history rows")
    ap.add_argument("--layers", type=int, default=28, help="attention: dependent launches per graph, one K/V plane each")
    ap.add_argument("--rows", type=int, default=256, help="prompt-gemm: prompt rows")
    ap.add_argument("--path", default="auto", choices=["auto", "dp4a", "mma", "rowwarp", "direct"])
    ap.add_argument("--calls", type=int, default=0, help="gemv-one: launches per step")
    ap.add_argument("--pdl", action="store_true",
                    help="gemv workloads: programmatic dependent launch between the calls, as in the decode replay")
    ap.add_argument("--mode", default="hybrid", choices=["ar", "conf", "spec", "hybrid"])
    ap.add_argument("--accept", default="forced", choices=["forced", "categorical", "free"],
                    help="decode: accepted length per step (forced = whole block; categorical = seeded "
                         "draw over 1..8 with mean 4; free = measured)")
    ap.add_argument("--model", default="1p7b", choices=["1p7b", "4b", "tiny"])
    ap.add_argument("--draft-head", default="native", choices=["native", "fp8", "bf16"],
                    help="decode: head of the draft role (native = packed T2; fp8 / bf16 = dense tied head)")
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="decode: skip the per-shape GEMV table and the multi-GPU extra keys")
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


def gemv_alg_bytes(W: int, N: int, K: int, esz: int = 2) -> int:
    """Algorithmic bytes of one T2-g128 GEMV: codes + scales + INT8 activations + multipliers + output."""
    return N * K // 4 + N * (K // 128) * 2 + W * K + 4 * W + esz * W * N


# DRAM traffic of the GEMV kernels relative to their algorithmic bytes, from the ncu captures summarised
# under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum per launch over bm_t2_gemv_bytes):
# cooperative-tile kernel on 4096 x 2048 at width 16: 2.31 MB measured for 2.40 MB algorithmic (the INT8
# activations and part of the scales come from L2); row-per-warp kernel on the head at width 1: 83.6 MB
# for 83.0 MB.  Traffic grows with the rows of the weight matrix, so a launch of another shape is scaled
# by its algorithmic bytes.
DRAM_TRAFFIC_RATIO = {"cooperative": 2.31 / 2.40, "rowwarp": 83.6 / 83.0}


# ----------------------------------------------------------------------------- GEMV workloads
class GemvSet:
    """Device-resident GEMV problems whose weights together exceed L2 several times over,
    so that back-to-back calls always stream from HBM.  Generated on the device: only the
    distribution matters for timing (codes uniform over {1,2,3}, scales U[0.01,0.05])."""

    def __init__(self, device, shapes_w, min_bytes=512 << 20, path=0, seed=0, pdl=False):
        import torch
        from bitmtp_b200 import synthetic        # pure torch: the reference arm builds its buffers here too
        self.path, self.pdl = path, pdl
        self.calls = []
        gen = torch.Generator(device=device).manual_seed(seed)
        per_pass = sum(n * k // 4 for (_, n, k, _) in shapes_w)
        self.copies = max(2, -(-min_bytes // per_pass))
        for c in range(self.copies):
            for (name, n, k, w) in shapes_w:
                B, ws = synthetic.device_ternary(n, k, gen, device)
                A = torch.randint(-127, 128, (w, k), generator=gen, device=device, dtype=torch.int8)
                s = torch.rand(w, generator=gen, device=device) * 40 + 20
                C = torch.empty(w, n, dtype=torch.bfloat16, device=device)
                self.calls.append((A, B, s, ws, C, w, n, k))
        self.bytes_per_pass = sum(gemv_alg_bytes(w, n, k) for (_, _, _, _, _, w, n, k) in self.calls)

    def run_pass(self):
        from bitmtp_b200 import ops
        for (A, B, s, ws, C, w, n, k) in self.calls:
            ops.t2_gemv(A, B, s, ws, path=self.path, out=C, ldc=n, pdl=self.pdl)


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


def time_graph(graph, calls: int, reps: int = 10) -> float:
    """Seconds per call of a captured graph of `calls` launches: CUDA events on the launching stream
    around `reps` replays after 3 warm-up replays."""
    import torch
    for _ in range(3):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (reps * calls)


def time_cases(gs, launch, device, reps=10):
    """Per (shape, width) GB/s: for each case a graph of its calls over all weight copies (distinct
    buffers, together larger than L2).  `launch(call)` issues one call on the current stream."""
    by_case = {}
    for call in gs.calls:
        by_case.setdefault((call[6], call[7], call[5]), []).append(call)
    out = {}
    for (n, k, w), calls in by_case.items():
        graph = capture(lambda: [launch(c) for c in calls], device)
        sec = time_graph(graph, len(calls), reps)
        out[f"{n}x{k}:W{w}"] = {"us": round(sec * 1e6, 2), "gbs": round(gemv_alg_bytes(w, n, k) / sec / 1e9, 1)}
    return out


def gemv_table(device, launchers, shapes=TABLE_SHAPES, widths=TABLE_W, min_bytes=320 << 20):
    """The metric's second half: per (N x K, W) the time and algorithmic GB/s of one GEMV launch, over
    weights that rotate through more than L2 of distinct copies, for each named launcher.  A launcher
    maps a GemvSet to a function issuing one launch on the current stream (or None when it does not
    serve the case); every launcher sees the same buffers."""
    import torch
    peak, _ = peaks()
    table = {}
    for (n, k) in shapes:
        for w in widths:
            gs = GemvSet(device, [("t", n, k, w)], min_bytes=min_bytes, seed=n + w)
            row = {"bytes": gemv_alg_bytes(w, n, k)}
            for name, make in launchers.items():
                launch = make(gs, n, k, w)
                if launch is None:
                    continue
                graph = capture(lambda: [launch(c) for c in gs.calls], device)
                sec = time_graph(graph, len(gs.calls))
                gbs = row["bytes"] / sec / 1e9
                row[name] = {"us": round(sec * 1e6, 2), "gbs": round(gbs, 1), "frac_of_measured": round(gbs / peak, 4),
                             "frac_of_8TBps": round(gbs / 8000.0, 4)}
                del graph
            table[f"{n}x{k}:W{w}"] = row
            del gs
            torch.cuda.empty_cache()
    return table


def our_gemv_launchers():
    """`isolated`: the drop-in call on natural-order INT8 rows, launches back to back with no overlap;
    `chained`: GEMV-ready activations and programmatic dependent launch between consecutive calls, as a
    decode replay issues them."""
    import torch
    from bitmtp_b200 import ops

    def isolated(gs, n, k, w):
        return lambda c: ops.t2_gemv(c[0], c[1], c[2], c[3], out=c[4], ldc=n)

    def chained(gs, n, k, w):
        if k % 256:
            return None
        dev = gs.calls[0][0].device
        prep = torch.randint(-127, 128, (w, k), device=dev, dtype=torch.int8)
        asum = torch.randint(-4000, 4000, (w, k // 128), device=dev, dtype=torch.int32)
        return lambda c: ops.t2_gemv_prepared(prep, asum, c[1], c[2], c[3], out=c[4], ldc=n, pdl=True)

    return {"isolated": isolated, "chained": chained}


REFERENCE_WIDTHS = (1, 4, 5, 6, 7, 8, 9, 10, 12, 16, 17)      # widths the reference kernel registers
REFERENCE_SHAPES = {(1024, 2048), (2048, 2048), (4096, 2048), (6144, 2048), (12288, 2048), (2048, 6144),
                    (151936, 2048)}                           # (N, K) of its 1.7B table


def reference_kernel_lib():
    """ctypes handle of the reference's own CUDA GEMV (built from its source into oracle/_ref by
    oracle/build.py), or None.  Reference arm only."""
    import ctypes
    from oracle.build import reference_kernel_path
    path = reference_kernel_path()
    if not path:
        return None
    lib = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    lib.t2g128_int8xint2_linear.argtypes = [vp, vp, vp, vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, vp]
    lib.t2g128_int8xint2_linear.restype = None
    return lib


def reference_cuda_table(shapes_w=None):
    """The reference's CUDA kernel timed on the GPU with the buffers and protocol of `gemv_table`
    (cases it registers only).  None when the library or a GPU is absent."""
    import torch
    if not torch.cuda.is_available():
        return None
    lib = reference_kernel_lib()
    if lib is None:
        return None
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)

    def ref(gs, n, k, w):
        if w not in REFERENCE_WIDTHS or (n, k) not in REFERENCE_SHAPES:
            return None

        def launch(c):
            A, B, sc, ws, C, w_, n_, k_ = c
            lib.t2g128_int8xint2_linear(A.data_ptr(), B.data_ptr(), C.data_ptr(), sc.data_ptr(), ws.data_ptr(),
                                        w_, n_, k_, torch.cuda.current_stream(device).cuda_stream)
        return launch

    if shapes_w is None:
        table = gemv_table(device, {"reference_kernel": ref})
    else:
        table = {}
        for (n, k, w) in shapes_w:
            table.update(gemv_table(device, {"reference_kernel": ref}, shapes=[(n, k)], widths=[w]))
    table = {key: row for key, row in table.items() if "reference_kernel" in row}
    return {"per_case": table,
            "what": "the reference's t2g128_kernels.cu compiled for sm_100a with its own flags; same buffers "
                    "and timing protocol as gemv_table.isolated of the GPU arm; cases it does not register "
                    "are left out"}


def cpu_gemv_baseline(shapes_w, budget_s=12.0):
    """The CPU oracle timed on this box's host cores over the same sweep (bounded)."""
    import numpy as np
    from oracle import oracle as O
    from bitmtp_b200 import synthetic
    O.lib()
    total_bytes, total_t, done = 0, 0.0, []
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
        total_bytes += gemv_alg_bytes(w, n, k)
        done.append(f"{name}:W{w}")
        if time.time() - t_start > budget_s:
            break
    return total_bytes / total_t / 1e9, O.lib().bmo_num_threads(), done


def run_gemv(args, world, rank, local, dist):
    import torch
    from bitmtp_b200 import native, ops
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    path = {"auto": 0, "dp4a": 1, "mma": 2, "rowwarp": 3, "direct": 4}[args.path]
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
        gs.bytes_per_pass = sum(gemv_alg_bytes(w, n, k) for (_, _, _, _, _, w, n, k) in gs.calls)
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
                     "frac": round(gbs_rank / peak, 4),
                     "traffic": round(gs.bytes_per_pass / len(gs.calls) * DRAM_TRAFFIC_RATIO["cooperative"]),
                     "traffic_note": "average algorithmic bytes per launch x the DRAM/algorithmic ratio ncu measured "
                                     "for the cooperative-tile kernel (profiles/)",
                     "peak_kind": peak_kind, "kernel": "t2_gemv (all launches of the pass)",
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
    """CPU arm of the GEMV workloads: the oracle port of the reference GEMV on all host threads."""
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
    nbytes = sum(gemv_alg_bytes(w, n, k) for (*_, w, n, k) in cases)

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
    ref_cuda = reference_cuda_table([(n, k, w) for (_, n, k, w) in shapes_w])
    return {"impl": "reference", "reference_cuda_kernel": ref_cuda,
            "metric": "T2-g128 GEMV algorithmic HBM GB/s", "value": round(v, 3),
            "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8 x ternary -> s32", "data": "synthetic",
            "config": {"workload": "same sweep on host cores (CPU oracle port of the reference kernel)"},
            "cpu_baseline": {"value": round(v, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                             "sample": "full sweep per step"},
            "e2e": {"value": round(v, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


# ----------------------------------------------------------------------------- decode workload
def decode_shape(args):
    """(prompt_len, new_tokens, segment ladder, replay width that dominates the mode)."""
    prompt_len = args.prompt_len or (512 if args.model == "4b" else 256)
    new_tokens = args.new_tokens or 512
    need = prompt_len + new_tokens + max(D8_WIDTHS)
    ladder = tuple(s for s in (256, 1024, 4096) if s >= need)[:1] or (4096,)
    width = 16 if args.mode in ("hybrid", "conf") else (1 if args.mode == "ar" else 9)
    return prompt_len, new_tokens, ladder, width


def decode_metric(args) -> str:
    return ("decode tok/s (Bonsai-1.7B-arch D8, bs1)" if args.model == "1p7b"
            else f"decode tok/s (Bonsai-{args.model}-arch D8, bs1 per GPU)")


def decode_config(args, world: int) -> dict:
    """The `config` of a decode line; both arms print the same dictionary."""
    prompt_len, new_tokens, ladder, _ = decode_shape(args)
    accept_words = {"forced": "forced full-block acceptance", "free": "measured acceptance",
                    "categorical": "accepted length per step drawn from a seeded categorical over 1..8 "
                                   "(p ~ 0.9083^k, mean 4)"}[args.accept]
    head = {"native": "native packed T2 head for draft and verify",
            "fp8": "dense e4m3 tied head for the draft role, native packed T2 head for verify",
            "bf16": "dense bf16 tied head for the draft role, native packed T2 head for verify"}[args.draft_head]
    return {"workload": f"Bonsai-{args.model}-architecture {args.mode} MTP decode, random-init ternary "
                        f"weights, block 8, {accept_words}, {prompt_len}-token random "
                        f"prompt, {new_tokens} new tokens, batch 1, CUDA-graph replay, {head}",
            "segment": ladder[0], "widths": list(D8_WIDTHS),
            "timing": "value = timed decode tokens / decode seconds as the reference defines them "
                      "(first token and prefill excluded, host clock between device synchronisations); "
                      "ms_per_step and e2e = CUDA events around whole generate calls (prefill + all new tokens, "
                      "host prompt in, tokens out)",
            "l2": "the packed weights and scales streamed per replay (459 MB for the 1.7B geometry) are > 3x L2",
            "one_request_stream_per_gpu": world > 1}


class _ReplayCounter:
    """Stands in for a CapturedGraph's cuda_graph: forwards replay() and counts the calls."""

    def __init__(self, graph):
        self.graph, self.replays = graph, 0

    def replay(self):
        self.replays += 1
        self.graph.replay()

    def __getattr__(self, name):
        return getattr(self.graph, name)


def build_decode(model_name: str, device, prompt_len: int, new_tokens: int, seed: int = 0, draft_head: str = "native"):
    """(model, atlas, cfg) for a synthetic checkpoint of the named geometry."""
    from bitmtp_b200 import generate, synthetic
    from bitmtp_b200.fast_runtime import GraphAtlas
    geometry = getattr(synthetic, GEOMETRIES[model_name])
    cfg = synthetic.make_config(geometry, block_size=8)
    sd = synthetic.device_state(cfg, device, seed=seed)
    head_w, head_s = sd.pop("_head.weight"), sd.pop("_head.weight_scale")
    model = generate.model_from_state(generate.args_from_config(cfg), sd, device)
    n_pad = (cfg["vocab_size"] + 31) // 32 * 32
    if n_pad != cfg["vocab_size"]:
        model.prepare_t2_lm_head()
    else:
        model._lm_head_t2_w, model._lm_head_t2_scale = head_w, head_s
        model._lm_head_t2_vocab, model._lm_head_n_pad = cfg["vocab_size"], n_pad
    need = prompt_len + new_tokens + max(D8_WIDTHS)
    ladder = tuple(s for s in (256, 1024, 4096) if s >= need)[:1] or (4096,)
    model.prepare_merged_weights(max_positions=ladder[0] + max(D8_WIDTHS))
    draft_role = {"native": "draft", "fp8": "draft_fp8", "bf16": "draft_bf16"}[draft_head]
    atlas = GraphAtlas(model, model.args, device, segment_ladder=ladder, m_set=D8_WIDTHS,
                       roles=("ar", draft_role, "verify"), capture_verbose=False)
    return model, atlas, cfg


def replay_gemv_roofline(model, M: int, device, steps: int = 20):
    """Average device time of the GEMV launches of one width-M replay, measured live: the
    same calls on the model's own weights (layer l, then l+1, ...: 376 MB of distinct
    weights per pass, three times L2), captured in one graph and replayed."""
    import torch
    from bitmtp_b200 import native, ops
    a = model.args
    W = model.workspace(M)
    rows = a.block_size if M > a.block_size + 1 else M     # logit rows of a draft / verify / AR replay
    logits = torch.empty((rows, W.n_pad), dtype=torch.float32, device=device)
    calls, nbytes = 0, 0
    pdl = model.use_pdl

    def gemvs():
        # the GEMV launches of one replay as the replay issues them: GEMV-ready activations,
        # programmatic dependent launch between consecutive kernels
        nonlocal calls, nbytes
        calls, nbytes = 0, 0
        for layer in model.layers:
            at, ff = layer.attention, layer.feed_forward
            for (A, asum, s, w, ws, out) in (
                    (W.q, W.q_sum, W.s, at.wqkv_weight, at.wqkv_scale, W.xqkv),
                    (W.att_q, W.att_sum, W.att_s, at.o_proj.weight.data, at.o_proj.weight_scale, W.attn_out),
                    (W.q, W.q_sum, W.s, ff.w_gu, ff.w_gu_scale, W.gu),
                    (W.iq, W.i_sum, W.is_, ff.down_proj.weight.data, ff.down_proj.weight_scale, W.ffn_out)):
                ops.t2_gemv_prepared(A, asum, w, s, ws, out=out, ldc=out.shape[1], pdl=pdl)
                calls += 1
                nbytes += gemv_alg_bytes(M, w.shape[0], w.shape[1] * 4)
        ops.t2_gemv_prepared(W.hq[:rows], W.h_sum[:rows], model._lm_head_t2_w, W.hs[:rows], model._lm_head_t2_scale,
                             out_kind=native.OUT_F32_OF_BF16, out=logits, ldc=W.n_pad, pdl=pdl)
        calls += 1
        nbytes += gemv_alg_bytes(rows, W.n_pad, a.dim, 4)

    for t in (W.q, W.att_q, W.iq, W.hq):
        t.random_(-127, 128)
    for t in (W.s, W.att_s, W.is_, W.hs):
        t.fill_(30.0)
    for t in (W.q_sum, W.att_sum, W.i_sum, W.h_sum):      # any integers: only the timing matters here
        t.random_(-4000, 4000)
    gemvs()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        gemvs()
    sec = time_graph(g, 1, steps)
    return {"calls": calls, "bytes": nbytes, "seconds": sec, "gbs": nbytes / sec / 1e9,
            "us_per_launch": sec / calls * 1e6}


def timed_generations(args, device, local, dist, model, atlas, cfg, steps, warmup, new_tokens, prompt_len, rank,
                      seed_base=100):
    """W warm-up and K timed whole generations through the public decode call, host prompt in and
    tokens out; returns the figures of the timed region."""
    import torch
    from bitmtp_b200 import fast_generate as FG, native, synthetic
    D = cfg["block_size"]
    policy = synthetic.AcceptancePolicy(args.accept, D, seed=rank)
    saved = FG._fused_draft_chain, FG._fused_verify_accept
    FG._fused_draft_chain, FG._fused_verify_accept = synthetic.acceptance_hooks(FG, policy)
    counted = list(atlas.graphs.values()) + list(atlas.prefill_graphs.values())
    for g in counted:
        if not isinstance(g.cuda_graph, _ReplayCounter):
            g.cuda_graph = _ReplayCounter(g.cuda_graph)
    fn = {"ar": FG.fast_ar_generate, "spec": FG.fast_speculative_generate,
          "hybrid": FG.fast_hybrid_generate, "conf": FG.fast_confidence_generate}[args.mode]
    kwargs = {}
    if args.mode != "ar":
        kwargs = {"use_fp8_draft": args.draft_head == "fp8", "use_bf16_draft": args.draft_head == "bf16"}
    prompt_host = synthetic.random_prompt(prompt_len, cfg["vocab_size"], seed=seed_base + rank).pin_memory()

    def one():
        # end to end through the public call: prompt from pinned host memory, tokens back
        ids = prompt_host.to(device, non_blocking=True)
        out, st = fn(model, atlas, ids, max_gen_len=new_tokens, eos_ids=(), **kwargs)
        return out.cpu(), st

    try:
        for _ in range(warmup):
            one()
        barrier(dist)
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tok = dec_t = tot_t = iters = ttft = 0.0
        for g in counted:
            g.cuda_graph.replays = 0
        eager_before = native.lib().bm_launch_count()
        e0.record()
        for _ in range(steps):
            out, st = one()
            tok += st["timed_decode_tokens"]
            dec_t += st["decode_time"]
            tot_t += st["total_time"]
            iters += st["n_iters"]
            ttft += st["ttft"]
        e1.record()
        barrier(dist)
        clocks = sampler.stop()
    finally:
        FG._fused_draft_chain, FG._fused_verify_accept = saved
    ms = max_over_ranks(dist, e0.elapsed_time(e1), device)
    err = native.lib().bm_device_error()
    if err:
        raise RuntimeError(f"device error word = {err}")
    # this library's kernels inside the timed region: launches it issued eagerly (staging, argmax / chain /
    # accept, KV promotion) + its kernel nodes in every replayed graph
    launches = int(native.lib().bm_launch_count() - eager_before
                   + sum(g.cuda_graph.replays * g.n_kernels for g in counted))
    replays = {f"{r}:M{M}": g.cuda_graph.replays for (M, _, r), g in sorted(atlas.graphs.items())
               if g.cuda_graph.replays}
    replays["prompt-slab:M16"] = sum(g.cuda_graph.replays for g in atlas.prefill_graphs.values())
    return {"ms": ms, "clocks": clocks, "tok": tok, "dec_t": dec_t, "tot_t": tot_t, "iters": iters, "ttft": ttft,
            "launches": launches, "replays": replays,
            "dec_t_max": max_over_ranks(dist, dec_t, device), "tok_all": sum_over_ranks(dist, tok, device),
            "new_all": sum_over_ranks(dist, float(new_tokens * steps), device)}


def run_decode(args, world, rank, local, dist):
    """GPU arm: every rank decodes its own request stream on its own replica (no data-path
    collective); value = sum of timed decode tokens / max over ranks of the decode time."""
    import torch
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    prompt_len, new_tokens, ladder, roof_m = decode_shape(args)
    steps = args.steps or 3
    warmup = args.warmup if args.warmup is not None else 3
    model, atlas, cfg = build_decode(args.model, device, prompt_len, new_tokens, seed=rank, draft_head=args.draft_head)
    r = timed_generations(args, device, local, dist, model, atlas, cfg, steps, warmup, new_tokens, prompt_len, rank)
    value = r["tok_all"] / r["dec_t_max"]
    e2e = r["new_all"] / (r["ms"] * 1e-3)
    rf = replay_gemv_roofline(model, roof_m, device)
    peak, peak_kind = peaks()
    res = {
        "metric": decode_metric(args),
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(r["ms"] / steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "s8 x ternary -> s32 (bf16 activations in memory)",
        "data": "synthetic", "config": decode_config(args, world),
        "gpu_launches": r["launches"], "clocks": r["clocks"],
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": prompt_len * 8,
                "d2h_bytes_per_step": new_tokens * 8},
        "roofline": {"bound": "hbm", "achieved": round(rf["gbs"], 1), "peak": peak, "unit": "GB/s",
                     "frac": round(rf["gbs"] / peak, 4),
                     "traffic": round(rf["bytes"] / rf["calls"] * DRAM_TRAFFIC_RATIO["cooperative"]),
                     "traffic_note": "per launch: average algorithmic bytes of the replay's GEMV launches x the "
                                     "DRAM/algorithmic ratio ncu measured on one of them (profiles/)",
                     "peak_kind": peak_kind,
                     "kernel": f"t2_gemv (cooperative-tile and row-per-warp kernels), the {rf['calls']} GEMV launches of "
                               f"one width-{roof_m} replay ({rf['bytes'] / 1e6:.1f} MB algorithmic, "
                               f"{rf['us_per_launch']:.2f} us average per launch)",
                     "frac_of_8TBps": round(rf["gbs"] / 8000.0, 4)},
        "decode": {"iters_per_generation": r["iters"] / steps, "decode_ms_per_generation": r["dec_t"] / steps * 1e3,
                   "total_ms_per_generation": r["tot_t"] / steps * 1e3, "ttft_ms": r["ttft"] / steps * 1e3,
                   "graph_replays_timed": r["replays"],
                   "tokens_per_iteration": round(r["tok"] / max(r["iters"] - steps, 1.0), 3)},
    }
    if not args.no_extras:
        del atlas, model
        torch.cuda.empty_cache()
        if rank == 0:
            res["gemv_table"] = gemv_table(device, our_gemv_launchers())
        if world > 1:
            barrier(dist)
            res["nsplit"] = nsplit_extra(world, rank, local, dist)
            if args.model == "1p7b" and args.accept == "forced":
                res["streams_4b_categorical"] = streams_4b_extra(args, world, rank, local, dist)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        res["cpu_baseline"] = cpu_decode_baseline(args.model, roof_m)
    return res


def streams_4b_extra(args, world, rank, local, dist) -> dict:
    """Independent request streams on the 4B geometry with the seeded categorical acceptance, one per
    GPU: aggregate tokens/s (sum of timed decode tokens / max decode time) of two timed generations."""
    import copy
    import torch
    device = torch.device("cuda", local)
    a4 = copy.copy(args)
    a4.model, a4.accept, a4.mode, a4.prompt_len, a4.new_tokens, a4.draft_head = "4b", "categorical", "hybrid", 512, 512, "native"
    model, atlas, cfg = build_decode("4b", device, 512, 512, seed=rank)
    r = timed_generations(a4, device, local, dist, model, atlas, cfg, 2, 1, 512, 512, rank)
    out = {"value": round(r["tok_all"] / r["dec_t_max"], 2), "unit": "tok/s", "n_gpus": world, "steps": 2, "warmup": 1,
           "e2e_tok_s": round(r["new_all"] / (r["ms"] * 1e-3), 2), "scaling": "weak",
           "config": decode_config(a4, world)["workload"], "graph_replays_timed": r["replays"]}
    del atlas, model
    torch.cuda.empty_cache()
    return out


def cpu_decode_baseline(model_name: str, M: int, reps: int = 5) -> dict:
    """The CPU oracle's full-depth forward at width M on this box's host cores: `reps` timed forwards
    after one warm-up, median.  tokens/s = D tokens per width-16 or width-9 replay, 1 per AR replay."""
    times, cores = oracle_forward_times(model_name, M, 1, reps)
    times.sort()
    t = times[len(times) // 2]
    tokens = 8 if M > 1 else 1
    return {"value": round(tokens / t, 3), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{reps} full-depth oracle forwards at width {M} (one replay each, {tokens} tokens), "
                      f"median {t * 1e3:.0f} ms per replay"}


def oracle_forward_times(model_name: str, M: int, warmup: int, steps: int):
    """Seconds of `steps` full-depth CPU oracle forwards at width M (after `warmup` untimed ones) and
    the threads used."""
    import numpy as np
    from bitmtp_b200 import synthetic
    from oracle import oracle as O
    geometry = dict(getattr(synthetic, GEOMETRIES[model_name]))
    sigma = 1024
    # every host core, also under a launcher that exports OMP_NUM_THREADS=1 for its ranks
    O.lib().bmo_set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cfg = synthetic.make_config(geometry, block_size=8)
    state = synthetic.device_state(cfg, "cpu", seed=0)
    head = (state.pop("_head.weight"), state.pop("_head.weight_scale"))
    om = O.OracleModel(cfg, state, max_positions=sigma + 17, head=head)
    del state
    kv = om.new_kv(sigma, 17)
    D = cfg["block_size"]
    role = O.ROLE_DRAFT if M > D + 1 else (O.ROLE_VERIFY if M > 1 else O.ROLE_AR)
    toks = np.arange(M) % cfg["vocab_size"]
    pos = np.arange(500, 500 + M)
    ls, le = (M - D, M) if role == O.ROLE_DRAFT else (0, M)
    out = []
    for i in range(warmup + steps):
        t0 = time.time()
        om.forward(toks, pos, kv, sigma, role, 500, max(M - D, 0) if role == O.ROLE_DRAFT else 0, ls, le)
        if i >= warmup:
            out.append(time.time() - t0)
    return out, O.lib().bmo_num_threads()


# ----------------------------------------------------------------------------- N-split
def nsplit_layers(world, rank, device, widths, fused, copies_bytes=256 << 20):
    import torch
    from bitmtp_b200 import ops, synthetic
    from bitmtp_b200.nsplit import FusedNSplitLinear, NSplitLinear, shard_rows
    N, K = 28672, 8192
    n0, n1 = shard_rows(N, world, rank)
    rows = n1 - n0
    shard_bytes = rows * K // 4
    copies = max(2, -(-copies_bytes // shard_bytes))
    if copies % 2:
        copies += 1                      # an even number of calls per pass: a replayed graph returns to the same buffers
    gen = torch.Generator(device=device).manual_seed(1 + rank)

    def gemv(a, s_, weight, scale, out):
        ops.t2_gemv(a, weight, s_, scale, out=out, ldc=out.shape[1])

    layers = []
    for _ in range(copies):
        w_, sc = synthetic.device_ternary(rows, K, gen, device)
        if fused:
            layers.append(FusedNSplitLinear(w_, sc, n_full=N, max_w=max(widths)))
        else:
            layers.append(NSplitLinear(w_, sc, rank=rank, world=world, gemv=gemv, sharded=True))
    return layers, rows, copies, shard_bytes


def nsplit_extra(world, rank, local, dist) -> dict:
    """The 8192 -> 28672 layer split by rows over the ranks, exchange inside the GEMV kernel (peer stores
    over NVLink, no multicast): per width the time per call (max over ranks), per-GPU and whole-layer
    GB/s, and a bit-identity check of the gathered output against the unsplit product on one GPU."""
    import torch
    from bitmtp_b200 import native, ops, synthetic
    from bitmtp_b200.nsplit import FusedNSplitLinear, shard_rows
    device = torch.device("cuda", local)
    N, K = 28672, 8192
    out = {"layer": "8192->28672", "exchange": "peer stores + flags inside the GEMV kernel", "n_gpus": world}
    # bit identity: every rank builds the same full layer, computes the unsplit product and its own shard's split call
    gen = torch.Generator(device=device).manual_seed(1234)
    Bf, wsf = synthetic.device_ternary(N, K, gen, device)
    n0, n1 = shard_rows(N, world, rank)
    lin = FusedNSplitLinear(Bf[n0:n1].contiguous(), wsf[n0:n1].contiguous(), n_full=N, max_w=8)
    same = True
    for W in (1, 8):
        A = torch.randint(-127, 128, (W, K), generator=gen, device=device, dtype=torch.int8)
        s = torch.rand(W, generator=gen, device=device) * 40 + 20
        want = ops.t2_gemv(A, Bf, s, wsf)
        for _ in range(2):
            got = lin.forward(A, s)
            torch.cuda.synchronize(device)
            same = same and bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
            dist.barrier()
    same = same and lin.failed_call() == 0
    out["bit_identical_to_single_gpu"] = bool(sum_over_ranks(dist, 0.0 if same else 1.0, device) == 0.0)
    del lin, Bf, wsf
    torch.cuda.empty_cache()
    for W in (1, 8):
        layers, rows, copies, shard_bytes = nsplit_layers(world, rank, device, (W,), fused=True)
        A = torch.randint(-127, 128, (W, K), device=device, dtype=torch.int8)
        s = torch.rand(W, device=device) * 40 + 20
        graph = capture(lambda: [lin.forward(A, s) for lin in layers], device)
        for _ in range(3):
            graph.replay()
        barrier(dist)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        reps = 10
        for _ in range(reps):
            graph.replay()
        e1.record()
        barrier(dist)
        sec = max_over_ranks(dist, e0.elapsed_time(e1), device) * 1e-3 / (reps * copies)
        failed = sum_over_ranks(dist, float(any(lin.failed_call() for lin in layers)), device)
        out[f"W{W}"] = {"us_per_call": round(sec * 1e6, 2),
                        "per_gpu_gbs": round(gemv_alg_bytes(W, rows, K) / sec / 1e9, 1),
                        "layer_gbs": round(gemv_alg_bytes(W, N, K) / sec / 1e9, 1),
                        "shard_rows": rows, "copies_rotated": copies, "peer_wait_failures": int(failed)}
        del graph, layers
        torch.cuda.empty_cache()
    err = native.lib().bm_device_error()
    out["device_error"] = int(sum_over_ranks(dist, float(err), device))
    return out


def run_nsplit(args, world, rank, local, dist):
    """Wide-layer stress shape (K = 8192 -> N = 28672) split by output rows over the ranks:
    every rank streams its own N/world rows and ends with the full [W, N] output (exchange inside
    the kernel, or NCCL all-gather with BM_NSPLIT_NCCL=1).  Total work is fixed (strong scaling);
    value = algorithmic bytes of the whole layer / time per call (max over ranks).  Each rank rotates
    over enough distinct copies of its shard to exceed L2."""
    import torch
    from bitmtp_b200 import native
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    N, K = 28672, 8192
    widths = (1, 8)
    steps = args.steps or 20
    warmup = args.warmup if args.warmup is not None else 5
    fused = world > 1 and os.environ.get("BM_NSPLIT_NCCL", "0") != "1"
    layers, rows, copies, shard_bytes = nsplit_layers(world, rank, device, widths, fused)
    gen_cpu = torch.Generator().manual_seed(7)          # activations are replicated: same seed everywhere
    acts = {w: (torch.randint(-127, 128, (w, K), generator=gen_cpu, dtype=torch.int8),
                (torch.rand(w, generator=gen_cpu) * 40 + 20)) for w in widths}
    dev_acts = {w: (a.to(device), s_.to(device)) for w, (a, s_) in acts.items()}
    host_acts = {w: (a.pin_memory(), s_.pin_memory()) for w, (a, s_) in acts.items()}

    def one_pass():
        for w in widths:
            a, s_ = dev_acts[w]
            for lin in layers:
                lin.forward(a, s_)

    def e2e_pass():
        outs = []
        for w in widths:
            ha, hs = host_acts[w]
            a, s_ = ha.to(device, non_blocking=True), hs.to(device, non_blocking=True)
            for lin in layers:
                outs.append(lin.forward(a, s_)[:, :8].float().sum().cpu())   # result read back every call
        return outs

    # The fused exchange keeps its call counter on the device, so the pass replays as a CUDA graph
    # (the host cost of a launch would otherwise exceed the 15 us kernel); NCCL calls stay eager.
    timed = one_pass
    if fused or world == 1:
        graph = capture(one_pass, device)
        timed = graph.replay
    for _ in range(warmup):
        timed()
    barrier(dist)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        timed()
    e1.record()
    barrier(dist)
    clocks = sampler.stop()
    ms = max_over_ranks(dist, e0.elapsed_time(e1), device)
    calls = len(widths) * copies
    layer_bytes = sum(gemv_alg_bytes(w, N, K) for w in widths) * copies     # whole layer, all ranks
    value = layer_bytes * steps / (ms * 1e-3) / 1e9
    shard_alg = sum(gemv_alg_bytes(w, rows, K) for w in widths) * copies
    gbs_rank = shard_alg * steps / (ms * 1e-3) / 1e9

    e2e_pass()
    barrier(dist)
    t0 = time.time()
    e2e_steps = max(1, min(steps, 5))
    for _ in range(e2e_steps):
        e2e_pass()
    barrier(dist)
    e2e_s = max_over_ranks(dist, time.time() - t0, device)
    err = native.lib().bm_device_error()
    if err:
        raise RuntimeError(f"device error word = {err}")
    peak, peak_kind = peaks()
    return {
        "metric": "T2-g128 GEMV algorithmic HBM GB/s", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8 x ternary -> s32",
        "data": "synthetic",
        "config": {"workload": f"N-split of the 8192->28672 layer over {world} GPU(s), W in {{1,8}}, bf16 outputs "
                               + ("exchanged inside the GEMV kernel (peer stores over NVLink + flags)" if fused
                                  else "all-gathered with NCCL after every GEMV"),
                   "l2": f"each rank rotates over {copies} copies of its {shard_bytes >> 20} MiB shard (> L2)",
                   "timing": ("CUDA events around graph replays" if (fused or world == 1)
                              else "CUDA events around eager launches") + ", max over ranks"},
        "gpu_launches": calls * steps, "clocks": clocks,
        "e2e": {"value": round(layer_bytes * e2e_steps / e2e_s / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": sum(w * K + 4 * w for w in widths), "d2h_bytes_per_step": 4 * calls},
        "roofline": {"bound": "hbm", "achieved": round(gbs_rank, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(gbs_rank / peak, 4),
                     "traffic": round(shard_alg / calls * DRAM_TRAFFIC_RATIO["rowwarp"]),
                     "traffic_note": "per launch: algorithmic bytes of the shard x the DRAM/algorithmic ratio ncu measured "
                                     "for the row-per-warp kernel (profiles/)",
                     "peak_kind": peak_kind,
                     "kernel": f"t2_gemv on this rank's {rows} x {K} shard, all-gather time included",
                     "frac_of_8TBps": round(gbs_rank / 8000.0, 4)},
    }


# ----------------------------------------------------------------------------- reference arm
def reference_cpu_linear_path(shapes, iters=100, warm=20):
    """The reference's own CPU-capable T2 arithmetic (src/bonsai_sft/gpu/model.py:638-656, 672-678:
    cached `_unpack_to_bf16()` + `Q1Linear.act_quant` + `F.linear`), imported from the copy of the
    reference installed under baseline/_ref, timed on all host threads at W = 1: median of `iters`
    after `warm` calls (fewer for the head, stated).  Says why where that copy is absent."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "bonsai_sft")):
        return {"unavailable": "baseline/_ref holds no copy of the reference's Python package"}
    import torch
    import torch.nn.functional as F
    sys.path.insert(0, ref_root)
    try:
        from bonsai_sft.gpu import runtime_config
        runtime_config.select_runtime_profile("orin-d8")          # its eager profile, chosen before its model imports
        from bonsai_sft.gpu import model as RM
        from bitmtp_b200 import synthetic
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        torch.set_num_threads(threads)
        out = {"threads": torch.get_num_threads(), "cpu_count": os.cpu_count(), "per_case": {}}
        gen = torch.Generator().manual_seed(0)
        for (n, k) in shapes:
            lin = RM.T2LinearKernel(k, n)
            packed, scale, _ = synthetic.ternary_weight(min(n, 16384), k, gen)
            reps_rows = -(-n // packed.shape[0])
            lin.weight.data.copy_(packed.repeat(reps_rows, 1)[:n])
            lin.weight_scale.data.copy_(scale.repeat(reps_rows, 1)[:n])
            w = lin._unpack_to_bf16()                              # cached dense bf16 weight, as the fallback keeps it
            x = torch.randn(1, k, generator=gen).to(torch.bfloat16)
            it, wm = (iters, warm) if n * k <= 64 << 20 else (10, 3)
            ts = []
            with torch.no_grad():
                for i in range(wm + it):
                    t0 = time.perf_counter()
                    F.linear(RM.Q1Linear.act_quant(x), w)
                    if i >= wm:
                        ts.append(time.perf_counter() - t0)
            ts.sort()
            med = ts[len(ts) // 2]
            out["per_case"][f"{n}x{k}:W1"] = {"us": round(med * 1e6, 1), "iters": it,
                                              "gbs_of_packed_bytes": round(gemv_alg_bytes(1, n, k) / med / 1e9, 2)}
        return out
    except Exception as e:                                         # the reference arm must still print its line
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    finally:
        sys.path.remove(ref_root)


def reference_gpu_decode(model_name: str, prompt_len: int, new_tokens: int, timeout_s: int = 420):
    """The reference's own GPU decode loops (its Python runtime, its CUDA kernel from oracle/_ref) on
    the synthetic checkpoint of this workload, in a child process.  Returns its JSON, or why not."""
    script = os.path.join(ROOT, "oracle", "reference_decode.py")
    if not os.path.exists(script):
        return {"unavailable": "oracle/reference_decode.py is absent"}

    def attempt(profile, limit):
        try:
            p = subprocess.run([sys.executable, script, "--model", model_name, "--prompt-len", str(prompt_len),
                                "--new-tokens", str(new_tokens), "--profile", profile],
                               capture_output=True, text=True, timeout=limit)
        except subprocess.TimeoutExpired:
            return {"unavailable": f"profile {profile}: not finished within {limit} s"}
        for line in reversed(p.stdout.strip().splitlines()):
            if line.startswith("{"):
                try:
                    return json.loads(line)
                except Exception:
                    break
        return {"unavailable": (f"profile {profile}: exit {p.returncode}: ")
                + (p.stderr.strip().splitlines() or ["no output"])[-1][:300]}

    # its default (compiled helpers, FlexAttention) first; the eager profile with the explicit attention
    # if that cannot run here
    first = attempt("standard", timeout_s)
    if "unavailable" not in first:
        return first
    second = attempt("eager", timeout_s // 2)
    second["standard_profile"] = first["unavailable"]
    return second


def run_reference_decode(args) -> dict:
    """CPU arm of the decode workload.  A step is one full-depth forward of the oracle port at the
    replay width that dominates the workload (16 for hybrid / confidence with forced acceptance: 8
    tokens per replay; 9 for speculative; 1 for AR), on all host threads: a bounded sample of the
    workload's replays.  value = tokens per replay / mean seconds per step."""
    import torch
    steps = args.steps or 5
    warmup = args.warmup if args.warmup is not None else 1
    prompt_len, new_tokens, ladder, M = decode_shape(args)
    times, cores = oracle_forward_times(args.model, M, warmup, steps)
    mean = sum(times) / len(times)
    tokens = 8 if M > 1 else 1
    value = tokens / mean
    sample = (f"{steps} full-depth forwards of the CPU oracle port at width {M} (one replay each, {tokens} tokens per "
              f"replay), mean {mean * 1e3:.0f} ms; min {min(times) * 1e3:.0f} / max {max(times) * 1e3:.0f} ms")
    extras = {}
    if not args.no_extras:
        if torch.cuda.is_available():
            extras["reference_cuda_kernel"] = reference_cuda_table()
            if extras["reference_cuda_kernel"] and args.model == "1p7b":
                rows = {1: 1, 9: 9, 16: 8}[M]
                per_layer = [(4096, 2048, M), (2048, 2048, M), (12288, 2048, M), (2048, 6144, M)]
                replay = reference_cuda_table(per_layer + [(151936, 2048, rows)])
                if replay:
                    rc = replay["per_case"]
                    layer_us = sum(rc[f"{n}x{k}:W{w}"]["reference_kernel"]["us"] for (n, k, w) in per_layer)
                    extras["reference_cuda_kernel"]["replay_width"] = M
                    extras["reference_cuda_kernel"]["replay_cases"] = rc
                    extras["reference_cuda_kernel"]["gemv_us_per_replay"] = round(
                        28 * layer_us + rc[f"151936x2048:W{rows}"]["reference_kernel"]["us"], 1)
        extras["reference_cpu_linear_path"] = reference_cpu_linear_path(
            [(1024, 2048), (2048, 2048), (6144, 2048), (2048, 6144), (151936, 2048)])
        if torch.cuda.is_available():
            extras["reference_gpu_decode"] = reference_gpu_decode(args.model, prompt_len, new_tokens)
    line = {"impl": "reference", "metric": decode_metric(args), "value": round(value, 3), "unit": "tok/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(mean * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8 x ternary -> s32 (bf16 activations in memory)", "data": "synthetic",
            "config": decode_config(args, max(args.gpus, 1)),
            "cpu_baseline": {"value": round(value, 3), "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 3), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    line.update(extras)
    return line


# ----------------------------------------------------------------------------- single-kernel workloads
def run_kernel(args, world, rank, local, dist):
    """`attention`: the replay's attention launch (q/k norm, RoPE, KV append, split-KV, merge) on the 1.7B head
    geometry, `--layers` dependent launches per graph over distinct K/V planes.  `prompt-gemm`: the many-row
    T2 x int8 GEMM of the prompt forward over weight copies that exceed L2.  One JSON line each; these are the
    commands the ncu summaries under profiles/ were captured from."""
    import torch
    from bitmtp_b200 import native, ops, synthetic
    from bitmtp_b200.model import _LayerView
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    steps = args.steps or 20
    warmup = args.warmup if args.warmup is not None else 5
    peak, peak_kind = peaks()
    gen = torch.Generator(device=device).manual_seed(0)
    if args.workload == "attention":
        H, Hkv, sigma, M, L, cl = 16, 8, 1024, args.w, args.layers, args.cache_len
        kv_rows = sigma + 17
        kvb = (torch.randn(2, L, 1, Hkv, kv_rows, 128, device=device, generator=gen) * 0.5).to(torch.bfloat16)
        cos = torch.rand(kv_rows, 128, device=device, generator=gen).to(torch.bfloat16)
        sin = torch.rand(kv_rows, 128, device=device, generator=gen).to(torch.bfloat16)
        qw = torch.ones(128, dtype=torch.bfloat16, device=device)
        xqkv = torch.randn(M, (H + 2 * Hkv) * 128, device=device, generator=gen).to(torch.bfloat16)
        att = torch.empty(M, H * 128, dtype=torch.bfloat16, device=device)
        amax = torch.zeros(2, M, dtype=torch.int32, device=device)
        scratch = ops.attention_scratch(17, H, sigma, device)
        pos = torch.arange(cl, cl + M, device=device)
        state = ops.new_step_state(device)
        role = native.ROLE_AR if M == 1 else native.ROLE_DRAFT
        ops.set_step_state(state, cl, min(8, max(M - 8, 0)), role, max(M - 8, 0))
        pdl = native.PDL_OVERLAP | native.PDL_STABLE_STATE

        def chain():
            for i in range(L):
                ops.rope_verify_attention_rows(xqkv, qw, qw, 1e-6, cos, sin, pos, H, Hkv, _LayerView(kvb[0, i], kv_rows),
                                               _LayerView(kvb[1, i], kv_rows), sigma, state, scratch, att=att,
                                               amax=amax[i & 1], pdl=pdl)
        calls = L
        alg = 2 * Hkv * (cl + M) * 256 + M * (H + 2 * Hkv) * 256 + M * H * 256      # live K/V rows + qkv in + rows out
        label = f"attention launch, 16/8 heads, width {M}, cache_len {cl}, segment {sigma}, {L} dependent launches per graph"
        bound, unit, scale, pk = "hbm", "GB/s", 1e9, peak
    else:
        n, k = (int(x) for x in args.shape.lower().split("x"))
        T = args.rows
        copies = max(2, (160 << 20) // (n * k // 4) + 1)
        Bs = [synthetic.device_ternary(n, k, gen, device) for _ in range(copies)]
        A = torch.randint(-127, 128, (T, k), device=device, dtype=torch.int8, generator=gen)
        asum = A.view(T, k // 128, 128).sum(dim=2, dtype=torch.int32)
        sc = torch.rand(T, device=device, generator=gen) * 40 + 20
        C = torch.empty(T, n, dtype=torch.bfloat16, device=device)

        def chain():
            for B, ws in Bs:
                ops.t2_gemm_wide(A, asum, B, sc, ws, out=C)
        calls = copies
        alg = 2 * T * n * k                                                             # integer multiply-adds x 2
        label = f"prompt GEMM {n}x{k}, {T} rows, {copies} weight copies (> L2) per graph"
        bound, unit, scale = "tensor", "TOP/s", 1e12
        try:
            pk = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        except Exception:
            pk, peak_kind = 1590.0, "fallback"
    graph = capture(chain, device)
    sampler = ClockSampler(local)
    ms, clocks = time_replays(graph, steps, warmup, dist, device, sampler)
    err = native.lib().bm_device_error()
    if err:
        raise RuntimeError(f"device error word = {err}")
    us = ms * 1e3 / (steps * calls)
    achieved = alg / (us * 1e-6) / scale
    return {"metric": f"{args.workload} us per launch", "value": round(us, 3), "unit": "us", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": round(ms / steps, 5), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 -> fp32" if args.workload == "attention" else "s8 x ternary -> s32",
            "data": "synthetic", "config": {"workload": label, "timing": "CUDA events around graph replays"},
            "gpu_launches": steps * calls, "clocks": clocks,
            "roofline": {"bound": bound, "achieved": round(achieved, 3), "peak": pk, "unit": unit,
                         "frac": round(achieved / pk, 5), "traffic": None, "peak_kind": peak_kind,
                         "note": "peak = measured bf16 cuBLAS rate; the int8 tensor path is nominally 2x that"
                         if bound == "tensor" else "algorithmic bytes = live K/V rows + the replay's qkv rows in and attention rows out"}}


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        if rank != 0:
            return 0
        out = run_reference_decode(args) if args.workload == "decode" else run_reference_gemv(args, rank)
        print(json.dumps(out), flush=True)
        return 0
    world, rank, local, dist = init_dist(args)
    if args.workload == "decode":
        out = run_decode(args, world, rank, local, dist)
    elif args.workload == "gemv-nsplit":
        out = run_nsplit(args, world, rank, local, dist)
    elif args.workload in ("attention", "prompt-gemm"):
        out = run_kernel(args, world, rank, local, dist)
    else:
        out = run_gemv(args, world, rank, local, dist)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
