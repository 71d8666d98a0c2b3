"""Decode workloads behind bench.py: the Bonsai-architecture hybrid MTP decode on synthetic
weights (GPU arm) and its bounded CPU counterpart on the oracle (reference arm).

Definitions follow the reference's benchmark adapter: decode speed = timed decode tokens /
decode seconds, the first token and the prefill excluded
(benchmarks/bonsai_adapter.py:55-58, src/bonsai_sft/gpu/fast_generate.py:1147-1172).
"""
from __future__ import annotations

import json
import os
import time

import torch

GEOMETRIES = {"1p7b": "BONSAI_1P7B", "4b": "BONSAI_4B", "tiny": "TINY"}
D8_WIDTHS = (1, 8, 9, 10, 12, 16, 17)


def acceptance_hooks(FG, policy):
    """Replacements for the loops' confidence-chain and prefix-accept reductions that apply
    a synthetic.AcceptancePolicy.  The kernels still run.  A replaced chain length is handed to the
    loop as a host value; a replaced accepted-prefix length is written over the kernel's count in
    place, so that it stays part of the record the loop reads in one copy."""
    chain, accept = FG._fused_draft_chain, FG._fused_verify_accept

    def hooked_chain(logits, threshold, out=None):
        idx, n = chain(logits, threshold, out)
        a = policy.chain_count()
        # the replacement count is a host value: the loop then reads only the ids from the device (still one
        # copy), and no extra kernel of the harness runs inside the timed region
        return idx, (n if a is None else torch.tensor([a], dtype=torch.int64))

    def hooked_accept(draft, verify, Dd, out=None):
        n = accept(draft, verify, Dd, out)
        a = policy.accept_count()
        return n if a is None else n.fill_(a)

    return hooked_chain, hooked_accept


class _ReplayCounter:
    """Stands in for a CapturedGraph's cuda_graph: forwards replay() and counts the calls."""

    def __init__(self, graph):
        self.graph, self.replays = graph, 0

    def replay(self):
        self.replays += 1
        self.graph.replay()

    def __getattr__(self, name):
        return getattr(self.graph, name)


def build_decode(model_name: str, device, prompt_len: int, new_tokens: int, seed: int = 0):
    """(model, atlas, cfg) for a synthetic checkpoint of the named geometry."""
    from . import generate, synthetic
    from .fast_runtime import GraphAtlas
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
    atlas = GraphAtlas(model, model.args, device, segment_ladder=ladder, m_set=D8_WIDTHS,
                       roles=("ar", "draft", "verify"), capture_verbose=False)
    return model, atlas, cfg


def _gemv_roofline(model, M: int, device, steps: int = 20):
    """Average device time of the GEMV launches of one width-M replay, measured live: the
    same calls on the model's own weights (layer l, then l+1, ...: 376 MB of distinct
    weights per pass, three times L2), captured in one graph and replayed."""
    from . import native, ops
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
                nbytes += ops.gemv_bytes(M, w.shape[0], w.shape[1] * 4)
        ops.t2_gemv_prepared(W.hq[:rows], W.h_sum[:rows], model._lm_head_t2_w, W.hs[:rows], model._lm_head_t2_scale,
                             out_kind=native.OUT_F32_OF_BF16, out=logits, ldc=W.n_pad, pdl=pdl)
        calls += 1
        nbytes += ops.gemv_bytes(rows, W.n_pad, a.dim, native.OUT_F32)

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
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / steps
    return {"calls": calls, "bytes": nbytes, "seconds": sec, "gbs": nbytes / sec / 1e9,
            "us_per_launch": sec / calls * 1e6}


def run_decode(args, world, rank, local, dist):
    """GPU arm: every rank decodes its own request stream on its own replica (no data-path
    collective); value = sum of timed decode tokens / max over ranks of the decode time."""
    import bench
    from . import fast_generate as FG, native, synthetic
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    prompt_len = args.prompt_len or (512 if args.model == "4b" else 256)
    new_tokens = args.new_tokens or 512
    steps = args.steps or 3
    warmup = args.warmup if args.warmup is not None else 3
    model, atlas, cfg = build_decode(args.model, device, prompt_len, new_tokens, seed=rank)
    D = cfg["block_size"]
    policy = synthetic.AcceptancePolicy(args.accept, D, seed=rank)
    FG._fused_draft_chain, FG._fused_verify_accept = acceptance_hooks(FG, policy)
    counted = list(atlas.graphs.values()) + list(atlas.prefill_graphs.values()) + list(atlas.dense_graphs.values())
    for g in counted:
        g.cuda_graph = _ReplayCounter(g.cuda_graph)
    fn = {"ar": FG.fast_ar_generate, "spec": FG.fast_speculative_generate,
          "hybrid": FG.fast_hybrid_generate, "conf": FG.fast_confidence_generate}[args.mode]
    prompt_host = synthetic.random_prompt(prompt_len, cfg["vocab_size"], seed=100 + rank).pin_memory()

    def one():
        # end to end through the public call: prompt from pinned host memory, tokens back
        ids = prompt_host.to(device, non_blocking=True)
        out, st = fn(model, atlas, ids, max_gen_len=new_tokens, eos_ids=())
        return out.cpu(), st

    for _ in range(warmup):
        one()
    bench.barrier(dist)
    sampler = bench.ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tok = dec_t = tot_t = iters = 0.0
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
    e1.record()
    bench.barrier(dist)
    clocks = sampler.stop()
    ms = bench.max_over_ranks(dist, e0.elapsed_time(e1), device)
    dec_t_max = bench.max_over_ranks(dist, dec_t, device)
    tot_t_max = bench.max_over_ranks(dist, tot_t, device)
    tok_all = bench.sum_over_ranks(dist, tok, device)
    new_all = bench.sum_over_ranks(dist, float(new_tokens * steps), device)
    err = native.lib().bm_device_error()
    if err:
        raise RuntimeError(f"device error word = {err}")
    value = tok_all / dec_t_max
    e2e = new_all / (ms * 1e-3)

    # this library's kernels inside the timed region: launches it issued eagerly (prefill slabs,
    # staging, argmax / chain / accept, KV promotion) + its kernel nodes in every replayed graph
    launches = int(native.lib().bm_launch_count() - eager_before
                   + sum(g.cuda_graph.replays * g.n_kernels for g in counted))
    replays = {f"{r}:M{M}": g.cuda_graph.replays for (M, _, r), g in sorted(atlas.graphs.items())
               if g.cuda_graph.replays}
    replays["prompt-slab:M16"] = sum(g.cuda_graph.replays for g in atlas.prefill_graphs.values())
    for (M, _, r), g in sorted(atlas.dense_graphs.items()):
        if g.cuda_graph.replays:
            replays[f"{r}:M{M}:3-per-SM attention"] = g.cuda_graph.replays
    roof_m = 16 if args.mode in ("hybrid", "conf") else (1 if args.mode == "ar" else 9)
    rf = _gemv_roofline(model, roof_m, device)
    peak, peak_kind = bench.peaks()
    accept_words = {"forced": "forced full-block acceptance", "free": "measured acceptance",
                    "categorical": "accepted length per step drawn from a seeded categorical over 1..8 "
                                   "(p ~ 0.9083^k, mean 4)"}[args.accept]
    res = {
        "metric": "decode tok/s (Bonsai-1.7B-arch D8, bs1)" if args.model == "1p7b" else
                  f"decode tok/s (Bonsai-{args.model}-arch D8, bs1 per GPU)",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "s8 x ternary -> s32 (bf16 activations in memory)",
        "data": "synthetic",
        "config": {"workload": f"Bonsai-{args.model}-architecture {args.mode} MTP decode, random-init ternary "
                               f"weights, block 8, {accept_words}, {prompt_len}-token random "
                               f"prompt, {new_tokens} new tokens, batch 1, CUDA-graph replay, native T2 head "
                               "for draft and verify",
                   "segment": atlas.segment_ladder[0], "widths": list(atlas.m_set),
                   "timing": "value = timed decode tokens / decode seconds as the reference defines them "
                             "(first token and prefill excluded, host clock between device synchronisations); "
                             "ms_per_step and e2e = CUDA events around whole generate calls",
                   "l2": f"{rf['bytes'] / 1e6:.0f} MB of packed weights and scales are streamed per replay (> 3x L2)",
                   "one_request_stream_per_gpu": world > 1},
        "gpu_launches": launches, "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": "tok/s (prefill + all new tokens, host prompt in, tokens out)",
                "h2d_bytes_per_step": prompt_len * 8, "d2h_bytes_per_step": new_tokens * 8},
        "roofline": {"bound": "hbm", "achieved": round(rf["gbs"], 1), "peak": peak, "unit": "GB/s",
                     "frac": round(rf["gbs"] / peak, 4), "traffic": None, "peak_kind": peak_kind,
                     "kernel": f"t2_gemv (cooperative-tile and row-per-warp kernels), the {rf['calls']} GEMV launches of one width-{roof_m} "
                               f"replay ({rf['bytes'] / 1e6:.1f} MB algorithmic, {rf['us_per_launch']:.2f} us "
                               "average per launch)",
                     "frac_of_8TBps": round(rf["gbs"] / 8000.0, 4)},
        "decode": {"iters_per_generation": iters / steps, "decode_ms_per_generation": dec_t / steps * 1e3,
                   "total_ms_per_generation": tot_t / steps * 1e3,
                   "graph_replays_timed": replays,
                   "tokens_per_iteration": round(tok / max(iters - steps, 1.0), 3)},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        res["cpu_baseline"] = cpu_decode_baseline(args.model, roof_m)
    return res


def cpu_decode_baseline(model_name: str, M: int, layers: int = 1, more_layers: int = 7) -> dict:
    """The CPU oracle's forward on this box's host cores, bounded: a `layers`-layer and a
    `more_layers`-layer model (same head) are timed at width M and the line through the two
    points is read at the full depth (every layer does the same work).  tokens/s = D tokens
    per width-16 replay, 1 per AR replay."""
    import numpy as np
    from . import synthetic
    from oracle import oracle as O
    geometry = dict(getattr(synthetic, GEOMETRIES[model_name]))
    full_layers = geometry["n_layers"]
    sigma = 1024
    # every host core, also under a launcher that exports OMP_NUM_THREADS=1 for its ranks
    O.lib().bmo_set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))

    def best_time(n_layers: int) -> float:
        cfg = synthetic.make_config(dict(geometry, n_layers=n_layers), block_size=8)
        state = {k: v.cpu() for k, v in synthetic.device_state(cfg, "cpu", seed=0).items()
                 if not k.startswith("_head")}
        om = O.OracleModel(cfg, state, max_positions=sigma + 17)
        kv = om.new_kv(sigma, 17)
        D = cfg["block_size"]
        role = O.ROLE_DRAFT if M > 1 else O.ROLE_AR
        toks = np.arange(M) % cfg["vocab_size"]
        pos = np.arange(500, 500 + M)
        ls = M - D if M > 1 else 0
        best = float("inf")
        for i in range(4):                              # first pass warms the caches
            t0 = time.time()
            om.forward(toks, pos, kv, sigma, role, 500, max(M - D, 0), ls, M)
            if i:
                best = min(best, time.time() - t0)
        return best

    t_small, t_big = best_time(layers), best_time(more_layers)
    per_layer = max(t_big - t_small, 0.0) / (more_layers - layers)
    t_full = t_small + per_layer * (full_layers - layers)
    tokens = 8 if M > 1 else 1
    return {"value": round(tokens / t_full, 3), "unit": "tok/s", "cores": O.lib().bmo_num_threads(),
            "kind": "port",
            "sample": f"oracle forward at width {M}: {layers} and {more_layers} layers + head timed "
                      f"({t_small * 1e3:.0f} / {t_big * 1e3:.0f} ms), read at {full_layers} layers "
                      f"({t_full * 1e3:.0f} ms per replay)"}


def run_nsplit(args, world, rank, local, dist):
    """Wide-layer stress shape (K = 8192 -> N = 28672) split by output rows over the ranks:
    every rank streams its own N/world rows and the [W, N/world] slices are all-gathered
    with NCCL, so that every rank ends with the full output.  Total work is fixed (strong
    scaling); value = algorithmic bytes of the whole layer / time per call (max over ranks).
    Each rank rotates over enough distinct copies of its shard to exceed L2."""
    import bench
    from . import native, ops, synthetic
    from .nsplit import NSplitLinear, shard_rows
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    N, K = 28672, 8192
    widths = (1, 8)
    steps = args.steps or 20
    warmup = args.warmup if args.warmup is not None else 5
    n0, n1 = shard_rows(N, world, rank)
    rows = n1 - n0
    shard_bytes = rows * K // 4
    copies = max(2, -(-(256 << 20) // shard_bytes))
    gen = torch.Generator(device=device).manual_seed(1 + rank)

    def gemv(a, s_, weight, scale, out):
        ops.t2_gemv(a, weight, s_, scale, out=out, ldc=out.shape[1])

    fused = world > 1 and os.environ.get("BM_NSPLIT_NCCL", "0") != "1"
    layers = []
    for _ in range(copies):
        w_, sc = synthetic.device_ternary(rows, K, gen, device)
        if fused:
            from .nsplit import FusedNSplitLinear
            layers.append(FusedNSplitLinear(w_, sc, n_full=N, max_w=max(widths)))
        else:
            layers.append(NSplitLinear(w_, sc, rank=rank, world=world, gemv=gemv, sharded=True))
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
        graph = bench.capture(one_pass, device)
        timed = graph.replay
    for _ in range(warmup):
        timed()
    bench.barrier(dist)
    sampler = bench.ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        timed()
    e1.record()
    bench.barrier(dist)
    clocks = sampler.stop()
    ms = bench.max_over_ranks(dist, e0.elapsed_time(e1), device)
    calls = len(widths) * copies
    layer_bytes = sum(ops.gemv_bytes(w, N, K) for w in widths) * copies     # whole layer, all ranks
    value = layer_bytes * steps / (ms * 1e-3) / 1e9
    shard_alg = sum(ops.gemv_bytes(w, rows, K) for w in widths) * copies
    gbs_rank = shard_alg * steps / (ms * 1e-3) / 1e9

    e2e_pass()
    bench.barrier(dist)
    t0 = time.time()
    e2e_steps = max(1, min(steps, 5))
    for _ in range(e2e_steps):
        e2e_pass()
    bench.barrier(dist)
    e2e_s = bench.max_over_ranks(dist, time.time() - t0, device)
    err = native.lib().bm_device_error()
    if err:
        raise RuntimeError(f"device error word = {err}")
    peak, peak_kind = bench.peaks()
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
                     "frac": round(gbs_rank / peak, 4), "traffic": None, "peak_kind": peak_kind,
                     "kernel": f"t2_gemv on this rank's {rows} x {K} shard, all-gather time included",
                     "frac_of_8TBps": round(gbs_rank / 8000.0, 4)},
    }


def run_reference_decode(args) -> dict:
    """CPU arm of bench.py: the oracle port of the reference path on all host threads, on a
    bounded sample of the same workload (see cpu_decode_baseline)."""
    steps = args.steps or 1
    warmup = args.warmup if args.warmup is not None else 0
    M = 16 if args.mode in ("hybrid", "conf") else (1 if args.mode == "ar" else 9)
    t0 = time.time()
    base = cpu_decode_baseline(args.model, M)
    dt = time.time() - t0
    ref_cuda = None
    if args.model == "1p7b":
        # the reference's own CUDA GEMV on the GEMV calls of one width-M replay (28 layers + head)
        import bench
        rows = {1: 1, 9: 9, 16: 8}[M]
        per_layer = [("qkv", 4096, 2048, M), ("o", 2048, 2048, M), ("gate|up", 12288, 2048, M),
                     ("down", 2048, 6144, M)]
        ref_cuda = bench.reference_cuda_sweep(per_layer + [("head", 151936, 2048, rows)])
        if ref_cuda is not None:
            pc = ref_cuda["per_case"]
            layer_us = sum(pc[f"{n}x{k}:W{w}"]["us"] for (_, n, k, w) in per_layer)
            ref_cuda["gemv_us_per_replay"] = round(28 * layer_us + pc[f"151936x2048:W{rows}"]["us"], 1)
    return {"impl": "reference", "reference_cuda_kernel": ref_cuda, "metric": "decode tok/s (Bonsai-1.7B-arch D8, bs1)" if args.model == "1p7b"
            else f"decode tok/s (Bonsai-{args.model}-arch D8, bs1 per GPU)",
            "value": base["value"], "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": round(dt * 1e3, 1), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8 x ternary -> s32 (bf16 activations in memory)",
            "data": "synthetic",
            "config": {"workload": f"same decode replay on host cores: CPU oracle port of the reference path, "
                                   f"{base['sample']}"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
