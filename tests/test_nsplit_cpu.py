"""World-size-2 gloo test of the N-split path: sharding + all-gather reproduce the
single-rank output bit for bit (per-row arithmetic does not depend on the rank)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_gemv(a, s, weight, scale, out):
    from oracle import oracle as O
    _, y16, _ = O.t2_gemv(a.numpy(), weight.numpy().view(np.uint8), O.torch_to_u16(scale), s.numpy().reshape(-1))
    out.copy_(O.u16_to_torch(y16))


def _worker(rank, world, port, W, N, K, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bitmtp_b200 import synthetic
    from bitmtp_b200.nsplit import NSplitLinear
    case = synthetic.gemv_case(W, N, K, seed=9)
    lin = NSplitLinear(case["B"], case["ws"], rank=rank, world=world, gemv=_oracle_gemv)
    full = lin.forward(case["A"], case["s"])
    if rank == 0:
        q.put(full.view(torch.int16).numpy().copy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("W", [1, 8])
def test_nsplit_matches_single_rank(W):
    from bitmtp_b200 import synthetic
    from bitmtp_b200.nsplit import shard_rows
    N, K, world = 256, 512, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + W
    procs = [ctx.Process(target=_worker, args=(r, world, port, W, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = None
    for _ in range(180):
        try:
            got = q.get(timeout=1)
            break
        except Exception:
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    assert got is not None, "a worker exited without a result"
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    case = synthetic.gemv_case(W, N, K, seed=9)
    want = torch.empty(W, N, dtype=torch.bfloat16)
    _oracle_gemv(case["A"], case["s"], case["B"], case["ws"], want)
    assert np.array_equal(got, want.view(torch.int16).numpy())
    assert shard_rows(28672, 8, 3) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        shard_rows(100, 2, 0)
