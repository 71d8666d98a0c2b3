"""Two-GPU check of the fused N-split GEMV (bm_t2_gemv_nsplit): every rank ends with the full
output, bit-identical to the single-GPU GEMV, on repeated calls.  Needs two CUDA devices; on a
one-GPU box the test is skipped.  The ranks are child processes; every wait in the kernel is bounded,
and the children leave only between calls."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from bitmtp_b200 import native, ops, synthetic
    from bitmtp_b200.nsplit import FusedNSplitLinear, shard_rows
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok = True
    try:
        for (W, N, K) in ((1, 28672, 8192), (8, 28672, 8192), (12, 4096, 2048)):
            case = synthetic.gemv_case(W, N, K, seed=11 + W)
            A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
            want = ops.t2_gemv(A, B, s, ws)
            n0, n1 = shard_rows(N, world, rank)
            lin = FusedNSplitLinear(B[n0:n1].contiguous(), ws[n0:n1].contiguous(), n_full=N)
            for rep in range(3):
                got = lin.forward(A, s)
                torch.cuda.synchronize(dev)
                ok = ok and bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
                dist.barrier()                  # nobody starts the next call while a peer still reads
            ok = ok and native.lib().bm_device_error() == 0
    finally:
        q.put((rank, ok))
        dist.barrier()
        dist.destroy_process_group()


def test_fused_nsplit_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    for _ in range(600):
        try:
            results.append(q.get(timeout=1))
            if len(results) == 2:
                break
        except Exception:
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    for p in procs:
        p.join(timeout=60)
    assert len(results) == 2 and all(ok for _, ok in results), results
