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


def test_peer_wait_runs_out_and_is_reported():
    """One GPU stands in for rank 0 of a two-rank split whose peer never answers: the "peer's" output
    buffers and flag array are local scratch nobody publishes to.  With a small poll limit the
    kernel's bounded wait must run out and RETURN (no trap, no hang), name the call in its status
    word, set the device error word to 4, and still leave this rank's own columns correct."""
    import ctypes

    from bitmtp_b200 import native, ops, synthetic
    dev = torch.device("cuda:0")
    W, N, K, world = 4, 4096, 2048, 2
    case = synthetic.gemv_case(W, N, K, seed=3)
    A, B, ws, s = (case[k].to(dev) for k in ("A", "B", "ws", "s"))
    rows = N // world
    want = ops.t2_gemv(A, B[:rows].contiguous(), s, ws[:rows].contiguous())          # this rank's shard
    mine = [torch.zeros(W, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    theirs = [torch.zeros(W, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    my_flags = torch.zeros(16, dtype=torch.int32, device=dev)       # the silent peer never writes here
    their_flags = torch.zeros(16, dtype=torch.int32, device=dev)
    state = torch.zeros(4, dtype=torch.int32, device=dev)
    vp = ctypes.c_void_p
    arr = lambda a, b: ctypes.cast((vp * 8)(vp(a.data_ptr()), vp(b.data_ptr()), *([vp(0)] * 6)), ctypes.POINTER(vp))
    lib = native.lib()
    assert lib.bm_device_error() == 0
    w_shard, ws_shard = B[:rows].contiguous(), ws[:rows].contiguous()
    rc = lib.bm_t2_gemv_nsplit(A.data_ptr(), w_shard.data_ptr(), s.data_ptr(), ws_shard.data_ptr(), W, rows, K, N, 0,
                               world, 0, arr(mine[0], theirs[0]), arr(mine[1], theirs[1]), arr(my_flags, their_flags),
                               state.data_ptr(), 2000, 0, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(dev)                                       # returns: the wait was bounded
    st = state.cpu().tolist()
    assert st[0] == 0 and st[1] == 1 and st[2] == 1, st              # call 1 is marked as failed
    assert lib.bm_device_error() == 4                                 # and the error word says why
    assert lib.bm_device_error() == 0                                 # (read-and-clear)
    got = mine[1][:, :rows]                                           # call 1 uses buffer 1
    assert torch.equal(got.contiguous().view(torch.int16), want.view(torch.int16))
    assert torch.equal(theirs[1][:, :rows].contiguous().view(torch.int16), want.view(torch.int16))   # pushed to the peer too
    assert int(their_flags[0].item()) == 1                            # published to the peer before waiting
    # a healthy call afterwards (peer flag set by hand) leaves the status word alone
    my_flags[1] = 2
    rc = lib.bm_t2_gemv_nsplit(A.data_ptr(), w_shard.data_ptr(), s.data_ptr(), ws_shard.data_ptr(), W, rows, K, N, 0,
                               world, 0, arr(mine[0], theirs[0]), arr(mine[1], theirs[1]), arr(my_flags, their_flags),
                               state.data_ptr(), 2000, 0, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(dev)
    assert state.cpu().tolist()[1:3] == [2, 1] and lib.bm_device_error() == 0
