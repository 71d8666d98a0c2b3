"""N-split of one wide T2-g128 layer across the GPUs of a node.

Output rows of the packed weight are independent, so rank r keeps rows
[r*N/G, (r+1)*N/G) of the codes and scales (activations and multipliers are replicated,
a few KB), computes its [W, N/G] slice with the ordinary GEMV and the slices are
all-gathered over NVLink with NCCL.  Every rank ends with the full [W, N] output, and
because the per-row arithmetic does not depend on which rank computes it, the gathered
result is bit-identical to the single-GPU one.  The reference has no multi-GPU inference
path; this is the exchange step the wide-layer configuration of the baseline asks for.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

ROW_ALIGN = 32     # a shard is a whole number of 32-row tiles


def shard_rows(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Row range of `rank`.  Requires N divisible by world * 32 (28672 / {1,2,4,8} is)."""
    if n % (world * ROW_ALIGN) != 0:
        raise ValueError(f"N={n} is not divisible into {world} shards of whole {ROW_ALIGN}-row tiles")
    per = n // world
    return rank * per, (rank + 1) * per


class NSplitLinear:
    """One rank's shard of a [N, K] packed layer plus the gather of the outputs.

    `gemv(a, s, weight, scale, out)` computes out[W, rows] for this shard; on a GPU it is
    `ops.t2_gemv`, in the CPU tests an oracle-backed stand-in, so the sharding and the
    gather are exercised with gloo."""

    def __init__(self, weight: torch.Tensor, scale: torch.Tensor, *, rank: int, world: int,
                 gemv: Callable, group: Optional[dist.ProcessGroup] = None, sharded: bool = False):
        n_full = weight.shape[0] * (world if sharded else 1)
        self.n, self.rank, self.world, self.group, self.gemv = n_full, rank, world, group, gemv
        n0, n1 = shard_rows(n_full, world, rank)
        self.rows = n1 - n0
        self.weight = weight if sharded else weight[n0:n1].contiguous()
        self.scale = scale if sharded else scale[n0:n1].contiguous()
        self._gathered = None

    def forward(self, a_int8: torch.Tensor, s: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        """Returns the full [W, N] output on every rank."""
        W = a_int8.shape[0]
        local = torch.empty((W, self.rows), dtype=out_dtype, device=a_int8.device)
        self.gemv(a_int8, s, self.weight, self.scale, local)
        if self.world == 1:
            return local
        if (self._gathered is None or self._gathered.shape[0] != self.world * W
                or self._gathered.dtype != out_dtype):
            self._gathered = torch.empty((self.world * W, self.rows), dtype=out_dtype, device=a_int8.device)
        dist.all_gather_into_tensor(self._gathered, local, group=self.group)   # rank-major rows
        # [G*W, N/G] -> [W, N]; for W = 1 this is already contiguous
        return self._gathered.view(self.world, W, self.rows).permute(1, 0, 2).reshape(W, self.n)


class FusedNSplitLinear:
    """The same split with the exchange inside the GEMV kernel (bm_t2_gemv_nsplit): every rank's
    epilogue stores its [W, N/G] slice straight into every rank's output buffer over NVLink and one
    flag per peer says "my slice is there".  No collective library call on the data path.

    The output buffers and flag arrays live in torch symmetric memory (peer-mapped allocations).
    All ranks must call `forward` the same number of times with the same W.  A peer that never
    publishes (a rank that died or is far behind) ends the kernel's bounded wait: `failed_call()`
    then names the call whose output is invalid."""

    def __init__(self, weight: torch.Tensor, scale: torch.Tensor, *, n_full: int, max_w: int = 16,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import native
        self._ctypes, self._native = ctypes, native
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n = n_full
        n0, n1 = shard_rows(n_full, self.world, self.rank)
        if weight.shape[0] != n1 - n0:
            raise ValueError("weight must be this rank's shard of the rows")
        self.col0, self.rows, self.max_w = n0, n1 - n0, max_w
        self.weight, self.scale = weight, scale
        dev = weight.device
        # one allocation per rank: two [max_w, N] bf16 output buffers used in turn (a peer that is one
        # call ahead writes into the other one while this rank's consumers still read the current one),
        # then `world` uint32 flags (16-byte aligned)
        self.half_bytes = (max_w * n_full * 2 + 15) // 16 * 16
        self.out_bytes = 2 * self.half_bytes
        total = self.out_bytes + 64
        self.buf = symm_mem.empty((total,), dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        flag_off = self.out_bytes
        vp = ctypes.c_void_p
        pad = [vp(0)] * (8 - len(ptrs))
        self._peer_c = [(vp * 8)(*[vp(p + b * self.half_bytes) for p in ptrs] + pad) for b in range(2)]
        self._peer_flags = (vp * 8)(*[vp(p + flag_off) for p in ptrs] + pad)
        # CTA counter, completed calls, number of the last call whose peer wait ran out (0: none), unused
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)
        self.poll_limit = 0                     # polls of a peer's flag before the wait is given up (0: default)
        self.calls = 0
        self.out = [self.buf[b * self.half_bytes: b * self.half_bytes + max_w * n_full * 2]
                    .view(torch.bfloat16).view(max_w, n_full) for b in range(2)]
        torch.cuda.synchronize(dev)
        dist.barrier(group)                     # every rank's buffer is zeroed before anyone writes into it

    def forward(self, a_int8: torch.Tensor, s: torch.Tensor, pdl: bool = False) -> torch.Tensor:
        """Returns the full [W, N] output: a view of one of this rank's two symmetric buffers, valid
        until the call after the next one.  Capturable: the call number lives on the device, so a graph
        with an even number of calls returns to the same buffers on every replay."""
        native, ctypes = self._native, self._ctypes
        W, K = a_int8.shape
        if W > self.max_w:
            raise ValueError(f"W={W} exceeds the buffer's {self.max_w} rows")
        self.calls += 1
        b = self.calls & 1
        stream = torch.cuda.current_stream(a_int8.device).cuda_stream
        cast = lambda arr: ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p))
        rc = native.lib().bm_t2_gemv_nsplit(
            a_int8.data_ptr(), self.weight.data_ptr(), s.data_ptr(), self.scale.data_ptr(), W, self.rows, K, self.n,
            self.col0, self.world, self.rank, cast(self._peer_c[0]), cast(self._peer_c[1]), cast(self._peer_flags),
            self.state.data_ptr(), int(self.poll_limit), int(pdl), stream)
        native.check(rc, "bm_t2_gemv_nsplit")
        return self.out[b][:W]

    def failed_call(self) -> int:
        """Number of the last `forward` call (1, 2, ...) whose wait for a peer ran out, 0 if none did.
        The output of that call holds stale columns for the silent peer and must not be used.  One
        4-byte device-to-host copy; callers that already read a result every step can read
        `self.state[2]` with it instead."""
        return int(self.state[2].item())
