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
