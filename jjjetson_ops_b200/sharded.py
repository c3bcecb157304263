"""One Q4_0 linear, column-sharded along N over the ranks of a process group.

Output column ``n`` of ``Y = X W^T`` depends only on weight row ``n`` and on all of ``X``, so the
weight rows are split into contiguous shards (multiples of 32 rows), every rank keeps its shard
resident, the activations are replicated, each rank computes ``Y[:, shard]`` with the single-GPU
kernels, and one all-gather along N assembles ``[M, N]`` on every rank.  One process per GPU;
``torch.distributed`` (NCCL over NVLink, or gloo on CPU for tests) is the only plumbing.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import synth


class ShardedLinearQ4_0:
    def __init__(self, w_q4_0: torch.Tensor, N: int, K: int,
                 compute: Optional[Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor]] = None,
                 group=None, device: Optional[torch.device] = None, already_sharded: bool = False):
        """``w_q4_0``: uint8 ``[N, K/32*18]`` (all rows; this rank's rows are kept) or, with
        ``already_sharded``, just this rank's rows.  ``compute(w_shard, x, n_rows) -> [M, n_rows]``
        defaults to the CUDA linear."""
        self.N, self.K = N, K
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.row_span: Tuple[int, int] = synth.shard_rows(N, self.world, self.rank)
        b, e = self.row_span
        row_bytes = K // 32 * 18
        w2d = w_q4_0.reshape(-1, row_bytes)
        shard = w2d if already_sharded else w2d[b:e]
        if shard.shape[0] != e - b:
            raise ValueError("weight shard has %d rows, expected %d" % (shard.shape[0], e - b))
        if device is not None:
            shard = shard.to(device)
        self.w_shard = shard.contiguous()
        self.max_rows = max(synth.shard_rows(N, self.world, r)[1] - synth.shard_rows(N, self.world, r)[0]
                            for r in range(self.world))
        if compute is None:
            from . import capi

            def compute(w, x, n_rows):  # noqa: ANN001
                return capi.linear_q4_0(w, x, n_rows)

        self._compute = compute
        self._gather_buf: Optional[torch.Tensor] = None
        self._local_buf: Optional[torch.Tensor] = None

    def local(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's band ``Y[:, begin:end]``."""
        b, e = self.row_span
        return self._compute(self.w_shard, x, e - b)

    def gather(self, y_local: torch.Tensor) -> torch.Tensor:
        """All-gather of the bands along N -> ``[M, N]`` on every rank."""
        M = y_local.shape[0]
        if self.world == 1:
            return y_local
        b, e = self.row_span
        if self._local_buf is None or self._local_buf.shape != (M, self.max_rows) or self._local_buf.device != y_local.device:
            self._local_buf = torch.zeros((M, self.max_rows), dtype=torch.float32, device=y_local.device)
            self._gather_buf = torch.empty((self.world * M, self.max_rows), dtype=torch.float32, device=y_local.device)
        self._local_buf[:, : e - b].copy_(y_local)
        dist.all_gather_into_tensor(self._gather_buf, self._local_buf, group=self.group)
        bands = self._gather_buf.view(self.world, M, self.max_rows)
        if self.max_rows * self.world == self.N:
            return bands.permute(1, 0, 2).reshape(M, self.N)
        parts = []
        for r in range(self.world):
            rb, re = synth.shard_rows(self.N, self.world, r)
            parts.append(bands[r, :, : re - rb])
        return torch.cat(parts, dim=1)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.gather(self.local(x))
