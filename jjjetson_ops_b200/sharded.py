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


class PeerBands:
    """Output buffers of the fused multiply + all-gather (``jq_linear_q4_0_allgather_device``).

    Every rank allocates one block of peer-mappable memory holding two ``[M_max, N_total]`` fp32
    output buffers (used alternately, so that a fast rank never overwrites what a slow rank's
    consumer still reads) and its arrival counts, and maps the blocks of all other ranks.  The
    64-byte handles travel through ``all_gather_object``.
    """

    FLAG_BYTES = 256

    def __init__(self, M_max: int, N_total: int, device: torch.device, group=None, share_with: "Optional[PeerBands]" = None):
        """``share_with``: another ``PeerBands`` whose arrival counts and step counter this one uses too.  The
        layers of a chain share them, so that all-gathers are numbered across the chain and a layer's
        ``wait_previous`` waits for the bands of the layer before it."""
        from . import capi

        self._capi = capi
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("the fused all-gather handles up to 8 ranks")
        self.M_max, self.N_total = M_max, N_total
        self.y_bytes = (M_max * N_total * 4 + 255) // 256 * 256
        self._shared = share_with
        with torch.cuda.device(device):
            self.local_ptr, handle = capi.peer_alloc(2 * self.y_bytes + self.FLAG_BYTES)
        handles = [handle]
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
        self.ptrs = []
        with torch.cuda.device(device):
            for q in range(self.world):
                self.ptrs.append(self.local_ptr if q == self.rank else capi.peer_open(handles[q]))
        if share_with is None:
            self.counter = torch.zeros(1, dtype=torch.int32, device=device)
            self.epoch = torch.zeros(1, dtype=torch.int32, device=device)  # finished all-gathers, kept on the device
            self.flag_ptrs = [p + 2 * self.y_bytes for p in self.ptrs]
        else:
            self.counter, self.epoch, self.flag_ptrs = share_with.counter, share_with.epoch, share_with.flag_ptrs
        self._views = [capi.tensor_from_ptr(self.local_ptr + b * self.y_bytes, (M_max, N_total), torch.float32, device)
                       for b in range(2)]
        if self.world > 1:
            dist.barrier(group=group)  # everyone has mapped everyone before the first store

    def view(self, parity: int) -> torch.Tensor:
        """The ``[M, N_total]`` buffer that all-gathers of this parity (number & 1) fill."""
        return self._views[parity & 1]

    def linear(self, w_shard: torch.Tensor, x: torch.Tensor, ws: torch.Tensor, n_offset: int, N_local: int,
               s_mode: Optional[int] = None) -> None:
        """Queue one fused step.  The step first waits (on the device) for the previous step's bands;
        call ``wait()`` and then ``latest()`` to read the gathered output."""
        capi = self._capi
        M = x.shape[0]
        if M != self.M_max:
            raise ValueError("PeerBands was sized for M = %d" % self.M_max)
        y_peers = list(self.ptrs)
        flag_peers = list(self.flag_ptrs)
        capi.linear_q4_0_allgather(w_shard, x, ws, N_local, capi.S_D_SUM_Q if s_mode is None else s_mode, y_peers,
                                   flag_peers, self.world, self.rank, n_offset, self.N_total, self.y_bytes, True,
                                   self.epoch, self.counter)

    def wait(self) -> None:
        """Queue a wait (on the current stream) for the bands of the latest step from every rank."""
        self._capi.allgather_wait(self.device, self.flag_ptrs[self.rank], self.world, self.epoch)

    def latest(self) -> torch.Tensor:
        """After ``wait()``: the gathered ``[M, N_total]`` output of the latest step (synchronises to
        read the device-side step counter, which picks the buffer)."""
        return self._views[int(self.epoch.item()) & 1]

    def close(self) -> None:
        if self.local_ptr is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody is still storing into anybody
        with torch.cuda.device(self.device):
            for q, p in enumerate(self.ptrs):
                if q != self.rank:
                    self._capi.peer_close(p)
        if self.world > 1:
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            self._capi.peer_free(self.local_ptr)
        self.local_ptr = None


class TaggedBands:
    """Output buffers of the decode form of the fused all-gather (``jq_linear_q4_0_allgather_tagged_device``).

    Every output value travels as one 8-byte word ``{fp32 bits, number of its all-gather}``; the next sharded
    layer polls the words it needs, so nothing but the flight of the stores lies between one rank's last store
    and another rank's first use.  Every rank allocates one block of peer-mappable memory with two
    ``[M, N_total]`` word buffers (used alternately) and maps the blocks of all other ranks.  The all-gathers
    are numbered by a 64-bit count on the device, which the layers of a chain share (``share_with``).
    """

    def __init__(self, M: int, N_total: int, device: torch.device, group=None, share_with: "Optional[TaggedBands]" = None):
        from . import capi

        self._capi = capi
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("the fused all-gather handles up to 8 ranks")
        if M > 2:
            raise ValueError("the tagged form is the decode form: M <= 2")
        self.M, self.N_total = M, N_total
        self.y_bytes = (M * N_total * 8 + 255) // 256 * 256
        with torch.cuda.device(device):
            self.local_ptr, handle = capi.peer_alloc(2 * self.y_bytes)
        handles = [handle]
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
        self.ptrs = []
        with torch.cuda.device(device):
            for q in range(self.world):
                self.ptrs.append(self.local_ptr if q == self.rank else capi.peer_open(handles[q]))
        self.ticket = torch.zeros(1, dtype=torch.int64, device=device) if share_with is None else share_with.ticket
        self._out: Optional[torch.Tensor] = None
        if self.world > 1:
            dist.barrier(group=group)  # everyone has mapped everyone before the first store

    def linear(self, w_shard: torch.Tensor, K: int, n_offset: int, N_local: int, x: Optional[torch.Tensor] = None,
               source: "Optional[TaggedBands]" = None, seg_len: Optional[int] = None, seg_stride: int = 0,
               back: int = 0, s_mode: Optional[int] = None) -> None:
        """Queue one fused step.  The activations are the plain tensor ``x``, or an all-gather of ``source``:
        the one queued just before this call (``back`` = 0) or ``back`` calls earlier.  Activation ``k`` is
        word ``(k // seg_len) * seg_stride + k % seg_len`` of its row (``seg_len`` defaults to ``K``: the first
        ``K`` words).  ``seg_len`` is a multiple of 8 and ``seg_stride`` even; with ``seg_stride`` and the source's
        ``N_total`` multiples of 4 the kernel polls with 32-byte loads, which is faster."""
        capi = self._capi
        if (x is None) == (source is None):
            raise ValueError("exactly one of x and source")
        if x is not None and tuple(x.shape) != (self.M, K):
            raise ValueError("x must be [%d, %d]" % (self.M, K))
        if source is not None and source.M != self.M:
            raise ValueError("the source all-gather has a different M")
        capi.linear_q4_0_allgather_tagged(
            w_shard, x, 0 if source is None else source.local_ptr, 0 if source is None else source.y_bytes,
            0 if source is None else source.N_total, K if seg_len is None else seg_len, seg_stride, back, K, N_local, self.M,
            capi.S_D_SUM_Q if s_mode is None else s_mode, list(self.ptrs), self.world, self.rank, n_offset, self.N_total,
            self.y_bytes, self.ticket)

    def read(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Queue (on the current stream) a wait for every word of the latest all-gather, which must be this
        object's, and their conversion to a plain fp32 ``[M, N_total]`` tensor."""
        if out is None:
            if self._out is None:
                self._out = torch.empty((self.M, self.N_total), dtype=torch.float32, device=self.device)
            out = self._out
        self._capi.allgather_tagged_read(self.device, self.local_ptr, self.y_bytes, self.M, self.N_total, self.ticket, out)
        return out

    def close(self) -> None:
        if self.local_ptr is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody is still storing into anybody
        with torch.cuda.device(self.device):
            for q, p in enumerate(self.ptrs):
                if q != self.rank:
                    self._capi.peer_close(p)
        if self.world > 1:
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            self._capi.peer_free(self.local_ptr)
        self.local_ptr = None


def segments_of(gathered: torch.Tensor, K: int, seg_len: int, seg_stride: int) -> torch.Tensor:
    """The ``[M, K]`` activations that a layer reading ``gathered`` (``[M, N_total]``) with
    (``seg_len``, ``seg_stride``) sees: ``K / seg_len`` runs of ``seg_len`` columns, ``seg_stride`` apart."""
    parts = [gathered[:, q * seg_stride: q * seg_stride + seg_len] for q in range(K // seg_len)]
    return torch.cat(parts, dim=1).contiguous()
