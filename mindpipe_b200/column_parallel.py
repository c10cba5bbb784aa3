"""Column-parallel W4A16 linear for the 70B-shaped layers: split the output rows of the
packed weight over the ranks, replicate the activations, all-gather the outputs.

Rank ``r`` of ``P`` holds rows ``[r*N/P, (r+1)*N/P)`` of ``weight_packed``, ``weight_scale`` and
``weight_zero_point``; each rank computes ``y[:, slice]`` with the single-GPU kernels and one
``all_gather_into_tensor`` assembles ``y[M, N]`` on every rank (tensor parallelism of the
column-parallel kind, as the third-party runtime does around ``AscendLinearMethod``;
acceleration/runtime_patches/vllm_ascend.patch:3260-3305 shows its all-gather call sites).
Per GPU the weight stream shrinks by ``P``; the collective moves ``2*M*N`` bytes in total.

At decode sizes the gather is a few hundred kilobytes and a library collective is all latency, so the
default exchange is a device-driven one over peer-mapped memory (``torch.distributed._symmetric_memory``):
one kernel stores this rank's slice into every peer's receive buffer with plain peer stores whose every
8 bytes carry 4 bytes of payload and the call number, and polls (bounded) its own receive buffer for the
peers' slices while it assembles ``y[M, N]`` -- one one-way NVLink flight, no fence, arrival word, NCCL
call or host synchronisation, replayable from a CUDA graph.  ``forward_nccl`` is the plain form
(``all_gather_into_tensor``), used for batches above ``max_rows`` and without peer mappings.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Row range of ``rank``; ``n_rows`` must divide evenly (it does for the 70B shapes and P <= 8)."""
    if n_rows % world_size != 0:
        raise ValueError(f"{n_rows} output rows do not divide over {world_size} ranks")
    per = n_rows // world_size
    return rank * per, (rank + 1) * per


def shard_packed_linear(packed, scale, zero_point, bias, world_size: int, rank: int):
    """Slices of the four weight-side tensors for ``rank`` (views; call ``.contiguous()`` after ``.to(device)``)."""
    lo, hi = shard_rows(packed.shape[0], world_size, rank)
    return (packed[lo:hi], scale[lo:hi], None if zero_point is None else zero_point[lo:hi],
            None if bias is None else bias[lo:hi])


def assemble_gathered(gathered: torch.Tensor) -> torch.Tensor:
    """``[P, M, N/P]`` (what all-gather returns, rank-major) -> ``[M, N]``."""
    p, m, n_loc = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, p * n_loc)


class ColumnParallelW4A16Linear(torch.nn.Module):
    """``VllmPackedInt4Linear`` sharded by output rows over a process group."""

    def __init__(self, local_linear, out_features: int, group=None, gather_output: bool = True,
                 max_rows: int = 64, symmetric: bool = True):
        super().__init__()
        self.local = local_linear
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.out_features = int(out_features)
        self.gather_output = gather_output
        self.max_rows = int(max_rows)
        lo, hi = shard_rows(self.out_features, self.world, self.rank)
        if local_linear.out_features != hi - lo:
            raise ValueError(f"rank {self.rank} must hold {hi - lo} rows, got {local_linear.out_features}")
        self.symmetric = bool(symmetric) and self.world > 1 and gather_output and ((hi - lo) * 2) % 16 == 0
        if self.symmetric:
            self._setup_symmetric()

    def _setup_symmetric(self):
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        dev = self.local.weight_packed.device
        n_loc = self.out_features // self.world
        # one receive buffer per call parity, in the flag-in-data wire form (twice the payload)
        self.recv_bytes = (_lib.load().mp_peer_allgather_recv_bytes(self.max_rows, n_loc * 2, self.world) + 255) // 256 * 256
        self.buf = symm.empty(2 * self.recv_bytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()                                                              # call numbers start at 1
        torch.cuda.synchronize(dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)                                                      # every rank zeroed its buffer
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self.p_recv = [(ctypes.c_void_p * self.world)(*[b + par * self.recv_bytes for b in bases]) for par in range(2)]
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)     # blocks of the running call that are done
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)       # calls completed (advanced by the kernel)

    @staticmethod
    def from_full(packed, scale, zero_point, bias, in_features: int, group=None, device=None, **kw):
        from .modules import VllmPackedInt4Linear
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        p, s, z, b = shard_packed_linear(packed, scale, zero_point, bias, world, rank)
        to = (lambda t: None if t is None else t.to(device).contiguous())
        local = VllmPackedInt4Linear(packed_weight=to(p), scale=to(s), bias=to(b), in_features=in_features,
                                     out_features=p.shape[0], zero_point=to(z))
        return ColumnParallelW4A16Linear(local, packed.shape[0], group, **kw)

    @torch.no_grad()
    def forward(self, x):
        y_loc = self.local(x)
        if not self.gather_output or self.world == 1:
            return y_loc
        lead = y_loc.shape[:-1]
        y2 = y_loc.reshape(-1, y_loc.shape[-1]).contiguous()
        m, n_loc = y2.shape
        if not self.symmetric or m > self.max_rows or m == 0:
            return self._gather_nccl(y2).reshape(*lead, self.out_features)
        from . import _lib, ops
        out = torch.empty((m, self.out_features), dtype=y2.dtype, device=y2.device)
        st = _lib.load().mp_peer_allgather_push(y2.data_ptr(), m, n_loc * 2, self.p_recv[0], self.p_recv[1],
                                                self.epoch.data_ptr(), self.counter.data_ptr(), self.world,
                                                self.rank, out.data_ptr(), ops._error_word(y2.device).data_ptr(),
                                                torch.cuda.current_stream().cuda_stream)
        _lib.check(st, "peer_allgather_push", M=m, N=self.out_features)
        return out.reshape(*lead, self.out_features)

    @torch.no_grad()
    def forward_nccl(self, x):
        """Local linear, then ``all_gather_into_tensor`` (the exchange for process groups without peer mappings)."""
        y_loc = self.local(x)
        if not self.gather_output or self.world == 1:
            return y_loc
        y2 = y_loc.reshape(-1, y_loc.shape[-1]).contiguous()
        return self._gather_nccl(y2).reshape(*y_loc.shape[:-1], self.out_features)

    def _gather_nccl(self, y2):
        m, n_loc = y2.shape
        gathered = torch.empty((self.world * m, n_loc), dtype=y2.dtype, device=y2.device)   # rank-major rows
        dist.all_gather_into_tensor(gathered, y2, group=self.group)
        return assemble_gathered(gathered.view(self.world, m, n_loc))
