"""Row-parallel W4A16 decode linear for the 70B-shaped layers: the input features (columns of the
packed weight) are split over the ranks, every rank multiplies its slice, and the partial sums are
added across GPUs.

Rank ``r`` of ``P`` holds columns ``[r*K/P, (r+1)*K/P)`` of the weight (tensor parallelism of the
row-parallel kind, what a serving runtime does for ``down_proj`` / ``o_proj``; the reference computes
the unsharded ``nn.Linear``, algorithm/quantization/ptq/awq/source/awq/quantize/quantizer.py:109-130).

The exchange is driven from the device: the decode kernel leaves its fp32 partial sums in a peer-mapped
buffer (``torch.distributed._symmetric_memory``) and its last block raises an arrival word on every
peer; a small second kernel waits for all arrival words, reads the ``P`` buffers over NVLink and adds
them in rank order -- so all ranks end with bit-identical fp16 outputs, and no NCCL call, barrier
kernel or host synchronisation sits on the path.  ``forward_nccl`` is the plain fallback (local linear +
``all_reduce``) for process groups without peer mappings.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


def shard_columns(n_cols: int, world_size: int, rank: int, group_size: int) -> tuple[int, int]:
    """Column range of ``rank``; shards are whole quantisation groups (and whole packed words)."""
    if n_cols % world_size != 0:
        raise ValueError(f"{n_cols} input features do not divide over {world_size} ranks")
    per = n_cols // world_size
    if per % group_size != 0 or per % 8 != 0:
        raise ValueError(f"a shard of {per} columns is not a whole number of groups of {group_size}")
    return rank * per, (rank + 1) * per


def unpack_nibbles(packed: torch.Tensor, count: int) -> torch.Tensor:
    """int32 ``[N, ceil(count/8)]`` -> uint8 ``[N, count]``; nibble ``j`` of word ``c`` is element ``8c+j``."""
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    vals = (packed.unsqueeze(-1) >> shifts) & 0xF
    return vals.reshape(packed.shape[0], -1)[:, :count].to(torch.uint8)


def pack_nibbles(vals: torch.Tensor) -> torch.Tensor:
    """uint8 ``[N, count]`` (values 0..15) -> int32 ``[N, ceil(count/8)]``, same nibble order."""
    n, count = vals.shape
    words = (count + 7) // 8
    padded = torch.zeros((n, words * 8), dtype=torch.int64, device=vals.device)
    padded[:, :count] = vals.to(torch.int64)
    shifts = torch.arange(0, 32, 4, device=vals.device, dtype=torch.int64)
    word = (padded.reshape(n, words, 8) << shifts).sum(dim=-1)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)          # two's-complement int32 bit pattern
    return word.to(torch.int32)


def shard_packed_linear_columns(packed, scale, zero_point, world_size: int, rank: int, group_size: int):
    """Column slices of the weight-side tensors for ``rank``: packed codes and scales are plain slices;
    the packed zero points (8 groups per word) are re-packed, since a shard need not start on a word."""
    k = packed.shape[1] * 8
    lo, hi = shard_columns(k, world_size, rank, group_size)
    g_lo, g_hi = lo // group_size, hi // group_size
    z = None
    if zero_point is not None:
        z = pack_nibbles(unpack_nibbles(zero_point, k // group_size)[:, g_lo:g_hi])
    return packed[:, lo // 8:hi // 8], scale[:, g_lo:g_hi], z


class RowParallelW4A16Linear(torch.nn.Module):
    """``VllmPackedInt4Linear`` sharded by input features; ``forward(x_local)`` takes this rank's slice
    ``x[:, K_r]`` (<= ``max_rows`` rows) and returns the full ``y[M, N]`` on every rank."""

    def __init__(self, local_linear, bias=None, group=None, max_rows: int = 16, symmetric: bool = True):
        super().__init__()
        self.local = local_linear
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.out_features = local_linear.out_features
        self.max_rows = int(max_rows)
        if local_linear.bias is not None:
            raise ValueError("the local shard must not carry the bias (it would be added once per rank)")
        self.bias = bias
        self.symmetric = bool(symmetric)
        if self.symmetric:
            self._setup_symmetric()

    def _setup_symmetric(self):
        import torch.distributed._symmetric_memory as symm
        dev = self.local.weight_packed.device
        self.slot_bytes = self.max_rows * self.out_features * 4                      # one [m_cap][N] fp32 buffer
        self.off_partial = 256                                                        # arrival words first
        total = self.off_partial + 2 * self.slot_bytes
        self.buf = symm.empty(total, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize(dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)                                                      # every rank zeroed its words
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self.p_flags = (ctypes.c_void_p * self.world)(*bases)
        self.p_partial = [(ctypes.c_void_p * self.world)(*[b + self.off_partial + par * self.slot_bytes for b in bases])
                          for par in range(2)]
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)     # blocks of the running call that have stored
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)       # calls completed (advanced by the kernel)

    @staticmethod
    def from_full(packed, scale, zero_point, bias, group_size: int, group=None, device=None, **kw):
        from .modules import VllmPackedInt4Linear
        g = dist.group.WORLD if group is None else group
        world, rank = dist.get_world_size(g), dist.get_rank(g)
        p, s, z = shard_packed_linear_columns(packed, scale, zero_point, world, rank, group_size)
        to = (lambda t: None if t is None else t.to(device).contiguous())
        local = VllmPackedInt4Linear(packed_weight=to(p), scale=to(s), bias=None, in_features=p.shape[1] * 8,
                                     out_features=p.shape[0], zero_point=to(z))
        return RowParallelW4A16Linear(local, None if bias is None else to(bias), group, **kw)

    @torch.no_grad()
    def forward(self, x_local):
        if not self.symmetric:
            return self.forward_nccl(x_local)
        from . import _lib, ops
        lib = _lib.load()
        x2 = x_local.reshape(-1, x_local.shape[-1]).contiguous()
        m, k_loc = x2.shape
        if m > self.max_rows or k_loc != self.local.in_features:
            raise ValueError(f"x_local must be [<= {self.max_rows}, {self.local.in_features}], got {tuple(x2.shape)}")
        if self.local._scale_zero is None:
            self.local.process_weights_after_loading()
        stream = torch.cuda.current_stream().cuda_stream
        y = torch.empty((m, self.out_features), dtype=torch.float16, device=x2.device)
        mine = self.buf.data_ptr() + self.off_partial
        st = lib.mp_w4a16_rowparallel_push(x2.data_ptr(), self.local.weight_packed.data_ptr(),
                                           self.local._scale_zero.data_ptr(), mine, mine + self.slot_bytes,
                                           self.p_flags, self.counter.data_ptr(), self.epoch.data_ptr(), self.world,
                                           self.rank, m, self.out_features, k_loc, self.local.group_size, stream)
        _lib.check(st, "w4a16_rowparallel_push", M=m, N=self.out_features, K_local=k_loc)
        st = lib.mp_w4a16_rowparallel_finish(self.p_partial[0], self.p_partial[1], self.buf.data_ptr(), self.world,
                                             self.epoch.data_ptr(), m, self.out_features,
                                             None if self.bias is None else self.bias.data_ptr(), y.data_ptr(),
                                             ops._error_word(x2.device).data_ptr(), stream)
        _lib.check(st, "w4a16_rowparallel_finish", M=m, N=self.out_features)
        return y.reshape(*x_local.shape[:-1], self.out_features)

    @torch.no_grad()
    def forward_nccl(self, x_local):
        """Local linear, then an fp32 ``all_reduce`` (sum order is the library's, not rank order)."""
        y = self.local(x_local).to(torch.float32)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        if self.bias is not None:
            y = y + self.bias.to(torch.float32)
        return y.to(torch.float16)
