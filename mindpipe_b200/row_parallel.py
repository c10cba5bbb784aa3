"""Row-parallel W4A16 decode linear for the 70B-shaped layers: the input features (columns of the
packed weight) are split over the ranks, every rank multiplies its slice, and the partial sums are
added across GPUs.

Rank ``r`` of ``P`` holds columns ``[r*K/P, (r+1)*K/P)`` of the weight (tensor parallelism of the
row-parallel kind, what a serving runtime does for ``down_proj`` / ``o_proj``; the reference computes
the unsharded ``nn.Linear``, algorithm/quantization/ptq/awq/source/awq/quantize/quantizer.py:109-130).

The exchange is driven from the device, over peer-mapped memory (``torch.distributed._symmetric_memory``).
The decode kernel leaves its fp32 partial sums in a local buffer; a small second kernel then adds the ``P``
partial sums in rank order, in one of two forms.  Two-phase (the default): every rank sends each peer the
partial sums of the columns that peer owns, adds the ``P`` contributions to its own ``N / P`` columns, and
sends the fp16 result to everyone; every 8 bytes on the wire carry 4 bytes of payload and the call number,
so receivers poll the data itself and the all-reduce costs two one-way NVLink flights.  One-shot: the
decode kernel's last block raises an arrival word on every peer and every rank reads all ``P`` buffers
(``4 M N (P-1)`` bytes over NVLink, after an acknowledged fence).  Either way all ranks end with
bit-identical fp16 outputs, and no NCCL call, barrier kernel or host synchronisation sits on the path.  ``forward_nccl`` is the plain fallback (local linear + ``all_reduce``) for process groups
without peer mappings.
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

    def __init__(self, local_linear, bias=None, group=None, max_rows: int = 16, symmetric: bool = True,
                 two_phase: bool | None = None):
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
        # two-phase (reduce own columns, then exchange fp16 slices) needs N to split into 4-column units per rank
        can_split = self.out_features % (4 * self.world) == 0
        self.two_phase = (True if two_phase is None else bool(two_phase)) and can_split
        if self.symmetric:
            self._setup_symmetric()

    def _setup_symmetric(self):
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        dev = self.local.weight_packed.device
        self.slot_bytes = self.max_rows * self.out_features * 4                      # one [m_cap][N] fp32 buffer
        self.off_partial = 256                                                        # arrival words first
        lib = _lib.load()
        up = lambda v: (int(v) + 255) // 256 * 256
        self.recv1_bytes = up(lib.mp_w4a16_rowparallel_recv_bytes(self.max_rows, self.out_features, 1))
        self.recv2_bytes = up(lib.mp_w4a16_rowparallel_recv_bytes(self.max_rows, self.out_features, 2))
        self.off_recv1 = self.off_partial + 2 * self.slot_bytes
        self.off_recv2 = self.off_recv1 + 2 * self.recv1_bytes
        total = self.off_recv2 + 2 * self.recv2_bytes
        self.buf = symm.empty(total, dtype=torch.uint8, device=dev)
        self.buf.zero_()                                                              # call numbers start at 1
        torch.cuda.synchronize(dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)                                                      # every rank zeroed its words
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self.p_flags = (ctypes.c_void_p * self.world)(*bases)
        self.p_flags_self = (ctypes.c_void_p * 1)(bases[self.rank])
        self.p_partial = [(ctypes.c_void_p * self.world)(*[b + self.off_partial + par * self.slot_bytes for b in bases])
                          for par in range(2)]
        self.p_recv1 = [(ctypes.c_void_p * self.world)(*[b + self.off_recv1 + par * self.recv1_bytes for b in bases])
                        for par in range(2)]
        self.p_recv2 = [(ctypes.c_void_p * self.world)(*[b + self.off_recv2 + par * self.recv2_bytes for b in bases])
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
        self.local._ensure_prepared()
        stream = torch.cuda.current_stream().cuda_stream
        y = torch.empty((m, self.out_features), dtype=torch.float16, device=x2.device)
        mine = self.buf.data_ptr() + self.off_partial
        # the two-phase finish polls the data itself, so the decode kernel announces to nobody but this rank
        flags, world, rank = (self.p_flags_self, 1, 0) if self.two_phase else (self.p_flags, self.world, self.rank)
        st = lib.mp_w4a16_rowparallel_push(x2.data_ptr(), self.local.weight_packed.data_ptr(),
                                           self.local._scale_zero.data_ptr(), mine, mine + self.slot_bytes,
                                           flags, self.counter.data_ptr(), self.epoch.data_ptr(), world,
                                           rank, m, self.out_features, k_loc, self.local.group_size, stream)
        _lib.check(st, "w4a16_rowparallel_push", M=m, N=self.out_features, K_local=k_loc)
        bias = None if self.bias is None else self.bias.data_ptr()
        err = ops._error_word(x2.device).data_ptr()
        if self.two_phase:
            st = lib.mp_w4a16_rowparallel_finish_ll(mine, mine + self.slot_bytes, self.p_recv1[0], self.p_recv1[1],
                                                    self.p_recv2[0], self.p_recv2[1], self.world, self.rank,
                                                    self.epoch.data_ptr(), m, self.out_features, bias, y.data_ptr(), err,
                                                    stream)
        else:
            st = lib.mp_w4a16_rowparallel_finish(self.p_partial[0], self.p_partial[1], self.buf.data_ptr(), self.world,
                                                 self.epoch.data_ptr(), m, self.out_features, bias, y.data_ptr(), err,
                                                 stream)
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


class RowParallelW8A8Linear(torch.nn.Module):
    """W8A8 linear sharded by input features, the role of the runtime's fused "int8 matmul + all-reduce"
    (``npu_mm_all_reduce_base``, acceleration/runtime_patches/vllm_ascend.patch:1428-1449).

    Rank ``r`` holds ``weight[:, K_r]`` (int8 ``[N, K/P]``) and the per-channel ``weight_scale[N]`` of the
    whole weight (the same on every rank, as stored in a W8A8 checkpoint);
    ``forward(x_local)`` takes ``x[:, K_r]`` (fp16), quantises it per token *on this rank* (each rank has
    its own per-token scales, as in the runtime op), multiplies into raw int32 accumulators that live
    in peer-mapped memory, raises an arrival word on the peers, and a finish kernel on every rank reads all
    accumulators and token scales over NVLink and adds the dequantised partial products in rank order:
    bit-identical outputs on all ranks, no NCCL call or host synchronisation on the path.

    The quantiser and the GEMM write to ordinary local buffers; a publish kernel copies them into the
    receive slot of the call number's parity (the number lives in device memory), so the two slots
    alternate from call to call however the launches were issued -- eagerly, or from a captured graph
    with any number of forwards in it.
    """

    def __init__(self, weight_i8, weight_scale, bias=None, group=None, max_rows: int = 256):
        super().__init__()
        import torch.distributed._symmetric_memory as symm
        if weight_i8.dtype != torch.int8 or weight_i8.dim() != 2:
            raise TypeError("weight_i8 must be an int8 [N, K_local] tensor")
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.weight = weight_i8.contiguous()
        self.weight_scale = weight_scale.detach().flatten().to(torch.float32).contiguous()
        self.bias = None if bias is None else bias.detach().to(torch.float16).contiguous()
        self.out_features, self.in_features = self.weight.shape
        if self.weight_scale.numel() != self.out_features:
            raise ValueError("weight_scale must have one entry per output feature")
        self.max_rows = int(max_rows)
        dev = self.weight.device
        al = lambda n: (n + 255) // 256 * 256
        self.acc_bytes = al(self.max_rows * self.out_features * 4)
        self.scale_bytes = al(self.max_rows * 4)
        self.off_acc = [256, 256 + self.acc_bytes + self.scale_bytes]                # two (acc | xscale) buffers
        self.off_scale = [o + self.acc_bytes for o in self.off_acc]
        self.buf = symm.empty(256 + 2 * (self.acc_bytes + self.scale_bytes), dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize(dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)
        bases = [int(p) for p in self.handle.buffer_ptrs]
        mk = lambda off: (ctypes.c_void_p * self.world)(*[b + off for b in bases])
        self.p_flags = mk(0)
        self.p_acc = [mk(o) for o in self.off_acc]
        self.p_scale = [mk(o) for o in self.off_scale]
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)     # calls completed (advanced on the device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)   # blocks of the publish kernel that have copied
        self.acc_local = torch.empty(self.max_rows * self.out_features, dtype=torch.int32, device=dev)
        self.scale_local = torch.empty(self.max_rows, dtype=torch.float32, device=dev)

    @staticmethod
    def from_float(linear: torch.nn.Linear, group=None, **kw):
        """Quantise the FULL fp16 weight per output channel (the a8 producer: fp16 arithmetic) and keep
        this rank's column slice.  The per-channel scale comes from the whole row, so it is the same
        on every rank -- as in a W8A8 checkpoint, whose ``weight_scale`` is stored once per channel."""
        from . import ops
        g = dist.group.WORLD if group is None else group
        world, rank = dist.get_world_size(g), dist.get_rank(g)
        q, s, _ = ops.act_quant_per_token(linear.weight.detach().contiguous())
        k = q.shape[1]
        if k % world:
            raise ValueError(f"{k} input features do not divide over {world} ranks")
        lo, hi = rank * k // world, (rank + 1) * k // world
        return RowParallelW8A8Linear(q[:, lo:hi].contiguous(), s, linear.bias, g, **kw)

    @torch.no_grad()
    def forward(self, x_local):
        from . import _lib, ops
        lib = _lib.load()
        x2 = x_local.reshape(-1, x_local.shape[-1]).contiguous()
        m, k_loc = x2.shape
        if m > self.max_rows or k_loc != self.in_features or x2.dtype != torch.float16:
            raise ValueError(f"x_local must be fp16 [<= {self.max_rows}, {self.in_features}], got {tuple(x2.shape)}")
        stream = torch.cuda.current_stream().cuda_stream
        base = self.buf.data_ptr()
        qx = torch.empty((m, k_loc), dtype=torch.int8, device=x2.device)
        y = torch.empty((m, self.out_features), dtype=torch.float16, device=x2.device)
        err = ops._error_word(x2.device).data_ptr()
        _lib.check(lib.mp_act_quant_per_token(x2.data_ptr(), m, k_loc, qx.data_ptr(), self.scale_local.data_ptr(), None,
                                              stream), "act_quant_per_token", M=m, K=k_loc)
        _lib.check(lib.mp_w8a8_gemm_i32(qx.data_ptr(), self.weight.data_ptr(), self.acc_local.data_ptr(), m,
                                        self.out_features, k_loc, err, stream),
                   "w8a8_gemm_i32", M=m, N=self.out_features, K=k_loc)
        # a peer may still read call n while this rank computes call n+1: two slots, chosen on the device
        _lib.check(lib.mp_peer_publish(self.acc_local.data_ptr(), m * self.out_features * 4, 0,
                                       self.scale_local.data_ptr(), m * 4, self.acc_bytes,
                                       base + self.off_acc[0], base + self.off_acc[1], self.p_flags,
                                       self.epoch.data_ptr(), self.counter.data_ptr(), self.world, self.rank, stream),
                   "peer_publish", M=m, N=self.out_features)
        _lib.check(lib.mp_w8a8_rowparallel_finish_parity(self.p_acc[0], self.p_acc[1], self.p_scale[0], self.p_scale[1],
                                                         base, self.world, self.epoch.data_ptr(), m, self.out_features,
                                                         self.weight_scale.data_ptr(),
                                                         None if self.bias is None else self.bias.data_ptr(),
                                                         y.data_ptr(), err, stream),
                   "w8a8_rowparallel_finish", M=m, N=self.out_features)
        return y.reshape(*x_local.shape[:-1], self.out_features)

    @torch.no_grad()
    def forward_nccl(self, x_local):
        """Per-rank W8A8 linear in fp32, then ``all_reduce`` (sum order is the library's)."""
        from . import ops
        x2 = x_local.reshape(-1, x_local.shape[-1]).contiguous()
        qx, sx, _ = ops.act_quant_per_token(x2)
        acc = ops.w8a8_gemm_i32(qx, self.weight)
        y = acc.to(torch.float32) * sx[:, None] * self.weight_scale[None, :]
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        if self.bias is not None:
            y = y + self.bias.to(torch.float32)
        return y.to(torch.float16).reshape(*x_local.shape[:-1], self.out_features)
