"""Expert-parallel W8A8 MoE layer: one process per GPU, NCCL all-to-all dispatch / combine.

Experts are partitioned evenly over the ranks of a process group (rank ``p``
owns experts ``[p*E/P, (p+1)*E/P)``); tokens stay data-sharded.  A forward on
each rank is

1. route + gather + per-token int8 quantisation of the local tokens over ALL
   experts (``ops.moe_route_gather_quant``): rows sorted by expert, every
   expert segment padded to a multiple of 256 rows;
2. exchange of the per-expert row counts, then ``all_to_all_single`` of the
   int8 rows and of their fp32 scales -- the chunk for rank ``p`` is the
   contiguous run of its experts' segments, so nothing is re-packed before
   sending (activations travel as int8, the reference's "prequantize before
   communication", acceleration/runtime_patches/vllm_ascend.patch:1668-1682);
3. on the receiver, a row gather turns the source-major layout into
   expert-sorted rows (padding dropped), the expert stage runs on them
   (grouped int8 GEMM1 + SwiGLU + re-quant + grouped GEMM2), and the inverse
   gather puts the fp16 results back in arrival order;
4. ``all_to_all_single`` back (fp16) and the weighted combine at the token's
   home rank (``ops.moe_combine``), which indexes the returned rows with the
   ``dest_row`` table of step 1.

The layout arithmetic is pure Python over the exchanged counts
(:func:`plan_exchange`), so it is tested on CPU with ``gloo`` ranks; the
all-to-all role is that of the reference runtime's all-to-all dispatcher
(``TokenDispatcherWithAll2AllV``, vllm_ascend.patch:3228-3236).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

TILE = 128          # unit in which the device plan counts tiles
SEGMENT_ALIGN = 256  # every expert segment starts at a multiple of this (an even number of tiles)


def expert_partition(num_experts: int, world_size: int) -> list[tuple[int, int]]:
    """Contiguous, disjoint, complete expert ranges, one per rank."""
    if num_experts % world_size != 0:
        raise ValueError(f"{num_experts} experts do not divide over {world_size} ranks")
    per = num_experts // world_size
    return [(r * per, (r + 1) * per) for r in range(world_size)]


def _pad(n: np.ndarray | int):
    return (n + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN


@dataclass
class ExchangePlan:
    send_splits: list[int]        # rows sent to each rank (padded segments of its experts)
    recv_splits: list[int]        # rows received from each rank
    gather_map: np.ndarray        # int32 [padded_rows]: expert-sorted row -> row in the receive buffer (-1 = padding)
    scatter_map: np.ndarray       # int32 [recv_rows]: receive-buffer row -> expert-sorted row (-1 = padding)
    plan_ints: np.ndarray         # int32 device plan: counts | cursors | segment offsets | tile count | tile experts
    padded_rows: int              # rows of the expert-sorted buffers (multiple of 256, >= 256)
    recv_rows: int


def plan_exchange(send_counts: np.ndarray, recv_counts: np.ndarray, plan_len: int | None = None) -> ExchangePlan:
    """Layout of one dispatch from the per-expert row counts.

    ``send_counts[p, e]``: rows this rank routes to local expert ``e`` of rank ``p``;
    ``recv_counts[s, e]``: rows rank ``s`` routes to this rank's local expert ``e``.
    Segments are padded to 256 rows on the wire, exactly as the router laid them out.
    """
    send_counts = np.asarray(send_counts, dtype=np.int64)
    recv_counts = np.asarray(recv_counts, dtype=np.int64)
    world, e_loc = recv_counts.shape
    send_splits = _pad(send_counts).sum(axis=1)
    recv_pad = _pad(recv_counts)                      # [s, e] rows on the wire
    recv_splits = recv_pad.sum(axis=1)
    recv_rows = int(recv_splits.sum())
    # offset of segment (s, e) inside the receive buffer
    seg_start = np.zeros((world, e_loc), dtype=np.int64)
    off = 0
    for s in range(world):
        for e in range(e_loc):
            seg_start[s, e] = off
            off += recv_pad[s, e]
    per_expert = recv_counts.sum(axis=0)              # real rows per local expert
    padded = _pad(per_expert)
    padded_rows = max(int(padded.sum()), SEGMENT_ALIGN)
    gather_map = np.full(padded_rows, -1, dtype=np.int32)
    scatter_map = np.full(max(recv_rows, 1), -1, dtype=np.int32)
    seg_off = np.zeros(e_loc + 1, dtype=np.int64)
    pos = 0
    for e in range(e_loc):
        seg_off[e] = pos
        cur = pos
        for s in range(world):
            c = int(recv_counts[s, e])
            src = np.arange(seg_start[s, e], seg_start[s, e] + c, dtype=np.int64)
            gather_map[cur:cur + c] = src
            scatter_map[src] = np.arange(cur, cur + c, dtype=np.int32)
            cur += c
        pos += int(padded[e])
    seg_off[e_loc] = pos
    tiles = []
    for e in range(e_loc):
        tiles += [e] * int(padded[e] // TILE)
    n_ints = 3 * e_loc + 2 + max(len(tiles), padded_rows // TILE)
    if plan_len is not None:
        n_ints = max(n_ints, plan_len)
    plan = np.zeros(n_ints, dtype=np.int32)
    plan[:e_loc] = per_expert
    plan[2 * e_loc:3 * e_loc + 1] = seg_off
    plan[3 * e_loc + 1] = len(tiles)
    plan[3 * e_loc + 2:3 * e_loc + 2 + len(tiles)] = tiles
    return ExchangePlan([int(v) for v in send_splits], [int(v) for v in recv_splits], gather_map,
                        scatter_map[:recv_rows] if recv_rows else scatter_map[:0], plan, padded_rows, recv_rows)


class ExpertParallelMoE(torch.nn.Module):
    """W8A8 MoE experts sharded over a process group (drop-in for the single-GPU module's ``forward``).

    ``experts`` is a :class:`mindpipe_b200.modules.SmoothQuantPackedMoeExperts` built with
    ``expert_range`` = this rank's range; only its int8 buffers are used here.
    """

    def __init__(self, experts, num_experts: int, group=None):
        super().__init__()
        self.experts = experts
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_experts = int(num_experts)
        self.ranges = expert_partition(self.num_experts, self.world)
        if tuple(experts.expert_range) != self.ranges[self.rank]:
            raise ValueError(f"rank {self.rank} must hold experts {self.ranges[self.rank]}, got {experts.expert_range}")
        self.e_loc = self.num_experts // self.world

    @torch.no_grad()
    def forward(self, hidden_states, top_k_index, top_k_weights):
        from . import ops
        shape = hidden_states.shape
        hs = hidden_states.reshape(-1, shape[-1]).contiguous()
        t, h = hs.shape
        ids = top_k_index.reshape(t, -1).to(torch.int32).contiguous()
        w = top_k_weights.reshape(t, -1).to(torch.float16).contiguous()
        dev = hs.device
        # 1. local routing over all experts
        routing = ops.moe_route_gather_quant(hs, ids, 0, self.num_experts)
        send_counts = routing.counts.reshape(self.world, self.e_loc).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        both = torch.stack([send_counts, recv_counts]).cpu().numpy()          # the one host read of the layer
        plan = plan_exchange(both[0], both[1])
        # 2. dispatch: int8 rows + fp32 scales
        n_send = sum(plan.send_splits)
        recv_q = torch.empty((max(plan.recv_rows, 1), h), dtype=torch.int8, device=dev)[:plan.recv_rows]
        recv_s = torch.empty(max(plan.recv_rows, 1), dtype=torch.float32, device=dev)[:plan.recv_rows]
        dist.all_to_all_single(recv_q, routing.routed_q[:n_send], plan.recv_splits, plan.send_splits, group=self.group)
        dist.all_to_all_single(recv_s, routing.routed_scale[:n_send], plan.recv_splits, plan.send_splits,
                               group=self.group)
        # 3. expert stage on expert-sorted rows
        gmap = torch.from_numpy(plan.gather_map).to(dev, non_blocking=True)
        smap = torch.from_numpy(plan.scatter_map).to(dev, non_blocking=True)
        plan_dev = torch.from_numpy(plan.plan_ints).to(dev, non_blocking=True)
        q_sorted = ops.gather_rows(recv_q, gmap) if plan.recv_rows else torch.zeros((plan.padded_rows, h), dtype=torch.int8, device=dev)
        s_sorted = ops.gather_rows(recv_s, gmap) if plan.recv_rows else torch.zeros(plan.padded_rows, dtype=torch.float32, device=dev)
        ex = self.experts
        d_sorted = ops.moe_expert_stage(q_sorted, s_sorted, plan_dev, self.e_loc, ex.gate_up_proj,
                                        ex.gate_up_proj_scale, ex.down_proj, ex.down_proj_scale)
        d_recv = ops.gather_rows(d_sorted, smap) if plan.recv_rows else d_sorted[:0]
        # 4. return + combine at home
        back = torch.empty((routing.padded_rows, h), dtype=torch.float16, device=dev)
        dist.all_to_all_single(back[:n_send], d_recv, plan.send_splits, plan.recv_splits, group=self.group)
        out = ops.moe_combine(back, routing.dest_row, ids, w, t)
        return out.reshape(shape)


class SymmetricExpertParallelMoE(torch.nn.Module):
    """Expert-parallel W8A8 MoE whose dispatch and return run over NVLink peer memory, driven
    entirely from the device: no row count ever visits the host and the barrier epochs live in
    device memory, so a forward is a fixed sequence of stream-ordered launches (route -> barrier
    and plan -> pull -> expert stage -> push, which ends by signalling the peers -> combine, which begins by
    waiting for theirs; with ``overlap`` the pull, both GEMMs and the push run in two halves on two streams and a
    barrier launch closes the exchange) that can be captured in a CUDA graph and replayed (every rank must
    replay it the same number of times).

    Each rank keeps its routing plan, routed int8 rows, their scales and a result buffer in one
    symmetric allocation that every peer maps (``torch.distributed._symmetric_memory``).  Peers
    *pull* the rows their experts own and *push* the results back to the row's original position
    (``fuse_return=True`` lets the second expert GEMM's epilogue do those stores instead).
    ``max_tokens_per_rank`` fixes the buffer sizes; the expert-sorted buffers are sized for the
    worst case (every token of every rank routed to this rank).
    """

    def __init__(self, experts, num_experts: int, max_tokens_per_rank: int, top_k: int = 2, group=None,
                 fuse_return: bool = False, overlap: bool = False):
        super().__init__()
        import torch.distributed._symmetric_memory as symm
        # True: the expert GEMMs run in two halves of the row tiles and the exchange overlaps them on a second
        # stream -- the pull of the second half beside the first half's GEMM1, the push of the first half beside
        # the second half's GEMM2 (stream-level dependencies only, so the forward still captures into one graph).
        # Bit-identical; measured at 2 GPUs on the Mixtral-shaped layer it hides nothing (1.186 vs 1.176 ms): the
        # GEMMs run against the power cap, so a copy kernel beside them costs them the clocks it saves in time,
        # and each GEMM pays a second launch and tail.  Hence off by default.
        self.overlap = bool(overlap) and not fuse_return
        # True: the second GEMM's epilogue stores results at home instead of a push kernel.  Measured on the
        # Mixtral-shaped layer: equal at 2 GPUs, 11 % slower at 8 (0.418 vs 0.375 ms) -- the row-per-thread
        # 64-byte peer stores hold the epilogue warps -- so the separate push kernel stays the default.
        self.fuse_return = bool(fuse_return)
        from . import _lib
        self.experts = experts
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.num_experts = int(num_experts)
        self.e_loc = self.num_experts // self.world
        self.top_k = int(top_k)
        if tuple(experts.expert_range) != expert_partition(self.num_experts, self.world)[self.rank]:
            raise ValueError("experts.expert_range does not match this rank's partition")
        lib = _lib.load()
        dev = experts.gate_up_proj.device
        self.hidden = experts.hidden_dim
        self.inter = experts.intermediate_dim
        self.max_tokens = int(max_tokens_per_rank)
        entries = self.max_tokens * self.top_k
        self.r_cap = lib.mp_moe_padded_rows(self.num_experts, entries)            # rows of this rank's routed buffers
        self.sorted_cap = lib.mp_moe_padded_rows(self.e_loc, self.world * entries)  # rows of the expert-sorted buffers
        plan_ints = lib.mp_moe_plan_ints(self.num_experts, entries)
        al = lambda n: (n + 255) // 256 * 256
        self.off_flags = 0
        self.off_plan = 256
        self.off_scale = self.off_plan + al(plan_ints * 4)
        self.off_q = self.off_scale + al(self.r_cap * 4)
        self.off_back = self.off_q + al(self.r_cap * self.hidden)
        total = self.off_back + al(self.r_cap * self.hidden * 2)
        self.buf = symm.empty(total, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize(dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)                                                   # every rank zeroed its flags
        bases = [int(p) for p in self.handle.buffer_ptrs]

        def ptrs(off):
            import ctypes
            return (ctypes.c_void_p * self.world)(*[b + off for b in bases])

        self.p_flags, self.p_plan = ptrs(self.off_flags), ptrs(self.off_plan)
        self.p_scale, self.p_q, self.p_back = ptrs(self.off_scale), ptrs(self.off_q), ptrs(self.off_back)
        v = self.buf
        self.plan = v[self.off_plan:self.off_plan + plan_ints * 4].view(torch.int32)
        self.routed_scale = v[self.off_scale:self.off_scale + self.r_cap * 4].view(torch.float32)
        self.routed_q = v[self.off_q:self.off_q + self.r_cap * self.hidden].view(torch.int8).view(self.r_cap, self.hidden)
        self.back = v[self.off_back:self.off_back + self.r_cap * self.hidden * 2].view(torch.float16).view(
            self.r_cap, self.hidden)
        self.xplan = torch.zeros(lib.mp_moe_ep_plan_ints(self.world, self.e_loc, self.sorted_cap), dtype=torch.int32,
                                 device=dev)
        self.q_sorted = torch.empty((self.sorted_cap, self.hidden), dtype=torch.int8, device=dev)
        self.s_sorted = torch.empty(self.sorted_cap, dtype=torch.float32, device=dev)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)     # advanced by the barrier kernel itself
        self.push_blocks = torch.zeros(1, dtype=torch.int32, device=dev)   # block counter of the signalling push
        self.arrivals = v[self.off_flags:self.off_flags + 4 * self.world].view(torch.int32)   # peers' words, here
        if self.overlap:
            # buffers that two streams touch are owned by the module, not taken from the caching allocator per call
            self.side = torch.cuda.Stream(device=dev)
            self.stage_bytes = int(lib.mp_moe_expert_stage_workspace_bytes(self.sorted_cap, self.inter))
            self.stage_ws = torch.empty(self.stage_bytes, dtype=torch.uint8, device=dev)
            self.d_sorted = torch.empty((self.sorted_cap, self.hidden), dtype=torch.float16, device=dev)

    def _expert_stage_overlapped(self, h: int):
        """pull | GEMM1 | requant | GEMM2 | push with each GEMM in two halves of the row tiles; the second half's
        pull and the first half's push run on ``self.side`` next to the other half's GEMM.  Only events order the
        two streams, so the sequence captures into a CUDA graph as a fork and a join."""
        from . import _lib, ops
        lib = _lib.load()
        ex = self.experts
        main = torch.cuda.current_stream()
        side = self.side
        err = ops._error_word(self.buf.device).data_ptr()
        xp, ws, nb = self.xplan.data_ptr(), self.stage_ws.data_ptr(), self.stage_bytes

        def pull(part, stream):
            _lib.check(lib.mp_moe_ep_pull_part(self.p_q, self.p_scale, xp, self.world, self.e_loc, self.sorted_cap, h,
                                               self.q_sorted.data_ptr(), self.s_sorted.data_ptr(), part,
                                               stream.cuda_stream), "moe_ep_pull")

        def push(part, stream):
            _lib.check(lib.mp_moe_ep_push_part(self.d_sorted.data_ptr(), xp, self.world, self.e_loc, self.sorted_cap, h,
                                               self.p_back, part, stream.cuda_stream), "moe_ep_push")

        def gemm1(part):
            _lib.check(lib.mp_moe_gemm1_swiglu(self.q_sorted.data_ptr(), self.s_sorted.data_ptr(), xp, self.sorted_cap, h,
                                               self.inter, self.e_loc, ex.gate_up_proj.data_ptr(),
                                               ex.gate_up_proj_scale.data_ptr(), ws, nb, part, err, main.cuda_stream),
                       "moe_gemm1_swiglu")

        def gemm2(part):
            _lib.check(lib.mp_moe_gemm2(xp, self.sorted_cap, self.inter, h, self.e_loc, ex.down_proj.data_ptr(),
                                        ex.down_proj_scale.data_ptr(), self.d_sorted.data_ptr(), ws, nb, part, err,
                                        main.cuda_stream), "moe_gemm2")

        planned = torch.cuda.Event()
        planned.record(main)
        side.wait_event(planned)                           # fork: the plan is in place
        pull(0, main)
        pull(1, side)
        pulled = torch.cuda.Event()
        pulled.record(side)
        gemm1(0)
        main.wait_event(pulled)
        gemm1(1)
        _lib.check(lib.mp_moe_requant(xp, self.sorted_cap, self.inter, self.e_loc, ws, nb, main.cuda_stream), "moe_requant")
        gemm2(0)
        half_done = torch.cuda.Event()
        half_done.record(main)
        side.wait_event(half_done)
        push(0, side)
        pushed = torch.cuda.Event()
        pushed.record(side)
        gemm2(1)
        push(1, main)
        main.wait_event(pushed)                            # join

    def _barrier(self):
        from . import _lib, ops
        st = _lib.load().mp_peer_barrier_counted(self.p_flags, self.world, self.rank, self.epoch.data_ptr(),
                                                 ops._error_word(self.buf.device).data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream)
        _lib.check(st, "peer_barrier", world=self.world, rank=self.rank)

    @torch.no_grad()
    def forward(self, hidden_states, top_k_index, top_k_weights):
        from . import _lib, ops
        lib = _lib.load()
        shape = hidden_states.shape
        hs = hidden_states.reshape(-1, shape[-1]).contiguous()
        t, h = hs.shape
        if t > self.max_tokens or h != self.hidden:
            raise ValueError(f"{t} tokens x {h} exceed the buffers sized at construction "
                             f"({self.max_tokens} x {self.hidden})")
        ids = top_k_index.reshape(t, -1).to(torch.int32).contiguous()
        w = top_k_weights.reshape(t, -1).to(torch.float16).contiguous()
        stream = torch.cuda.current_stream().cuda_stream
        routing = ops.moe_route_gather_quant(hs, ids, 0, self.num_experts,
                                             out=(self.plan, self.routed_q, self.routed_scale))
        # barrier (every rank's routed rows and plan are in place), then this rank's layout from the peers' counts
        _lib.check(lib.mp_moe_ep_barrier_plan(self.p_flags, self.p_plan, self.world, self.rank, self.epoch.data_ptr(),
                                              self.num_experts, self.sorted_cap, self.xplan.data_ptr(),
                                              ops._error_word(self.buf.device).data_ptr(), stream),
                   "moe_ep_barrier_plan")
        ex = self.experts
        if self.overlap:
            self._expert_stage_overlapped(h)
            self._barrier()                                # every result row has landed at home
            out = ops.moe_combine(self.back, routing.dest_row, ids, w, t)
            return out.reshape(shape)
        _lib.check(lib.mp_moe_ep_pull(self.p_q, self.p_scale, self.xplan.data_ptr(), self.world, self.e_loc,
                                      self.sorted_cap, h, self.q_sorted.data_ptr(), self.s_sorted.data_ptr(), stream),
                   "moe_ep_pull")
        if self.fuse_return:
            # both grouped GEMMs; the second one's epilogue stores each result row at its original position in
            # the source rank's buffer (peer stores over NVLink): the return path costs no kernel of its own
            nbytes = lib.mp_moe_expert_stage_workspace_bytes(self.sorted_cap, self.inter)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=hs.device)
            _lib.check(lib.mp_moe_expert_stage_scatter(
                self.q_sorted.data_ptr(), self.s_sorted.data_ptr(), self.xplan.data_ptr(), self.sorted_cap, h,
                self.inter, self.e_loc, self.world, ex.gate_up_proj.data_ptr(), ex.gate_up_proj_scale.data_ptr(),
                ex.down_proj.data_ptr(), ex.down_proj_scale.data_ptr(), self.p_back, ws.data_ptr(), nbytes,
                ops._error_word(hs.device).data_ptr(), stream), "moe_expert_stage_scatter")
        else:
            d_sorted = ops.moe_expert_stage(self.q_sorted, self.s_sorted, self.xplan, self.e_loc, ex.gate_up_proj,
                                            ex.gate_up_proj_scale, ex.down_proj, ex.down_proj_scale)
            # the push ends by raising this rank's arrival word on every peer; the combine's blocks wait for the
            # peers' words: the closing barrier without a launch of its own
            _lib.check(lib.mp_moe_ep_push_signal(d_sorted.data_ptr(), self.xplan.data_ptr(), self.world, self.e_loc,
                                                 self.sorted_cap, h, self.p_back, self.p_flags, self.rank,
                                                 self.epoch.data_ptr(), self.push_blocks.data_ptr(), stream),
                       "moe_ep_push_signal")
            out = torch.empty((t, h), dtype=torch.float16, device=hs.device)
            if t:
                _lib.check(lib.mp_moe_combine_after_peers(
                    self.arrivals.data_ptr(), self.world, self.epoch.data_ptr(), self.back.data_ptr(),
                    routing.dest_row.data_ptr(), ids.data_ptr(), w.data_ptr(), t, h, ids.shape[1], out.data_ptr(),
                    ops._error_word(hs.device).data_ptr(), stream), "moe_combine_after_peers")
            return out.reshape(shape)
        self._barrier()                                    # every result row has landed at home
        out = ops.moe_combine(self.back, routing.dest_row, ids, w, t)
        return out.reshape(shape)
