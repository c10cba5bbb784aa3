"""Multi-GPU parity check, run from inside a multi-rank job: expert-parallel MoE, column-parallel and
row-parallel W4A16 and row-parallel W8A8 against the single-GPU modules on small seeded shapes.

The reference verifies its fused tensor-parallel path the same way -- a script that runs inside the
multi-rank job and reports exactness (scripts/repro/verify_qwen25_vl_72b_tp4_fused_allreduce.py:44-184).
``verify_multi_gpu`` is called by ``bench.py`` on N > 1 ranks before it times anything (the flags end up
in its JSON line) and by ``tests/test_multi_gpu.py``.  Everything compared here comes out of this
library's kernels; a test may pass ``oracle`` (the CPU restatement of the reference) to also pin the
row-parallel W8A8 result to the reference arithmetic.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def _graph_replays(fn, out_of, dev, replays=3):
    """Run ``fn`` once on a side stream, capture it there, replay ``replays`` times; returns the captured call's
    output tensor."""
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()                                       # per-stream scratch is created outside the capture
        torch.cuda.synchronize(dev)
        with torch.cuda.graph(graph, stream=side):
            out = fn()
        for _ in range(replays):
            out_of(out).zero_()
            graph.replay()
    torch.cuda.synchronize(dev)
    return out


def verify_multi_gpu(rank: int, world: int, dev: torch.device, oracle=None) -> dict:
    """Returns ``{"ep": bool, "column": bool, "row_w4": bool, "row_w8": bool}`` for this rank; every rank
    of the default process group must call it (the checks contain collectives)."""
    from . import _lib, ops, synth
    from .column_parallel import ColumnParallelW4A16Linear
    from .expert_parallel import ExpertParallelMoE, SymmetricExpertParallelMoE, expert_partition
    from .modules import SmoothQuantPackedMoeExperts, VllmPackedInt4Linear
    from .row_parallel import RowParallelW4A16Linear, RowParallelW8A8Linear, shard_columns

    def same_on_all_ranks(t):
        everyone = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(everyone, t)
        return all(torch.equal(e, everyone[0]) for e in everyone)

    # ---- expert-parallel MoE vs the single-GPU module (same kernels on the same rows: identical bits) ----
    ok_ep = True
    if 8 % world == 0:
        shape = synth.MoeShape(num_experts=8, hidden=256, ffn=512, top_k=2, tokens=64 * world + 10)
        gu, dn = synth.moe_weights(shape, seed=1, std=0.05)
        hs = synth.normal_activation(shape.tokens, shape.hidden, seed=1, index=11).to(dev)
        idx, w = ops.moe_router_topk(synth.router_logits(shape.tokens, shape.num_experts, seed=1).to(dev), 2)
        full = SmoothQuantPackedMoeExperts(gu.to(dev), dn.to(dev), torch.nn.SiLU())
        ref = full(hs, idx, w)
        lo, hi = expert_partition(shape.num_experts, world)[rank]
        local = SmoothQuantPackedMoeExperts(gu[lo:hi].to(dev), dn[lo:hi].to(dev), torch.nn.SiLU(),
                                            expert_range=(lo, hi), num_experts=shape.num_experts)
        # tokens are data-sharded: uneven shards on purpose
        bounds = [0] + [shape.tokens * (r + 1) // world + (3 if r == 0 else 0) for r in range(world - 1)] + [shape.tokens]
        a, b = bounds[rank], bounds[rank + 1]
        xa, ia, wa = hs[a:b].contiguous(), idx[a:b].contiguous(), w[a:b].contiguous()
        out = ExpertParallelMoE(local, shape.num_experts)(xa, ia, wa)          # NCCL all-to-all fallback
        ops.check_device_errors()
        ok_ep = torch.equal(out, ref[a:b])
        for overlap in (False, True):            # serial launch sequence; halves of the GEMMs overlapped with the exchange
            sym = SymmetricExpertParallelMoE(local, shape.num_experts, max_tokens_per_rank=b - a + 7, overlap=overlap)
            for _ in range(3):                                                   # repeated forwards reuse the buffers
                out2 = sym(xa, ia, wa)
            ops.check_device_errors()
            ok_ep = ok_ep and torch.equal(out2, ref[a:b])
            out3 = _graph_replays(lambda: sym(xa, ia, wa), lambda o: o, dev)    # barrier epochs live on the device
            ops.check_device_errors()
            ok_ep = ok_ep and torch.equal(out3, ref[a:b])
        # the same launch sequence with every launch allowed to be scheduled before its predecessor has finished
        # (each kernel waits on the device): eager and as a replayed graph
        before = _lib.load().mp_set_programmatic_launch(1)
        try:
            chained = SymmetricExpertParallelMoE(local, shape.num_experts, max_tokens_per_rank=b - a + 7)
            for _ in range(3):
                out5 = chained(xa, ia, wa)
            ops.check_device_errors()
            ok_ep = ok_ep and torch.equal(out5, ref[a:b])
            out6 = _graph_replays(lambda: chained(xa, ia, wa), lambda o: o, dev)
            ops.check_device_errors()
            ok_ep = ok_ep and torch.equal(out6, ref[a:b])
        finally:
            _lib.load().mp_set_programmatic_launch(before)
        sym2 = SymmetricExpertParallelMoE(local, shape.num_experts, max_tokens_per_rank=b - a + 7, fuse_return=True)
        for _ in range(3):
            out4 = sym2(xa, ia, wa)
        ops.check_device_errors()
        ok_ep = ok_ep and torch.equal(out4, ref[a:b])

    # ---- column-parallel W4A16 vs single GPU: the same rows of the same kernel, gathered ----
    n, k = 1024, 2048
    wt = synth.normal_weight(n, k, seed=2).to(dev)
    packed, scale, zero, _ = ops.w4a16_quantize(wt, 128)
    single = VllmPackedInt4Linear(packed_weight=packed, scale=scale, bias=None, in_features=k, out_features=n,
                                  zero_point=zero)
    cp = ColumnParallelW4A16Linear.from_full(packed, scale, zero, None, k, device=dev, max_rows=64)
    ok_col = True
    for i, m in enumerate((8, 1, 64, 16, 3)):           # five calls: both gathered buffers are reused
        x = synth.normal_activation(m, k, seed=2, index=i).to(dev)
        want = single(x).float()
        got = cp(x)
        # the shard's launch may cut K differently from the unsharded one (fp32 summation order), so the
        # comparison with the single-GPU linear is by norm; the two exchanges move the same bits
        ok_col = ok_col and ((got.float() - want).norm() / want.norm()).item() <= 2e-3
        ok_col = ok_col and torch.equal(got, cp.forward_nccl(x)) and same_on_all_ranks(got)
        ops.check_device_errors()
    x = synth.normal_activation(16, k, seed=2, index=9).to(dev)
    y_eager = cp(x).clone()
    y_graph = _graph_replays(lambda: cp(x), lambda o: o, dev)
    ops.check_device_errors()
    ok_col = ok_col and torch.equal(y_graph, y_eager)

    # ---- row-parallel W4A16 (K sharded; one-shot and two-phase all-reduce of the partial sums) ----
    bias = (synth.normal_activation(1, n, seed=2, index=5)[0] * 0.1).to(torch.float16).to(dev)
    single_b = VllmPackedInt4Linear(packed_weight=packed, scale=scale, bias=bias, in_features=k, out_features=n,
                                    zero_point=zero)
    c0, c1 = shard_columns(k, world, rank, 128)
    ok_row = True
    for two_phase in (False, True):
        rp = RowParallelW4A16Linear.from_full(packed, scale, zero, bias, 128, device=dev, two_phase=two_phase)
        for i, m in enumerate((1, 8, 16, 5, 16)):       # five calls: both partial buffers are reused
            xm = synth.normal_activation(m, k, seed=3, index=i).to(dev)
            y = rp(xm[:, c0:c1].contiguous())
            ops.check_device_errors()
            want = single_b(xm).float()
            ok_row = ok_row and ((y.float() - want).norm() / want.norm()).item() <= 1e-2
            ok_row = ok_row and same_on_all_ranks(y)    # fixed-order sums: the same bits everywhere
            y2 = rp.forward_nccl(xm[:, c0:c1].contiguous())
            ok_row = ok_row and ((y2.float() - want).norm() / want.norm()).item() <= 1e-2
        x16 = synth.normal_activation(16, k, seed=3, index=99).to(dev)[:, c0:c1].contiguous()
        y_eager = rp(x16).clone()
        y_graph = _graph_replays(lambda: rp(x16), lambda o: o, dev)   # the call counter lives on the device
        ops.check_device_errors()
        ok_row = ok_row and torch.equal(y_graph, y_eager)

    # ---- row-parallel W8A8 (per-rank token scales, int32 accumulators summed over NVLink in rank order) ----
    n8, k8 = 512, 2048
    w8 = synth.normal_weight(n8, k8, seed=4)
    b8 = (synth.normal_activation(1, n8, seed=4, index=5)[0] * 0.1).to(torch.float16)
    k_lo, k_hi = rank * k8 // world, (rank + 1) * k8 // world
    full8 = torch.nn.Linear(k8, n8, bias=True).half().to(dev)
    full8.weight.data.copy_(w8)
    full8.bias.data.copy_(b8)
    rp8 = RowParallelW8A8Linear.from_float(full8, max_rows=300)      # full-row channel scales, column shard
    qw_all, sw_all, _ = ops.act_quant_per_token(full8.weight.detach().contiguous())
    ok_row8 = True
    for i, m8 in enumerate((1, 16, 300, 64)):
        x8 = synth.outlier_activation(m8, k8, seed=5, index=i)
        y8 = rp8(x8[:, k_lo:k_hi].to(dev).contiguous())
        ops.check_device_errors()
        # the single-GPU composition of the per-rank pieces, added in rank order with the kernel's operations
        want = torch.zeros((m8, n8), dtype=torch.float32, device=dev)
        for r in range(world):
            a, b = r * k8 // world, (r + 1) * k8 // world
            qx_r, sx_r, _ = ops.act_quant_per_token(x8[:, a:b].to(dev).contiguous())
            acc_r = ops.w8a8_gemm_i32(qx_r, qw_all[:, a:b].contiguous()).to(torch.float32)
            want = want + (acc_r * sx_r.reshape(-1, 1)) * sw_all.reshape(1, -1)
        want = (want + b8.to(dev).float()).to(torch.float16)
        exact = torch.equal(y8, want)
        if oracle is not None:                                        # the reference arithmetic, piece by piece
            _, qw_full, sw_full = oracle.absmax_quant_last_dim(w8.numpy())
            ref = np.zeros((m8, n8), np.float32)
            for r in range(world):
                a, b = r * k8 // world, (r + 1) * k8 // world
                _, qx_r, sx_r = oracle.absmax_quant_last_dim(x8[:, a:b].numpy())
                acc_r = oracle.int32_accumulate(qx_r, np.ascontiguousarray(qw_full[:, a:b])).astype(np.float32)
                ref = ref + (acc_r * sx_r.astype(np.float32).reshape(-1, 1)) * sw_full.astype(np.float32).reshape(1, -1)
            ref = (ref + b8.numpy().astype(np.float32)).astype(np.float16)
            exact = exact and np.array_equal(y8.cpu().numpy().view(np.uint16), ref.view(np.uint16))
        same = same_on_all_ranks(y8)
        # against the unquantised linear this is per-token int8 with x20 outlier channels: a sanity bound only
        dense = (x8.float() @ w8.float().T + b8.float()).to(dev)
        sane = ((y8.float() - dense).norm() / dense.norm()).item() <= 0.15
        y8n = rp8.forward_nccl(x8[:, k_lo:k_hi].to(dev).contiguous())
        close = ((y8n.float() - y8.float()).norm() / dense.norm()).item() <= 2e-3
        if not (exact and same and sane and close):
            print(f"rank {rank} row-parallel W8A8 m={m8}: exact={exact} same={same} sane={sane} close={close}", flush=True)
        ok_row8 = ok_row8 and exact and same and sane and close
    # a captured graph with ONE forward in it, replayed an odd number of times and followed by eager calls:
    # the receive slots must keep alternating (their parity is the device-side call number's)
    x8 = synth.outlier_activation(16, k8, seed=5, index=50)[:, k_lo:k_hi].to(dev).contiguous()
    y_eager = rp8(x8).clone()
    y_graph = _graph_replays(lambda: rp8(x8), lambda o: o, dev, replays=3)
    ops.check_device_errors()
    ok_row8 = ok_row8 and torch.equal(y_graph, y_eager) and torch.equal(rp8(x8), y_eager)
    return {"ep": bool(ok_ep), "column": bool(ok_col), "row_w4": bool(ok_row), "row_w8": bool(ok_row8)}


def all_ranks_agree(flags: dict, dev: torch.device) -> dict:
    """Logical AND of every rank's flags (one all-reduce)."""
    keys = sorted(flags)
    t = torch.tensor([1 if flags[k] else 0 for k in keys], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return {k: bool(v) for k, v in zip(keys, t.tolist())}
