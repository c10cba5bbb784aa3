"""GPU parity of the W8A8 MoE expert path against the CPU oracle (through the C ABI).

Bit-exact: router indices, routed int8 rows and their scales, routing plan.
fp16 outputs: relative Frobenius error <= 1e-2 against the reference's
``SmoothQuantPackedMoeExperts.forward`` (golden fixture / oracle).
"""
import numpy as np
import pytest
import torch

from mindpipe_b200 import synth
from oracle import pseudo_quant as O

pytestmark = pytest.mark.gpu
TOL = 1e-2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_router_matches_reference(golden):
    from mindpipe_b200 import ops
    g = golden("moe_small.npz")
    idx, w = ops.moe_router_topk(dev(g["logits"]), 2)
    assert np.array_equal(idx.cpu().numpy(), g["top_k_index"].astype(np.int32))
    assert np.allclose(w.float().cpu().numpy(), g["top_k_weights"].astype(np.float32), atol=1e-3)
    lg = synth.router_logits(8192, 8, seed=0).numpy()            # config 4 router input
    idx, w = ops.moe_router_topk(dev(lg), 2)
    oi, ow = O.router_top2(lg, 2)
    assert np.array_equal(idx.cpu().numpy(), oi.astype(np.int32))
    assert np.allclose(w.float().cpu().numpy(), ow.astype(np.float32), atol=1e-3)


@pytest.mark.parametrize("h", [256, 4096, 4608])          # rows kept in registers (<= 4096 values) or read twice
@pytest.mark.parametrize("lo,hi", [(0, 8), (2, 5), (7, 8)])
def test_route_gather_quant_bit_exact(lo, hi, h):
    from mindpipe_b200 import ops
    t, e, k = 777, 8, 2
    hs = synth.outlier_activation(t, h, seed=3).numpy()
    ids, _ = O.router_top2(synth.router_logits(t, e, seed=3).numpy(), k)
    ids = ids.astype(np.int32)
    r = ops.moe_route_gather_quant(dev(hs), dev(ids), lo, hi)
    torch.cuda.synchronize()
    counts = r.counts.cpu().numpy()
    seg = r.segment_offsets.cpu().numpy()
    dest = r.dest_row.cpu().numpy().reshape(t, k)
    assert np.array_equal(counts, np.bincount(ids.ravel(), minlength=e)[lo:hi])
    assert (seg % 256 == 0).all() and seg[0] == 0                   # segments are 256-row aligned
    assert np.array_equal(np.diff(seg), (counts + 255) // 256 * 256)
    _, codes, sc = O.absmax_quant_last_dim(hs)
    rq, rs = r.routed_q.cpu().numpy(), r.routed_scale.cpu().numpy()
    local = (ids >= lo) & (ids < hi)
    assert (dest[~local] == -1).all()
    rows = dest[local]
    assert len(np.unique(rows)) == rows.size                       # a permutation: no row claimed twice
    ex = ids[local] - lo
    assert ((rows >= seg[ex]) & (rows < seg[ex] + counts[ex])).all()
    tok = np.nonzero(local)[0]
    assert np.array_equal(rq[rows], codes[tok])                     # int8 activations bit-exact
    assert np.array_equal(rs[rows], sc[tok, 0].astype(np.float32))
    pad = np.ones(r.padded_rows, dtype=bool)
    pad[rows] = False
    assert (rs[pad] == 0).all()                                     # padding rows are neutralised


def _module_case(e, h, i, t, seed, expert_range=None):
    from mindpipe_b200 import ops
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts
    shape = synth.MoeShape(num_experts=e, hidden=h, ffn=i, top_k=2, tokens=t)
    gu, dn = synth.moe_weights(shape, seed=seed, std=0.05)
    hs = synth.normal_activation(t, h, seed=seed, index=11)
    idx, w = ops.moe_router_topk(synth.router_logits(t, e, seed=seed).cuda(), 2)
    lo, hi = (0, e) if expert_range is None else expert_range
    mod = SmoothQuantPackedMoeExperts(gu[lo:hi].cuda(), dn[lo:hi].cuda(), torch.nn.SiLU(),
                                      expert_range=(lo, hi), num_experts=e)
    out = mod(hs.cuda(), idx, w)
    ops.check_device_errors()
    return gu.numpy(), dn.numpy(), hs.numpy(), idx.cpu().numpy(), w.cpu().numpy(), out.cpu().numpy()


def test_moe_module_matches_reference_golden(golden):
    from mindpipe_b200 import ops
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts
    g = golden("moe_small.npz")
    src = type("Src", (), {})()
    src.gate_up_proj, src.down_proj, src.act_fn = dev(g["gate_up"]), dev(g["down"]), torch.nn.SiLU()
    mod = SmoothQuantPackedMoeExperts.from_float(src)
    assert np.array_equal(mod.gate_up_proj.cpu().numpy(), O.absmax_quant_last_dim(g["gate_up"])[1])
    out = mod(dev(g["hidden"]), dev(g["top_k_index"]), dev(g["top_k_weights"]))
    ops.check_device_errors()
    assert O.rel_frobenius(out.cpu().numpy(), g["out"]) <= TOL      # expert 3 is never hit in this fixture


@pytest.mark.parametrize("e,h,i,t", [(8, 512, 1024, 512), (4, 256, 384, 1000), (8, 128, 256, 3)])
def test_moe_module_vs_oracle(e, h, i, t):
    gu, dn, hs, idx, w, out = _module_case(e, h, i, t, seed=e + t)
    guf, _, _ = O.absmax_quant_last_dim(gu)
    dnf, _, _ = O.absmax_quant_last_dim(dn)
    ref = O.moe_experts_forward(hs, idx.astype(np.int64), w, guf, dnf)
    assert O.rel_frobenius(out, ref) <= TOL


def test_moe_expert_ranges_sum_to_full_output():
    """Expert parallelism: the outputs of disjoint expert ranges add up (in fp16) to the full output."""
    full = _module_case(8, 256, 512, 600, seed=9)[-1]
    parts = [_module_case(8, 256, 512, 600, seed=9, expert_range=r)[-1] for r in ((0, 4), (4, 8))]
    assert np.array_equal((parts[0] + parts[1]).astype(np.float16), full)
    quarters = [_module_case(8, 256, 512, 600, seed=9, expert_range=(j, j + 2))[-1] for j in (0, 2, 4, 6)]
    acc = np.zeros_like(full, dtype=np.float32)
    for q in quarters:                                               # each token has two non-zero addends
        acc += q.astype(np.float32)
    assert np.array_equal(acc.astype(np.float16), full)


def test_moe_layer_under_programmatic_dependent_launch_same_bits():
    """Every launch of the layer may be scheduled before its predecessor has finished (each kernel waits for it on
    the device): same bits as the serialised sequence, eagerly and as a replayed CUDA graph."""
    from mindpipe_b200 import _lib, ops
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts
    shape = synth.MoeShape(num_experts=8, hidden=512, ffn=1024, top_k=2, tokens=700)
    gu, dn = synth.moe_weights(shape, seed=21, std=0.05)
    hs = synth.normal_activation(shape.tokens, shape.hidden, seed=21, index=11).cuda()
    idx, w = ops.moe_router_topk(synth.router_logits(shape.tokens, 8, seed=21).cuda(), 2)
    mod = SmoothQuantPackedMoeExperts(gu.cuda(), dn.cuda(), torch.nn.SiLU())
    base = mod(hs, idx, w)
    lib = _lib.load()
    before = lib.mp_set_programmatic_launch(1)
    try:
        for _ in range(3):
            assert torch.equal(mod(hs, idx, w), base)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            mod(hs, idx, w)                                   # allocations of the first call on this stream
            with torch.cuda.graph(graph, stream=side):
                out = mod(hs, idx, w)
            for _ in range(3):
                graph.replay()
        side.synchronize()
        assert torch.equal(out, base)
    finally:
        lib.mp_set_programmatic_launch(before)
    ops.check_device_errors()


@pytest.mark.parametrize("chained", [0, 1])
def test_expert_parallel_exchange_entries_with_this_gpu_as_its_only_peer(chained):
    """The device-driven exchange through the C ABI at world size 1 (the rank is its own peer, so one GPU is
    enough): route -> barrier + plan -> pull -> expert stage -> push that signals -> combine that waits, three
    forwards in a row (epochs advance, the push's block counter re-arms), against the module's forward."""
    import ctypes
    from mindpipe_b200 import _lib, ops
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts
    lib = _lib.load()
    e, h, inter, t, k = 4, 256, 512, 300, 2
    shape = synth.MoeShape(num_experts=e, hidden=h, ffn=inter, top_k=k, tokens=t)
    gu, dn = synth.moe_weights(shape, seed=31, std=0.05)
    mod = SmoothQuantPackedMoeExperts(gu.cuda(), dn.cuda(), torch.nn.SiLU())
    idx, w = ops.moe_router_topk(synth.router_logits(t, e, seed=31).cuda(), k)
    r_cap = lib.mp_moe_padded_rows(e, t * k)
    plan = torch.zeros(lib.mp_moe_plan_ints(e, t * k), dtype=torch.int32, device="cuda")
    routed_q = torch.empty((r_cap, h), dtype=torch.int8, device="cuda")
    routed_scale = torch.empty(r_cap, dtype=torch.float32, device="cuda")
    back = torch.zeros((r_cap, h), dtype=torch.float16, device="cuda")
    q_sorted = torch.empty((r_cap, h), dtype=torch.int8, device="cuda")
    s_sorted = torch.empty(r_cap, dtype=torch.float32, device="cuda")
    xplan = torch.zeros(lib.mp_moe_ep_plan_ints(1, e, r_cap), dtype=torch.int32, device="cuda")
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    blocks = torch.zeros(1, dtype=torch.int32, device="cuda")
    err = ops._error_word(torch.device("cuda", torch.cuda.current_device())).data_ptr()
    one = lambda tensor: (ctypes.c_void_p * 1)(tensor.data_ptr())
    before = lib.mp_set_programmatic_launch(chained)
    try:
        for call in range(3):
            hs = synth.normal_activation(t, h, seed=31, index=40 + call).cuda()
            want = mod(hs, idx, w)
            st = torch.cuda.current_stream().cuda_stream
            routing = ops.moe_route_gather_quant(hs, idx, 0, e, out=(plan, routed_q, routed_scale))
            _lib.check(lib.mp_moe_ep_barrier_plan(one(flags), one(plan), 1, 0, epoch.data_ptr(), e, r_cap,
                                                  xplan.data_ptr(), err, st), "barrier_plan")
            _lib.check(lib.mp_moe_ep_pull(one(routed_q), one(routed_scale), xplan.data_ptr(), 1, e, r_cap, h,
                                          q_sorted.data_ptr(), s_sorted.data_ptr(), st), "pull")
            d_sorted = ops.moe_expert_stage(q_sorted, s_sorted, xplan, e, mod.gate_up_proj, mod.gate_up_proj_scale,
                                            mod.down_proj, mod.down_proj_scale)
            _lib.check(lib.mp_moe_ep_push_signal(d_sorted.data_ptr(), xplan.data_ptr(), 1, e, r_cap, h, one(back),
                                                 one(flags), 0, epoch.data_ptr(), blocks.data_ptr(), st), "push")
            out = torch.empty((t, h), dtype=torch.float16, device="cuda")
            _lib.check(lib.mp_moe_combine_after_peers(flags.data_ptr(), 1, epoch.data_ptr(), back.data_ptr(),
                                                      routing.dest_row.data_ptr(), idx.data_ptr(), w.data_ptr(), t, h, k,
                                                      out.data_ptr(), err, st), "combine")
            torch.cuda.synchronize()
            assert torch.equal(out, want)
            assert epoch.item() == 2 * (call + 1) and flags[0].item() == 2 * (call + 1) and blocks.item() == 0
    finally:
        lib.mp_set_programmatic_launch(before)
    ops.check_device_errors()


def test_peer_barrier_wait_is_bounded_and_reports():
    """A peer that never shows up: the barrier's wait runs out (2 s), the kernel records an error
    word and returns, and the context stays usable.  The 'peer' is a second flag array on the same
    GPU that nothing ever signals."""
    import ctypes
    import time
    from mindpipe_b200 import _lib, ops
    lib = _lib.load()
    mine = torch.zeros(16, dtype=torch.int32, device="cuda")
    absent_peer = torch.zeros(16, dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(mine.data_ptr(), absent_peer.data_ptr())
    t0 = time.time()
    st = lib.mp_peer_barrier(ptrs, 2, 0, 1, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert err.item() == 4                          # "a peer did not arrive"
    assert 1.5 < waited < 10.0
    assert absent_peer[0].item() == 1               # our own arrival was published to the peer
    # a barrier whose peer has arrived passes at once, and ordinary work still runs afterwards
    err.zero_()
    mine[1] = 2
    st = lib.mp_peer_barrier(ptrs, 2, 0, 2, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == 0 and err.item() == 0
    q, s, _ = ops.act_quant_per_token(torch.ones(2, 64, dtype=torch.float16, device="cuda"))
    assert q.abs().max().item() == 127
