"""Host-side logic of the multi-GPU paths, on CPU: pure layout arithmetic plus
world_size-2 ``gloo`` runs of the dispatch / return exchange and the column gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mindpipe_b200.column_parallel import assemble_gathered, shard_packed_linear, shard_rows
from mindpipe_b200.expert_parallel import SEGMENT_ALIGN, TILE, expert_partition, plan_exchange
from mindpipe_b200.row_parallel import pack_nibbles, shard_columns, shard_packed_linear_columns, unpack_nibbles


def test_expert_partition_is_disjoint_and_complete():
    for e, p in [(8, 1), (8, 2), (8, 4), (8, 8), (64, 8)]:
        ranges = expert_partition(e, p)
        owned = [x for lo, hi in ranges for x in range(lo, hi)]
        assert owned == list(range(e))                      # every expert on exactly one rank, none extra
    with pytest.raises(ValueError):
        expert_partition(8, 3)


def test_plan_exchange_layout():
    rng = np.random.default_rng(0)
    world, e_loc = 4, 2
    send = rng.integers(0, 300, size=(world, e_loc))
    recv = rng.integers(0, 300, size=(world, e_loc))
    recv[2] = 0                                             # a peer that sends nothing
    recv[:, 1][recv[:, 1] > 250] = 0
    pl = plan_exchange(send, recv)
    pad = lambda a: (a + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
    assert pl.send_splits == list(pad(send).sum(axis=1))
    assert pl.recv_splits == list(pad(recv).sum(axis=1))
    assert pl.recv_rows == sum(pl.recv_splits)
    per_expert = recv.sum(axis=0)
    assert pl.padded_rows == max(int(pad(per_expert).sum()), SEGMENT_ALIGN)
    # the gather map is a bijection between real received rows and real sorted rows
    real_sorted = np.nonzero(pl.gather_map >= 0)[0]
    assert real_sorted.size == per_expert.sum()
    assert np.array_equal(pl.scatter_map[pl.gather_map[real_sorted]], real_sorted)
    assert (pl.scatter_map >= 0).sum() == per_expert.sum()
    # plan ints: counts | cursors | offsets | tile count | tile experts
    assert np.array_equal(pl.plan_ints[:e_loc], per_expert)
    seg = pl.plan_ints[2 * e_loc:3 * e_loc + 1]
    assert seg[0] == 0 and np.array_equal(np.diff(seg), pad(per_expert))
    n_tiles = pl.plan_ints[3 * e_loc + 1]
    assert n_tiles == pad(per_expert).sum() // TILE
    tiles = pl.plan_ints[3 * e_loc + 2:3 * e_loc + 2 + n_tiles]
    assert np.array_equal(np.bincount(tiles, minlength=e_loc), pad(per_expert) // TILE)
    # rows of expert e in sorted order come from sources in ascending rank order
    for e in range(e_loc):
        rows = pl.gather_map[seg[e]:seg[e] + per_expert[e]]
        assert (np.diff(rows) > 0).all()


def test_plan_exchange_no_rows():
    pl = plan_exchange(np.zeros((2, 1), int), np.zeros((2, 1), int))
    assert pl.recv_rows == 0 and pl.padded_rows == SEGMENT_ALIGN and pl.plan_ints[3 * 1 + 1] == 0
    assert (pl.gather_map == -1).all()


def test_column_shards_and_assembly():
    n, k8 = 64, 16
    packed = torch.arange(n * k8, dtype=torch.int32).reshape(n, k8)
    scale = torch.rand(n, 4).half()
    parts = [shard_packed_linear(packed, scale, None, None, 4, r) for r in range(4)]
    assert torch.equal(torch.cat([p[0] for p in parts]), packed)
    assert shard_rows(28672, 8, 7) == (25088, 28672)
    with pytest.raises(ValueError):
        shard_rows(10, 4, 0)
    y = torch.randn(5, 64)
    gathered = torch.stack([y[:, r * 16:(r + 1) * 16] for r in range(4)])
    assert torch.equal(assemble_gathered(gathered), y)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(rank)
        e, k, t, h = 4, 2, 37 + 5 * rank, 8
        e_loc = e // world
        ids = torch.stack([torch.randperm(e)[:k] for _ in range(t)]).to(torch.int32)
        hidden = torch.randn(t, h)
        # CPU stand-in for the router kernel: sort entries by expert into 256-padded segments
        counts = torch.bincount(ids.flatten().long(), minlength=e)
        pad = (counts + SEGMENT_ALIGN - 1) // SEGMENT_ALIGN * SEGMENT_ALIGN
        seg = torch.cat([torch.zeros(1, dtype=torch.long), pad.cumsum(0)])
        dest = torch.empty(t * k, dtype=torch.long)
        cursor = seg[:-1].clone()
        for i, ex in enumerate(ids.flatten().tolist()):
            dest[i] = cursor[ex]
            cursor[ex] += 1
        routed = torch.zeros(int(seg[-1]), h)
        routed[dest] = hidden.repeat_interleave(k, dim=0)
        send_counts = counts.reshape(world, e_loc).to(torch.int32)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        pl = plan_exchange(send_counts.numpy(), recv_counts.numpy())
        recv = torch.empty(pl.recv_rows, h)
        dist.all_to_all_single(recv, routed[:sum(pl.send_splits)], pl.recv_splits, pl.send_splits)
        gmap = torch.from_numpy(pl.gather_map).long()
        sorted_rows = torch.zeros(pl.padded_rows, h)
        sorted_rows[gmap >= 0] = recv[gmap[gmap >= 0]]
        # fake expert stage: expert e scales its rows by (global expert id + 1)
        seg_loc = pl.plan_ints[2 * e_loc:3 * e_loc + 1]
        out_sorted = torch.zeros_like(sorted_rows)
        for le in range(e_loc):
            cnt = int(pl.plan_ints[le])
            out_sorted[seg_loc[le]:seg_loc[le] + cnt] = sorted_rows[seg_loc[le]:seg_loc[le] + cnt] * (rank * e_loc + le + 1)
        smap = torch.from_numpy(pl.scatter_map).long()
        d_recv = torch.zeros(pl.recv_rows, h)
        d_recv[smap >= 0] = out_sorted[smap[smap >= 0]]
        back = torch.zeros(int(seg[-1]), h)
        dist.all_to_all_single(back[:sum(pl.send_splits)], d_recv, pl.send_splits, pl.recv_splits)
        got = back[dest].reshape(t, k, h).sum(dim=1)
        want = (hidden[:, None, :] * (ids[:, :, None].float() + 1)).sum(dim=1)
        ret[rank] = bool(torch.allclose(got, want, atol=1e-5))
        # column-parallel gather with a fake local linear
        y_full = torch.arange(3 * 8, dtype=torch.float32).reshape(3, 8)
        lo, hi = shard_rows(8, world, rank)
        gathered = torch.empty(world * 3, hi - lo)
        dist.all_gather_into_tensor(gathered, y_full[:, lo:hi].contiguous())
        ret[rank] = ret[rank] and bool(torch.equal(assemble_gathered(gathered.view(world, 3, hi - lo)), y_full))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_world2_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ep_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_parallel_column_shards(world):
    """K-sharding of the packed format: every shard dequantises to its column slice of the full Wdq
    (zero points are re-packed because a shard's first group need not start a packed word: 28 groups
    over 8 ranks gives 3.5 words per rank), and the shards' partial products add up to the full one."""
    from oracle import pseudo_quant as O
    from mindpipe_b200 import synth
    n, k, g = 24, 3584 * 2, 128                      # 56 groups: 7 per rank at world 8
    w = synth.normal_weight(n, k, seed=11, index=0).numpy()
    wdq, scales, zeros, codes = O.w4_group_asym_quantize(w, g)
    packed = torch.from_numpy(O.pack_int4_unsigned(codes))
    zp = torch.from_numpy(O.pack_int4_unsigned(zeros.astype(np.uint8)))
    assert np.array_equal(pack_nibbles(unpack_nibbles(zp, k // g)).numpy(), zp.numpy())
    x = synth.normal_activation(3, k, seed=11, index=1).numpy().astype(np.float32)
    total = np.zeros((3, n), np.float32)
    for rank in range(world):
        lo, hi = shard_columns(k, world, rank, g)
        p, s_, z = shard_packed_linear_columns(packed, torch.from_numpy(scales), zp, world, rank, g)
        part = O.w4_dequant(p.numpy(), s_.numpy(), z.numpy(), n, hi - lo, g)
        assert np.array_equal(part.view(np.uint16), wdq[:, lo:hi].view(np.uint16))
        total += x[:, lo:hi] @ part.astype(np.float32).T
    full = x @ wdq.astype(np.float32).T
    assert np.abs(total - full).max() <= 1e-3 * np.abs(full).max()
    with pytest.raises(ValueError):
        shard_columns(k, 3, 0, g)
    with pytest.raises(ValueError):
        shard_columns(1024, 8, 0, 256)                # 128 columns per rank is not a whole group of 256


def test_expert_parallel_constructor_rejects_wrong_partition():
    """Host-side failure injection: a rank holding the wrong experts is refused before any launch."""
    import types
    from mindpipe_b200 import expert_parallel as ep

    class FakeExperts:
        expert_range = (0, 3)

    fake_dist = types.SimpleNamespace(get_world_size=lambda g=None: 2, get_rank=lambda g=None: 1)
    real = ep.dist
    ep.dist = fake_dist
    try:
        with pytest.raises(ValueError, match="must hold experts"):
            ep.ExpertParallelMoE(FakeExperts(), 8)
    finally:
        ep.dist = real


# ---- wire layout of the flag-in-data collectives (csrc/peer_collectives.cu), replayed rank by rank in numpy ----
def _ll_pack(words, epoch):
    """uint32 words -> the wire form: every word followed by the call number."""
    out = np.empty(words.size * 2, dtype=np.uint32)
    out[0::2] = words.ravel()
    out[1::2] = epoch
    return out


@pytest.mark.parametrize("world,m,n", [(2, 1, 64), (4, 5, 256), (8, 16, 512)])
def test_row_parallel_two_phase_wire_layout(world, m, n):
    """rowparallel_finish_ll_kernel's offsets: step 1 sends the fp32 sums of the columns rank q owns to
    recv1[q][sender][m][n_loc] (8 bytes per sum), step 2 adds the P contributions in rank order and sends fp16
    pairs to recv2[q][m][N] (8 bytes per pair), step 3 reads the other ranks' columns.  Every wire word must be
    written exactly once and every rank must end with the rank-ordered sum."""
    rng = np.random.default_rng(world * 100 + m)
    epoch = 7
    partial = rng.standard_normal((world, m, n)).astype(np.float32)
    n_loc = n // world
    recv1 = np.zeros((world, world * m * n_loc * 2), dtype=np.uint32)        # per receiving rank, in 4-byte words
    recv2 = np.zeros((world, m * n), dtype=np.uint32)                         # 4 wire bytes per fp16 element
    for rank in range(world):                                                 # step 1 on every rank
        for mm in range(m):
            for nn in range(0, n, 4):
                q = nn // n_loc
                if q == rank:
                    continue
                off = ((rank * m + mm) * n_loc + (nn - q * n_loc)) * 8 // 4
                wire = _ll_pack(partial[rank, mm, nn:nn + 4].view(np.uint32), epoch)
                assert not recv1[q, off:off + 8].any()
                recv1[q, off:off + 8] = wire
    y = np.zeros((world, m, n), dtype=np.float16)
    for rank in range(world):                                                 # step 2
        for mm in range(m):
            for nl in range(0, n_loc, 4):
                nn = rank * n_loc + nl
                acc = np.zeros(4, dtype=np.float32)
                for r in range(world):
                    if r == rank:
                        v = partial[rank, mm, nn:nn + 4]
                    else:
                        off = ((r * m + mm) * n_loc + nl) * 8 // 4
                        w = recv1[rank, off:off + 8]
                        assert (w[1::2] == epoch).all()
                        v = w[0::2].view(np.float32)
                    acc = acc + v
                h = acc.astype(np.float16)
                y[rank, mm, nn:nn + 4] = h
                pairs = h.view(np.uint32)                                     # two fp16 per word
                for q in range(world):
                    if q != rank:
                        off = (mm * n + nn) * 4 // 4
                        assert not recv2[q, off:off + 4].any()
                        recv2[q, off:off + 4] = _ll_pack(pairs, epoch)
    for rank in range(world):                                                 # step 3
        for mm in range(m):
            for nn in range(0, n, 4):
                if nn // n_loc == rank:
                    continue
                w = recv2[rank, (mm * n + nn):(mm * n + nn) + 4]
                assert (w[1::2] == epoch).all()
                y[rank, mm, nn:nn + 4] = np.ascontiguousarray(w[0::2]).view(np.float16)
    want = np.zeros((m, n), dtype=np.float32)
    for r in range(world):
        want = want + partial[r]
    for rank in range(world):
        assert np.array_equal(y[rank].view(np.uint16), want.astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("world,rows,slice_bytes", [(2, 1, 32), (4, 3, 64), (8, 16, 128)])
def test_all_gather_wire_layout(world, rows, slice_bytes):
    """peer_allgather_push_kernel's offsets: rank r's 16-byte chunk j of row m lands at wire byte
    ((m * world + r) * chunks_per_row + j) * 32 of every peer's receive buffer."""
    rng = np.random.default_rng(world)
    cpr = slice_bytes // 16
    src = rng.integers(0, 2 ** 32, size=(world, rows, slice_bytes // 4), dtype=np.uint64).astype(np.uint32)
    recv = np.zeros((world, rows * world * slice_bytes * 2 // 4), dtype=np.uint32)
    epoch = 3
    for rank in range(world):
        for mm in range(rows):
            for j in range(cpr):
                off = ((mm * world + rank) * cpr + j) * 32 // 4
                for q in range(world):
                    if q != rank:
                        assert not recv[q, off:off + 8].any()
                        recv[q, off:off + 8] = _ll_pack(src[rank, mm, 4 * j:4 * j + 4], epoch)
    for rank in range(world):
        out = np.zeros((rows, world, slice_bytes // 4), dtype=np.uint32)
        out[:, rank] = src[rank]
        for mm in range(rows):
            for r in range(world):
                if r == rank:
                    continue
                for j in range(cpr):
                    off = ((mm * world + r) * cpr + j) * 32 // 4
                    w = recv[rank, off:off + 8]
                    assert (w[1::2] == epoch).all()
                    out[mm, r, 4 * j:4 * j + 4] = w[0::2]
        assert np.array_equal(out, np.transpose(src, (1, 0, 2)))


# ---- the expert-parallel layer's epoch protocol, replayed on the CPU under random interleavings ----
def _ep_rank_program(r, world, layers, flags, epoch, q_version, back_version, log):
    """One rank of SymmetricExpertParallelMoE.forward as a generator: every ``yield`` is a point where another
    rank may run; ``yield cond`` (a callable) blocks until the condition holds.  Buffers are modelled by version
    numbers: q_version[r] = layer whose routed rows rank r's buffer holds, back_version[r][p] = layer whose result
    rows rank p has stored into rank r's result buffer."""
    for layer in range(1, layers + 1):
        # route: overwrite this rank's routed buffer (peers must be done pulling the previous layer's rows)
        q_version[r] = ("writing", layer)
        yield None
        q_version[r] = layer
        yield None
        # barrier + plan (mp_moe_ep_barrier_plan): advance the epoch, raise the word on every peer, wait for theirs
        epoch[r] += 1
        e = epoch[r]
        for p in range(world):
            flags[p][r] = e
            yield None
        yield (lambda e=e: all((flags[r][p] - e) % (1 << 32) < (1 << 31) for p in range(world)))
        # pull: every peer's routed rows must be this layer's, completely written
        for p in range(world):
            assert q_version[p] == layer, (r, p, layer, q_version[p])
            yield None
        log.append(("pulled", r, layer))
        # expert stage, then push: store result rows into every peer's buffer
        for p in range(world):
            assert back_version[p][r] in (layer - 1, ("read", layer - 1)), (r, p, layer, back_version[p][r])
            back_version[p][r] = layer
            yield None
        # the push's last block: advance the epoch and raise the word on every peer (mp_moe_ep_push_signal)
        epoch[r] += 1
        e = epoch[r]
        for p in range(world):
            flags[p][r] = e
            yield None
        # combine (mp_moe_combine_after_peers): wait for every peer's word, then read this rank's result buffer
        yield (lambda e=e: all((flags[r][p] - e) % (1 << 32) < (1 << 31) for p in range(world)))
        for p in range(world):
            assert back_version[r][p] == layer, (r, p, layer, back_version[r][p])
            back_version[r][p] = ("read", layer)
            yield None
        log.append(("combined", r, layer))


@pytest.mark.parametrize("world,seed", [(2, 0), (2, 1), (4, 2), (8, 3), (8, 4)])
def test_expert_parallel_epoch_protocol_under_random_interleavings(world, seed):
    """Barrier-and-plan, push-then-signal and wait-then-combine with one epoch counter per rank: under any
    interleaving no rank pulls rows that are not this layer's, overwrites result rows a peer has not combined
    yet, or combines before every peer has stored.  The epochs start near the 32-bit wrap."""
    rng = np.random.default_rng(seed)
    layers = 6
    start = (1 << 32) - 5                                   # the counters wrap during the run
    flags = [[start] * world for _ in range(world)]
    epoch = [start] * world
    q_version = [0] * world
    back_version = [[0] * world for _ in range(world)]
    log = []
    progs = [_ep_rank_program(r, world, layers, flags, epoch, q_version, back_version, log) for r in range(world)]
    # wrap the model's epochs to 32 bits where they are stored
    waiting = [None] * world
    alive = set(range(world))
    steps = 0
    while alive:
        steps += 1
        assert steps < 10 ** 6, "deadlock"
        runnable = [r for r in alive if waiting[r] is None or waiting[r]()]
        assert runnable, "every rank is blocked"
        r = int(rng.choice(runnable))
        epoch[r] %= 1 << 32
        try:
            waiting[r] = next(progs[r])
        except StopIteration:
            alive.discard(r)
            waiting[r] = None
    assert sum(1 for ev in log if ev[0] == "combined") == world * layers
