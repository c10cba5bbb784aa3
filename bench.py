#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (N=1 and every N): the Llama-2-7B-shaped decoder-layer linear set in
W4A16 g128 asymmetric -- q/k/v/o 4096x4096, gate/up 4096->11008, down
11008->4096 -- at decode batch M=16, random-init N(0, 0.02) weights and
N(0, 1) fp16 activations (synthetic; no checkpoint is available offline).
One step = one pass of the seven linears over one layer set.  The timed
region cycles through a pool of layer sets whose packed weights exceed the
126 MB L2, so every step streams its weights from HBM.

Reported metric: algorithmic HBM bytes per second of the W4A16 decode linears
(packed codes + scales + packed zero points + X + Y, per linear, per step).
``value`` is measured with inputs resident in HBM and the step replayed from a
CUDA graph; ``e2e`` goes through ``VllmPackedInt4Linear.forward_host`` (the host-buffer
C-ABI entry: pinned H2D of X, kernels and D2H of Y inside the timed region; one ``forward_host_many`` call per
step, and the host keeps three independent steps in flight, each with its own pinned buffers and stream;
``e2e.timing.synchronous_ms_per_step`` is one ``forward_host`` call per linear with one step in flight).  With N>1
every rank runs an independent replica (this config does not shard) and the
values add up ("weak").  ``--impl reference`` times the reference's CPU path
for the same linears, ``F.linear(x, Wdq)`` on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_DECODE = 16
GROUP = 128
POOL_SETS = 6            # 6 x ~105 MB of packed weights: far beyond the 126 MB L2


def w4a16_bytes(n, k, m, g=GROUP):
    """Algorithmic bytes of one W4A16 linear: packed + scales + packed zeros + X + Y."""
    return n * k // 2 + 2 * n * k // g + n * k // (2 * g) + 2 * m * k + 2 * m * n


FUSE = True   # q/k/v and gate/up stored as one row-concatenated weight each (how serving runtimes hold them)


def base_shapes():
    from mindpipe_b200 import synth
    return list(synth.LLAMA2_7B_LINEARS.items())


def layer_shapes():
    """The linears one step launches: (name, (N, K)).  With FUSE the q/k/v weights are concatenated
    along the output rows into qkv_proj and gate/up into gate_up_proj (group quantisation is per row,
    so concatenation changes no code, scale or zero point)."""
    base = dict(base_shapes())
    if not FUSE:
        return list(base.items())
    return [("qkv_proj", (3 * base["q_proj"][0], base["q_proj"][1])), ("o_proj", base["o_proj"]),
            ("gate_up_proj", (2 * base["gate_proj"][0], base["gate_proj"][1])), ("down_proj", base["down_proj"])]


FUSED_PARTS = {"qkv_proj": ["q_proj", "k_proj", "v_proj"], "gate_up_proj": ["gate_proj", "up_proj"]}


def step_bytes(m):
    return sum(w4a16_bytes(n, k, m) for _, (n, k) in layer_shapes())


def step_flops(m):
    return sum(2 * m * n * k for _, (n, k) in layer_shapes())


# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs (read-only)."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._ready = threading.Event()      # NVML is up and the first sample has been taken
        self._thr = None

    def _run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            names = {
                pynvml.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                pynvml.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                pynvml.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                pynvml.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            }
            while not self._stop.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                self._ready.set()
                r = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(0.02)
        except Exception as err:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(err).__name__}")
            self._ready.set()

    def __enter__(self):
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        self._ready.wait(timeout=10)         # NVML start-up must not eat the region that is to be sampled
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thr.join(timeout=2)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


# ----------------------------------------------------------------------------
def cpu_reference_pass(sets, xs, repeats):
    """The reference's W4A16 forward on the host: nn.Linear on dequantised fp16 weights
    (algorithm/quantization/ptq/awq/source/awq/quantize/quantizer.py:109-130)."""
    import torch
    import torch.nn.functional as F
    t0 = time.perf_counter()
    with torch.no_grad():
        for r in range(repeats):
            layer = sets[r % len(sets)]
            for name, wdq in layer.items():
                F.linear(xs[name], wdq)
    return time.perf_counter() - t0


def build_cpu_sets(n_sets, m):
    """Dequantised fp16 weights produced by the oracle's restatement of pseudo_quantize_tensor."""
    import torch
    from mindpipe_b200 import synth
    from oracle import pseudo_quant as O
    sets, xs = [], {}
    for s in range(n_sets):
        layer = {}
        for i, (name, (n, k)) in enumerate(base_shapes()):
            w = synth.normal_weight(n, k, seed=s, index=i).numpy()
            wdq, _, _, _ = O.w4_group_asym_quantize(w, GROUP)
            layer[name] = torch.from_numpy(wdq)
        sets.append(layer)
    for i, (name, (n, k)) in enumerate(base_shapes()):
        xs[name] = synth.normal_activation(m, k, seed=0, index=100 + i)
    return sets, xs


def run_reference(args, rank, world):
    """The reference's CPU forward of the same linears on this box's host cores.  Under torchrun rank 0 alone
    runs it (the launcher pins every rank to one thread; that is undone here), and the line describes ONE
    replica of the workload whatever --gpus says."""
    import torch
    if rank != 0:
        return
    if world > 1 or os.environ.get("OMP_NUM_THREADS") == "1":
        torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    sets, xs = build_cpu_sets(2, M_DECODE)
    for _ in range(max(args.warmup, 1)):
        cpu_reference_pass(sets, xs, 1)
    runs = sorted(cpu_reference_pass(sets, xs, args.steps) for _ in range(5))
    dt = runs[len(runs) // 2]                                # median of five passes of `steps` steps
    gbs = step_bytes(M_DECODE) * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": "w4a16_decode_linear_algorithmic_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"median of 5 runs of {args.steps} steps of the 7-linear set at M={M_DECODE}: torch CPU "
                                   "F.linear on fp16 weights dequantised by the oracle, 2 layer sets alternating"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "replicas_timed": 1,
        "note": "one replica of the workload on the host cores; with --gpus N the GPU arm reports N replicas",
    }
    print(json.dumps(line), flush=True)


def _timed_pair(dist, dev, iters=50):
    """(eager, graph) timers for a multi-rank callable: device time per call, max over ranks, in us."""
    import torch

    def reduce_max(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3

    def timed(fn):
        for _ in range(5):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return reduce_max(e0.elapsed_time(e1) / iters)

    def timed_graph(fn):
        """`iters` calls captured in one graph and replayed once: removes the host launch path."""
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):              # warm on the capture stream: per-stream scratch exists before capture
            for _ in range(5):
                fn()
        dist.barrier()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(iters):
                    fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(side):
            e0.record(side)
            graph.replay()
            e1.record(side)
        torch.cuda.synchronize()
        return reduce_max(e0.elapsed_time(e1) / iters)

    return timed, timed_graph


def _rotating_shards(n_rows, k, dev, seed):
    """Enough independently drawn W4A16 shards of one shape that a pass over them streams more than twice the
    L2 (300 MB of packed weights), plus a callable that returns the next one: a shard of a 70B-shaped linear
    is 15-60 MB and would otherwise be timed out of the L2."""
    import itertools
    import torch
    from mindpipe_b200 import ops
    from mindpipe_b200.modules import VllmPackedInt4Linear
    copies = max(2, int(300e6 // (n_rows * k // 2)) + 1)
    shards = []
    g = torch.Generator(device=dev)
    for c in range(copies):
        g.manual_seed(seed * 1000003 + c)
        w = (torch.randn((n_rows, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.float16)
        packed, scale, zero, _ = ops.w4a16_quantize(w, GROUP)
        del w
        lin = VllmPackedInt4Linear(packed_weight=packed, scale=scale, bias=None, in_features=k, out_features=n_rows,
                                   zero_point=zero)
        lin.process_weights_after_loading()
        shards.append(lin)
    ring = itertools.cycle(shards)
    return shards, (lambda: next(ring))


def measure_row_parallel(world, rank, dev, dist, iters=50):
    """Llama-2-70B down_proj (8192 x 28672, W4A16 g128) at decode M=16 with the input features sharded
    over the ranks: the decode kernel leaves its partial sums in peer-mapped memory, a finish kernel adds them
    (one-shot: every rank adds everything; two-phase: every rank its own columns, then fp16 slices are exchanged)."""
    import torch
    from mindpipe_b200 import ops, synth
    from mindpipe_b200.modules import VllmPackedInt4Linear
    from mindpipe_b200.row_parallel import RowParallelW4A16Linear
    n, k = 8192, 28672
    if k % (world * 256):
        return {"skipped": f"{k} input features do not split into 256-column stages over {world} ranks"}
    k_loc = k // world
    shards, next_shard = _rotating_shards(n, k_loc, dev, seed=70 + rank)       # this rank's column slice, rotated
    local = shards[0]
    x = synth.normal_activation(M_DECODE, k_loc, seed=7, index=100 + rank).to(dev)
    timed, timed_graph = _timed_pair(dist, dev, iters)
    out = {"config": f"llama2-70b down_proj 8192x28672 W4A16 g128, M={M_DECODE}, K sharded over {world} ranks",
           "n_gpus": world, "weights": f"{len(shards)} shards rotated (> 2x L2 of packed weights per pass)"}

    def rotated(layer):
        def call():
            layer.local = next_shard()
            return layer(x)
        return call

    for name, two_phase in (("one_shot", False), ("two_phase", True)):
        layer = RowParallelW4A16Linear(local, None, max_rows=M_DECODE, two_phase=two_phase)
        if two_phase and not layer.two_phase:
            continue
        out[f"us_fused_{name}_eager_launches"] = timed(rotated(layer))
        ops.check_device_errors()
        out[f"us_fused_{name}"] = timed_graph(rotated(layer))
        ops.check_device_errors()
    layer = RowParallelW4A16Linear(local, None, max_rows=M_DECODE)            # default choice for this world size
    out["default_exchange"] = "two_phase" if layer.two_phase else "one_shot"
    out["us_fused_push_allreduce"] = out[f"us_fused_{out['default_exchange']}"]
    out["us_local_gemm_only"] = timed_graph(lambda: next_shard()(x))
    layer.local = local

    def nccl_call():
        layer.local = next_shard()
        return layer.forward_nccl(x)
    out["us_local_gemm_plus_nccl_allreduce_eager"] = timed(nccl_call)
    out["algorithmic_gbs_whole_job"] = w4a16_bytes(n, k, M_DECODE) / (out["us_fused_push_allreduce"] * 1e-6) / 1e9
    return out


def measure_column_parallel(world, rank, dev, dist, iters=50):
    """The split BASELINE config 5 names: Llama-2-70B-shaped W4A16 linears with the OUTPUT rows sharded over
    the ranks, decode M in {1, 8, 64}, all-gather of the output slices.  Local kernel and gather are timed
    separately; the gather both as the device-driven peer-store exchange and as NCCL all_gather_into_tensor."""
    import torch
    from mindpipe_b200 import ops, synth
    from mindpipe_b200.column_parallel import ColumnParallelW4A16Linear
    from mindpipe_b200.modules import VllmPackedInt4Linear
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks_path.read_text())["hbm_gbs"] if peaks_path.exists() else 6650.0
    timed, timed_graph = _timed_pair(dist, dev, iters)
    rows = []
    for name, (n, k) in (("gate_up_proj", (28672, 8192)), ("attn_proj", (8192, 8192))):
        if n % world or ((n // world) * 2) % 16:
            rows.append({"linear": name, "skipped": f"{n} rows do not split over {world} ranks"})
            continue
        n_loc = n // world
        shards, next_shard = _rotating_shards(n_loc, k, dev, seed=110 + rank)  # this rank's row slice, rotated
        local = shards[0]
        layer = ColumnParallelW4A16Linear(local, n, max_rows=64)

        def fused():
            layer.local = next_shard()
            return layer(x)

        def nccl():
            layer.local = next_shard()
            return layer.forward_nccl(x)

        for m in (1, 8, 64):
            x = synth.normal_activation(m, k, seed=11, index=200).to(dev)      # replicated activations
            layer.local = local
            same = bool(torch.equal(layer(x), layer.forward_nccl(x)))
            ops.check_device_errors()
            us_local = timed_graph(lambda: next_shard()(x))
            us_fused = timed_graph(fused)
            ops.check_device_errors()
            us_nccl = timed(nccl)
            y_loc = local(x).contiguous()
            us_gather_nccl = timed(lambda: layer._gather_nccl(y_loc))
            gbs = w4a16_bytes(n, k, m) / (us_fused * 1e-6) / 1e9
            rows.append({"linear": name, "N": n, "K": k, "M": m, "us_local_kernel": us_local,
                         "us_local_plus_peer_gather": us_fused, "us_peer_gather": max(us_fused - us_local, 0.0),
                         "us_local_plus_nccl_all_gather_eager": us_nccl, "us_nccl_all_gather_eager": us_gather_nccl,
                         "algorithmic_gbs_whole_job": gbs, "frac_of_n_x_measured_hbm": gbs / (world * hbm),
                         "gathers_agree_bitwise": same, "shards_rotated": len(shards)})
        del shards, layer
    return {"config": f"llama2-70b-shaped W4A16 g128 linears, output rows sharded over {world} ranks, all-gather of "
                      "the output slices; weight shards rotated (> 2x L2 per pass)", "n_gpus": world, "rows": rows,
            "parity": all(r.get("gathers_agree_bitwise", True) for r in rows)}


def measure_moe(world, rank, dev, dist, iters=10):
    """Mixtral-8x7B-shaped W8A8 MoE layer (8 experts, hidden 4096, ffn 14336, top-2, 8192 tokens):
    experts sharded over the ranks, tokens data-sharded, all-to-all dispatch/combine.  tokens/s of the
    whole job = 8192 / (max over ranks of the layer time)."""
    import torch
    from mindpipe_b200 import ops, synth
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts
    shape = synth.MIXTRAL_8X7B
    if shape.num_experts % world:
        return {"skipped": f"{shape.num_experts} experts do not divide over {world} ranks"}
    per = shape.num_experts // world
    lo, hi = rank * per, (rank + 1) * per
    parts = []
    for e in range(lo, hi):                                    # expert by expert: bounded host/device memory
        gu, dn = synth.moe_weights(shape, seed=0, experts=range(e, e + 1))
        parts.append(SmoothQuantPackedMoeExperts(gu.to(dev), dn.to(dev), torch.nn.SiLU(), expert_range=(e, e + 1),
                                                 num_experts=shape.num_experts))
    mod = parts[0]
    mod.gate_up_proj = torch.cat([m.gate_up_proj for m in parts])
    mod.gate_up_proj_scale = torch.cat([m.gate_up_proj_scale for m in parts])
    mod.down_proj = torch.cat([m.down_proj for m in parts])
    mod.down_proj_scale = torch.cat([m.down_proj_scale for m in parts])
    mod.expert_range = (lo, hi)
    del parts
    t_loc = shape.tokens // world
    hs = synth.normal_activation(shape.tokens, shape.hidden, seed=0)[rank * t_loc:(rank + 1) * t_loc].to(dev)
    logits = synth.router_logits(shape.tokens, shape.num_experts, seed=0)[rank * t_loc:(rank + 1) * t_loc].to(dev)
    idx, wts = ops.moe_router_topk(logits, shape.top_k)
    exchange = "none"
    if world > 1:
        from mindpipe_b200.expert_parallel import ExpertParallelMoE, SymmetricExpertParallelMoE
        try:
            layer = SymmetricExpertParallelMoE(mod, shape.num_experts, max_tokens_per_rank=t_loc, top_k=shape.top_k)
            exchange = ("peer-memory pull kernel, results stored at home by the second GEMM's epilogue"
                        if layer.fuse_return else "peer-memory pull/push kernels") + " (symmetric memory, no host sync)"
        except Exception as err:      # no peer mapping available: NCCL all-to-all with host-side split sizes
            layer = ExpertParallelMoE(mod, shape.num_experts)
            exchange = f"nccl all_to_all_single ({type(err).__name__})"
    else:
        layer = mod

    def time_layer(layer):
        for _ in range(2):
            layer(hs, idx, wts)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        replay = None
        if exchange.startswith("peer-memory") or world == 1:
            # the layer is a fixed launch sequence (no host read, barrier epochs in device memory): capture it
            # once and replay it, as a serving runtime would, so that host launch gaps are not timed
            side = torch.cuda.Stream(device=dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    layer(hs, idx, wts)
            replay = (graph, side)
            launch_mode = "cuda graph replay"
        else:
            launch_mode = "eager"
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if replay is not None:
            graph, side = replay
            with torch.cuda.stream(side):
                graph.replay()                               # one untimed replay
                e0.record(side)
                for _ in range(iters):
                    graph.replay()
                e1.record(side)
        else:
            e0.record()
            for _ in range(iters):
                layer(hs, idx, wts)
            e1.record()
        torch.cuda.synchronize()
        ops.check_device_errors()
        t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launch_mode

    # every launch of the layer waits for its predecessor on the device (griddepcontrol.wait), so the launches may be
    # scheduled early: the switch is read when a launch is issued, i.e. at capture time
    from mindpipe_b200 import _lib
    pdl_before = _lib.load().mp_set_programmatic_launch(1)
    ms, launch_mode = time_layer(layer)
    extra = {}
    if world > 1 and exchange.startswith("peer-memory"):
        # the same layer with the GEMMs in two halves of the row tiles and the exchange of one half overlapping the
        # other half's GEMMs on a second stream (an option of the module, off by default), for comparison
        halves = SymmetricExpertParallelMoE(mod, shape.num_experts, max_tokens_per_rank=t_loc, top_k=shape.top_k,
                                            overlap=True)
        extra["ms_per_layer_with_overlapped_exchange"] = time_layer(halves)[0]
    _lib.load().mp_set_programmatic_launch(pdl_before)
    int8_ops = 2 * (shape.top_k * shape.tokens) * shape.hidden * 2 * shape.ffn + \
        2 * (shape.top_k * shape.tokens) * shape.ffn * shape.hidden
    return {"config": "mixtral-8x7b-shaped layer, 8192 tokens, top-2, experts sharded over the ranks (all-to-all)",
            "ms_per_layer": ms, "tokens_per_s": shape.tokens / (ms * 1e-3), "int8_tops": int8_ops / (ms * 1e-3) / 1e12,
            "n_gpus": world, "exchange": exchange, "launches": launch_mode, **extra}


def workload_config():
    return {"workload": "llama2-7b decoder-layer linear set (q,k,v,o 4096x4096; gate,up 11008x4096; down 4096x11008), "
                        f"W4A16 asymmetric int4 g{GROUP}, decode M={M_DECODE}",
            "launches_per_step": [f"{name} {n}x{k}" for name, (n, k) in layer_shapes()],
            "weight_pool": f"{POOL_SETS} layer sets cycled, {POOL_SETS * step_bytes(M_DECODE) / 1e6:.0f} MB > 126 MB L2 "
                           "(inputs larger than L2; no explicit flush)",
            "parallelism": "replicas only (this config does not shard)"}


# ----------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    from mindpipe_b200 import ops, synth
    from mindpipe_b200.modules import VllmPackedInt4Linear

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    # Weights are static from here on, so the decode kernels may prefetch them while the
    # previous kernel of the stream drains (programmatic dependent launch).
    from mindpipe_b200 import _lib
    # ---- build the pool: quantise seeded weights on the GPU with the product's own kernel ----
    pool = []
    base_index = {name: i for i, (name, _) in enumerate(base_shapes())}
    for s in range(POOL_SETS):
        parts = {}
        for name, (n, k) in base_shapes():
            w = synth.normal_weight(n, k, seed=s, index=base_index[name]).to(dev)
            parts[name] = ops.w4a16_quantize(w, GROUP)[:3]
            del w
        layer = []
        for name, (n, k) in layer_shapes():
            members = FUSED_PARTS.get(name, [name]) if FUSE else [name]
            packed = torch.cat([parts[m_][0] for m_ in members]).contiguous()
            scale = torch.cat([parts[m_][1] for m_ in members]).contiguous()
            zero = torch.cat([parts[m_][2] for m_ in members]).contiguous()
            mod = VllmPackedInt4Linear(packed_weight=packed, scale=scale, bias=None, in_features=k,
                                       out_features=n, zero_point=zero)
            mod.process_weights_after_loading()
            layer.append((name, mod))
        del parts
        pool.append(layer)
    x_host = {name: synth.normal_activation(M_DECODE, k, seed=0, index=100 + i).pin_memory()
              for i, (name, (n, k)) in enumerate(layer_shapes())}
    x_dev = {name: t.to(dev) for name, t in x_host.items()}
    y_host = {name: torch.empty((M_DECODE, n), dtype=torch.float16).pin_memory() for name, (n, k) in layer_shapes()}
    torch.cuda.synchronize()
    _lib.load().mp_set_programmatic_launch(1 if args.pdl else 0)

    ws_bytes = max(ops.w4a16_decode_workspace_bytes(M_DECODE, n, k) for _, (n, k) in layer_shapes())
    # one scratch buffer per linear: with --fuse 0 --concurrent 1 some of them run side by side
    ws = {name: ops.new_workspace(ws_bytes, dev) for name, _ in layer_shapes()}
    umma_names = [name for name, (n, k) in layer_shapes() if ops.w4a16_decode_kernel_choice(M_DECODE, n, k) == "umma"]
    tma_names = [name for name, _ in layer_shapes() if name not in umma_names]
    kernel_names = " + ".join(
        f"{kern} ({', '.join(names)})" for kern, names in (("w4a16_decode_umma_kernel", umma_names),
                                                           ("w4a16_decode_tma_kernel", tma_names)) if names)
    y_dev = {name: torch.empty((M_DECODE, n), dtype=torch.float16, device=dev) for name, (n, k) in layer_shapes()}

    side = [torch.cuda.Stream(device=dev) for _ in range(2)]

    def launch(name, mod):
        ops.w4a16_linear_decode(x_dev[name], mod.weight_packed, mod._scale_zero, workspace=ws[name], out=y_dev[name])

    def step(layer):
        """The layer's dependency structure: q, k, v side by side; o; gate, up side by side; down."""
        mods = dict(layer)
        main = torch.cuda.current_stream()

        def parallel(names):
            if not args.concurrent:
                for n in names:
                    launch(n, mods[n])
                return
            for s_, n in zip(side, names[1:]):
                s_.wait_stream(main)
                with torch.cuda.stream(s_):
                    launch(n, mods[n])
            launch(names[0], mods[names[0]])
            for s_ in side[:len(names) - 1]:
                main.wait_stream(s_)

        if FUSE:
            for n in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj"):
                launch(n, mods[n])
            return
        parallel(["q_proj", "k_proj", "v_proj"])
        launch("o_proj", mods["o_proj"])
        parallel(["gate_proj", "up_proj"])
        launch("down_proj", mods["down_proj"])

    # ---- multi-rank parity first: the sharded paths against the single-GPU modules, inside this very job ----
    parity = None
    if dist is not None:
        try:
            from mindpipe_b200.verify import all_ranks_agree, verify_multi_gpu
            parity = all_ranks_agree(verify_multi_gpu(rank, world, dev), dev)
        except Exception as err:
            parity = {"error": f"{type(err).__name__}: {err}"[:200]}

    # ---- the timed steps as ONE CUDA graph (K steps back to back, as a serving runtime captures a whole
    # decode pass: no host launch gaps, and under programmatic dependent launch a linear's prologue runs under
    # its predecessor's tail across step boundaries too) ----
    for layer in pool[:2]:
        step(layer)
    torch.cuda.synchronize()
    launches_per_step = len(layer_shapes())

    def capture(first, count):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(count):
                step(pool[(first + i) % POOL_SETS])
        return g

    warm_graph = capture(0, args.warmup)
    timed_graph = capture(args.warmup, args.steps)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    warm_graph.replay()
    timed_graph.replay()                    # one untimed replay of the timed graph itself (first-replay set-up)
    warm_graph.replay()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        ev0.record()
        timed_graph.replay()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if ms < 200:                       # keep the sampler alive long enough to see clocks under load
            t_end = time.time() + 0.4
            while time.time() < t_end:
                warm_graph.replay()
            torch.cuda.synchronize()

    # ---- end to end: module API, host buffers, H2D + D2H inside the timed region ----
    # Steps are independent requests, so the host keeps E2E_DEPTH of them in flight, as a serving loop does: each
    # in-flight step has its own pinned input / output buffers and its own stream (forward_host_many only
    # enqueues the H2D copies of X, the kernels and the D2H copies of Y and returns), and before a step's buffers
    # are reused the host waits until the results of the step that used them last are in host memory.  One step's
    # copies then overlap another step's kernels.  `synchronous_ms_per_step` in `e2e.timing` is one forward_host
    # call per linear with a device synchronisation after every step (one step in flight, the set's linears on
    # separate streams).
    E2E_DEPTH = 3                                       # divides POOL_SETS: a module always meets the same slot
    x_slots = [x_host] + [{n: t.clone().pin_memory() for n, t in x_host.items()} for _ in range(E2E_DEPTH - 1)]
    y_slots = [y_host] + [{n: torch.empty_like(t).pin_memory() for n, t in y_host.items()} for _ in range(E2E_DEPTH - 1)]
    slot_streams = [torch.cuda.Stream(device=dev) for _ in range(E2E_DEPTH)]
    slot_done = [torch.cuda.Event() for _ in range(E2E_DEPTH)]
    e2e_streams = [torch.cuda.Stream(device=dev) for _ in layer_shapes()]

    waited = [0.0]                                     # seconds the host spent waiting for a slot's results

    from mindpipe_b200.modules import forward_host_many
    many_args = {}                                     # (layer set, slot) -> argument lists of forward_host_many

    def e2e_issue(i, layer):
        slot = i % E2E_DEPTH
        w0 = time.perf_counter()
        slot_done[slot].synchronize()                  # this slot's previous results have reached host memory
        waited[0] += time.perf_counter() - w0
        if args.e2e_call == "many":
            # the set's linears are independent: one library call enqueues their copies in, the kernels back to
            # back (programmatic dependent launch between them) and the copies out
            lists = many_args.get((id(layer), slot))
            if lists is None:
                lists = many_args[(id(layer), slot)] = ([mod for _, mod in layer],
                                                        [x_slots[slot][name] for name, _ in layer],
                                                        [y_slots[slot][name] for name, _ in layer])
            forward_host_many(*lists, stream=slot_streams[slot])
        else:
            for name, mod in layer:
                mod.forward_host(x_slots[slot][name], y_slots[slot][name], stream=slot_streams[slot],
                                 zero_copy_output=args.e2e_call == "single_zero_copy")
        slot_done[slot].record(slot_streams[slot])

    def e2e_run(count):
        t0 = time.perf_counter()
        for i in range(count):
            e2e_issue(i, pool[(args.warmup + i) % POOL_SETS])
        for ev in slot_done:                           # every result is in host memory before the clock stops
            ev.synchronize()
        return time.perf_counter() - t0

    def e2e_step(layer):                               # one step in flight
        for s_, (name, mod) in zip(e2e_streams, layer):
            mod.forward_host(x_host[name], y_host[name], stream=s_)   # H2D of X, kernel, D2H of Y on this stream
        torch.cuda.synchronize()

    def e2e_run_synchronous(count):
        t0 = time.perf_counter()
        for i in range(count):
            e2e_step(pool[(args.warmup + i) % POOL_SETS])
        return time.perf_counter() - t0

    e2e_s, e2e_detail = float("nan"), None
    if not args.no_e2e:
        # every (layer set, linear) pair is called once before the clock starts, whatever --warmup says: the
        # first forward_host of a module allocates its staging buffers and encodes its tensor maps
        for layer in pool:
            e2e_step(layer)
        e2e_run(2 * POOL_SETS + args.warmup)
        # `steps` steps take a few milliseconds: repeat the run until at least 0.5 s has been timed per sample,
        # take five samples and report the median per-step time
        probe = e2e_run(args.steps)
        inner = max(1, int(0.5 / max(probe, 1e-6)) + 1)
        barrier()
        samples = []
        waited[0] = 0.0
        for _ in range(5):
            samples.append(e2e_run(args.steps * inner) / inner)
        # share of the timed loop the host spent blocked on results: near 0 = the host's enqueue path is the
        # limit, near 1 = the device is
        host_wait_share = waited[0] / max(sum(samples) * inner, 1e-9)
        barrier()
        samples.sort()
        e2e_s = samples[len(samples) // 2]
        sync_samples = sorted(e2e_run_synchronous(args.steps * inner) / inner for _ in range(3))
        barrier()
        e2e_detail = {"samples_ms_per_step": [round(v / args.steps * 1e3, 4) for v in samples],
                      "steps_per_sample": args.steps * inner, "statistic": "median of 5",
                      "steps_in_flight": E2E_DEPTH, "host_wait_share": round(host_wait_share, 3),
                      "call": {"many": "forward_host_many (one call per step)", "single": "forward_host per linear",
                               "single_zero_copy": "forward_host per linear, zero-copy output"}[args.e2e_call],
                      "synchronous_ms_per_step": round(sync_samples[1] / args.steps * 1e3, 4)}
        # For information: the same host-buffer calls captured once per layer set in a CUDA graph (H2D copies, kernels
        # and D2H copies as graph nodes, the linears on forked streams) and replayed, one synchronisation per step --
        # what a serving loop that captures its step pays.  Not the headline `e2e`, which issues every call.
        try:
            cap = torch.cuda.Stream(device=dev)
            set_graphs = []
            for layer in pool:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.stream(cap):
                    with torch.cuda.graph(g, stream=cap):
                        fork = torch.cuda.Event()
                        fork.record(cap)
                        for s_, (name, mod) in zip(e2e_streams, layer):
                            s_.wait_event(fork)
                            mod.forward_host(x_host[name], y_host[name], stream=s_)
                            join = torch.cuda.Event()
                            join.record(s_)
                            cap.wait_event(join)
                set_graphs.append(g)

            def graph_run(count):
                t0 = time.perf_counter()
                with torch.cuda.stream(cap):
                    for i in range(count):
                        set_graphs[(args.warmup + i) % POOL_SETS].replay()
                        torch.cuda.synchronize()
                return time.perf_counter() - t0

            graph_run(2 * POOL_SETS)
            barrier()
            gs = sorted(graph_run(args.steps * inner) / inner for _ in range(3))
            barrier()
            e2e_detail["graph_replay_ms_per_step"] = round(gs[1] / args.steps * 1e3, 4)
        except Exception as err:          # informational only
            e2e_detail["graph_replay_error"] = f"{type(err).__name__}: {err}"[:160]

    t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()

    def extra(fn, *a):
        try:
            return fn(*a)
        except Exception as err:          # the headline number must not depend on an extra
            return {"error": f"{type(err).__name__}: {err}"[:200]}

    moe_extra = extra(measure_moe, world, rank, dev, dist) if args.moe else None
    tp_extra = col_extra = None
    if args.tp and world > 1:             # the sharded 70B linears
        tp_extra = extra(measure_row_parallel, world, rank, dev, dist)
        col_extra = extra(measure_column_parallel, world, rank, dev, dist)
    configs_extra = None
    if args.configs and world == 1 and rank == 0:
        configs_extra = extra(measure_other_configs, args, local_rank)

    if rank == 0:
        bytes_step = step_bytes(M_DECODE)
        value = world * bytes_step * args.steps / (ms * 1e-3) / 1e9
        e2e_val = world * bytes_step * args.steps / (e2e_ms * 1e-3) / 1e9
        peaks_path = ROOT / "MEASURED_PEAKS.json"
        if peaks_path.exists():
            peak, peak_src = json.loads(peaks_path.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = 6650.0, "fallback 6.65 TB/s"
        achieved = bytes_step * args.steps / (ms * 1e-3) / 1e9          # per GPU: the kernel's own rate
        traffic = None
        tr = ROOT / "profiles" / "w4a16_decode_traffic.json"
        if tr.exists():
            traffic = json.loads(tr.read_text()).get("dram_bytes_per_launch")
        line = {
            "metric": "w4a16_decode_linear_algorithmic_hbm_gbs", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_src, "kernel": kernel_names,
                         "launch_bytes_avg": bytes_step / launches_per_step,
                         "launch_us_avg": ms * 1e3 / (args.steps * launches_per_step)},
            "e2e": {"value": e2e_val, "unit": "GB/s",
                    "h2d_bytes_per_step": sum(t.numel() * 2 for t in x_host.values()),
                    "d2h_bytes_per_step": sum(t.numel() * 2 for t in y_host.values()),
                    "timing": e2e_detail},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "tflops": world * step_flops(M_DECODE) * args.steps / (ms * 1e-3) / 1e12,
            "moe_w8a8": moe_extra,
        }
        if parity is not None:
            line["multi_gpu_parity"] = parity
        if tp_extra is not None:
            line["tp_row_parallel"] = tp_extra
        if col_extra is not None:
            line["tp_column_parallel"] = col_extra
        if configs_extra is not None:
            line["configs"] = configs_extra
        if world == 1 and not args.no_cpu_baseline:
            cores = torch.get_num_threads()
            sets, xs = build_cpu_sets(2, M_DECODE)
            cpu_reference_pass(sets, xs, 2)
            reps = 40
            dt = cpu_reference_pass(sets, xs, reps)
            line["cpu_baseline"] = {"value": bytes_step * reps / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": f"{reps} passes of the 7-linear set at M={M_DECODE} (torch CPU F.linear on "
                                              "oracle-dequantised fp16 weights), 2 layer sets alternating"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def measure_other_configs(args, local_rank):
    """The other BASELINE configs at their full sizes, one compact record each (kernel-level timings, graph
    replay, operands rotated through more than twice the L2): config 2 prefill M=2048, config 3 W8A8 M=4096,
    config 5 decode M in {1, 8, 64}."""
    rows = []
    sub = argparse.Namespace(**vars(args))
    sub.suite, sub.decode_shapes, sub.decode_m, sub.suite_pdl = "decode,prefill,w8a8", "8192x8192,1024x8192,28672x8192,8192x28672", "1,8,64", 1
    sub.fast_weights = True
    errors = {}
    for one in sub.suite.split(","):             # a failure in one config must not lose the others
        sub.suite = one
        try:
            run_suite(sub, local_rank, collect=rows)
        except Exception as exc:                 # noqa: BLE001 -- reported in the record
            errors[one] = f"{type(exc).__name__}: {exc}"[:300]
    out = {"w4a16_decode_llama2_70b": [], "w4a16_prefill_llama2_7b": [], "w8a8_llama3_8b": []}
    for r in rows:
        if r["suite"] == "w4a16_decode":
            out["w4a16_decode_llama2_70b"].append({k: r[k] for k in ("N", "K", "M", "us", "gbs", "frac_of_measured_hbm")})
        elif r["suite"] == "w4a16_prefill":
            out["w4a16_prefill_llama2_7b"].append({k: r[k] for k in ("N", "K", "M", "us", "tflops", "frac_of_measured_bf16_burst")})
        elif r["suite"] == "w8a8":
            out["w8a8_llama3_8b"].append({k: r[k] for k in ("N", "K", "M", "act_quant_us", "act_quant_gbs", "gemm_us", "gemm_tops",
                                                          "linear_tops", "library_int8_gemm_tops")})
    if errors:
        out["errors"] = errors
    out["note"] = ("decode: chains of launches under programmatic dependent launch, weights rotated; M=64 goes where "
                   "ops.w4a16_linear sends it (tcgen05 weight-streaming kernel with a 64-token tile on the 70B-sized "
                   "weights, split-K tensor-core GEMM otherwise); library_int8_gemm_tops is torch._int_mm on the same box, "
                   "a timing yardstick only (MEASURED_PEAKS.json has no int8 figure)")
    return out


# ----------------------------------------------------------------------------
def run_suite(args, local_rank, collect=None):
    """Per-kernel numbers for the other configs (one JSON line each, after the headline line; appended to
    `collect` instead when a list is given)."""
    import torch
    from mindpipe_b200 import _lib, ops, synth
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_path.read_text()) if peaks_path.exists() else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

    def timed(fn, iters, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e-3

    def timed_graph(fns, rounds=4, warm=2):
        """Kernels shorter than the host's launch path: capture the callables (rotated, so that inputs
        larger than L2 are streamed from HBM) in one CUDA graph and time its replay."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(warm):
                for fn in fns:
                    fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(rounds):
                    for fn in fns:
                        fn()
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (rounds * len(fns)) * 1e-3

    def emit(**kw):
        if collect is not None:
            collect.append(kw)
        else:
            print(json.dumps(kw), flush=True)

    def weight(n, k, seed, index=0):
        """N(0, 0.02) fp16 weights: seeded on the CPU (reproducible bits), or drawn on the device when only
        timings are wanted (a 28672 x 8192 matrix takes seconds on the host)."""
        if getattr(args, "fast_weights", False):
            g = torch.Generator(device=dev)
            g.manual_seed(seed * 1000003 + index)
            return (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.float16)
        return synth.normal_weight(n, k, seed=seed, index=index).to(dev)

    want = set(args.suite.split(","))
    if "decode" in want or "all" in want:
        shapes = [(4096, 4096), (11008, 4096), (4096, 11008), (8192, 8192), (28672, 8192), (8192, 28672)]
        if args.decode_shapes:
            shapes = [tuple(int(v) for v in sh.split("x")) for sh in args.decode_shapes.split(",")]
        for (n, k) in shapes:
            copies = max(2, int(300e6 // (n * k // 2)) + 1)           # rotate > 2x L2 of packed weights
            mods = []
            for c in range(copies):
                w = weight(n, k, c)
                packed, scale, zero, _ = ops.w4a16_quantize(w, GROUP)
                mods.append((packed, ops.w4a16_prepare(scale, zero, k)))
                del w
            _lib.load().mp_set_programmatic_launch(1 if args.suite_pdl else 0)
            for m in [int(v) for v in args.decode_m.split(",")]:
                x = synth.normal_activation(m, k, seed=0).to(dev)
                y = torch.empty((m, n), dtype=torch.float16, device=dev)
                ws_dec = ops.new_workspace(max(ops.w4a16_decode_workspace_bytes(m, n, k), 20 << 20), dev)
                ws_pre = ops.new_workspace(_lib.load().mp_w4a16_prefill_workspace_bytes(m, n, k), dev) if m > 16 else None
                # 17..64 rows: what ops.w4a16_linear does -- the tcgen05 weight-streaming kernel with a 32/64-token
                # tile where the library's rule picks it (or when asked for), else the split-K tensor-core GEMM
                wide_umma = 16 < m <= 64 and (args.decode_kernel == "umma" or (
                    args.decode_kernel in ("default", "auto") and ops.w4a16_decode_kernel_choice(m, n, k) == "umma"))
                opt_umma = ops.decode_options(kernel="umma")

                def call(pk, sz):
                    if m <= 16:
                        ops.w4a16_linear_decode(x, pk, sz, workspace=ws_dec, out=y)
                    elif wide_umma:             # the tcgen05 weight-streaming kernel with a 32/64-token tile
                        ops.w4a16_linear_decode(x, pk, sz, workspace=ws_dec, out=y, options=opt_umma)
                    else:                       # above 16 rows ops.w4a16_linear takes the split-K tensor-core GEMM
                        ops.w4a16_linear_prefill(x, pk, sz, workspace=ws_pre)
                g = torch.cuda.CUDAGraph()
                for pk, sz in mods:
                    call(pk, sz)
                torch.cuda.synchronize()
                with torch.cuda.graph(g):
                    for pk, sz in mods:
                        call(pk, sz)
                t = timed(g.replay, 20) / copies
                b = w4a16_bytes(n, k, m)
                emit(suite="w4a16_decode", N=n, K=k, M=m, us=t * 1e6, gbs=b / t / 1e9,
                     frac_of_measured_hbm=b / t / 1e9 / peaks["hbm_gbs"],
                     kernel=args.decode_kernel if m <= 16 else ("umma" if wide_umma else "gemm"),
                     **({"pdl": 1} if args.suite_pdl else {}))
            _lib.load().mp_set_programmatic_launch(0)
            del mods
    if "prefill" in want or "all" in want:
        for (n, k) in [(4096, 4096), (11008, 4096), (4096, 11008)]:
            w = weight(n, k, 0)
            packed, scale, zero, _ = ops.w4a16_quantize(w, GROUP)
            sz = ops.w4a16_prepare(scale, zero, k)
            x = synth.normal_activation(2048, k, seed=0).to(dev)
            t = timed(lambda: ops.w4a16_linear_prefill(x, packed, sz), 20)
            fl = 2 * 2048 * n * k
            emit(suite="w4a16_prefill", N=n, K=k, M=2048, us=t * 1e6, tflops=fl / t / 1e12,
                 frac_of_measured_bf16_burst=fl / t / 1e12 / peaks["bf16_tflops"])
    if "midm" in want or "all" in want:
        # batch sizes between decode and prefill, through the dispatching entry (ops.w4a16_linear)
        for (n, k) in [(4096, 4096), (11008, 4096), (4096, 11008)]:
            copies = max(2, int(300e6 // (n * k // 2)) + 1)
            mods = []
            for c in range(copies):
                w = synth.normal_weight(n, k, seed=c, index=0).to(dev)
                packed, scale, zero, _ = ops.w4a16_quantize(w, GROUP)
                mods.append((packed, ops.w4a16_prepare(scale, zero, k)))
                del w
            for m in (32, 64, 128, 256, 512, 1024):
                x = synth.normal_activation(m, k, seed=0).to(dev)
                t = timed_graph([(lambda pk=pk, sz=sz: ops.w4a16_linear(x, pk, sz)) for pk, sz in mods], rounds=2)
                emit(suite="w4a16_mid_m", N=n, K=k, M=m, us=t * 1e6, gbs=w4a16_bytes(n, k, m) / t / 1e9,
                     tflops=2 * m * n * k / t / 1e12)
            del mods
    if "midm" in want or "all" in want:
        # the W8A8 linear (per-token quant + int8 GEMM) at decode / small-batch row counts
        for (n, k) in [(4096, 4096), (14336, 4096), (4096, 14336)]:
            copies = max(2, int(300e6 // (n * k)) + 1)
            ws_ = []
            for c in range(copies):
                w = synth.normal_weight(n, k, seed=c, index=0).to(dev)
                qw, sw, _ = ops.act_quant_per_token(w)
                ws_.append((qw, sw))
                del w
            for m in (1, 16, 64, 256, 1024):
                x = synth.outlier_activation(m, k, seed=0).to(dev)

                def lin(qw, sw):
                    qx, sx, _ = ops.act_quant_per_token(x)
                    return ops.w8a8_gemm(qx, sx, qw, sw)
                t = timed_graph([(lambda qw=qw, sw=sw: lin(qw, sw)) for qw, sw in ws_], rounds=2)
                emit(suite="w8a8_mid_m", N=n, K=k, M=m, us=t * 1e6, weight_gbs=n * k / t / 1e9,
                     tops=2 * m * n * k / t / 1e12)
            del ws_
    if "w8a8" in want or "all" in want:
        for (n, k) in [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]:
            m = 4096
            w = weight(n, k, 0)
            qw, sw, _ = ops.act_quant_per_token(w)
            x = synth.outlier_activation(m, k, seed=0).to(dev)
            qx, sx, _ = ops.act_quant_per_token(x)
            xs = [x] + [synth.outlier_activation(m, k, seed=0, index=i).to(dev)
                        for i in range(1, max(2, int(300e6 // (2 * m * k)) + 1))]       # rotate > 2x L2
            t_q = timed_graph([(lambda xi=xi: ops.act_quant_per_token(xi)) for xi in xs])
            t_g = timed(lambda: ops.w8a8_gemm(qx, sx, qw, sw), 20)
            op = 2 * m * n * k
            lib_tops = None
            try:                                   # library int8 GEMM: a timing yardstick only
                wt = qw.t().contiguous()
                t_l = timed(lambda: torch._int_mm(qx, wt), 20)
                lib_tops = op / t_l / 1e12
            except Exception:
                pass
            emit(suite="w8a8", N=n, K=k, M=m, library_int8_gemm_tops=lib_tops, act_quant_us=t_q * 1e6, act_quant_gbs=3 * m * k / t_q / 1e9,
                 gemm_us=t_g * 1e6, gemm_tops=op / t_g / 1e12, linear_tops=op / (t_g + t_q) / 1e12,
                 note="int8 dense peak is 2x the bf16 figure nominally (4.5 vs 2.25 POP/s)")
    if "moe" in want or "all" in want:
        shape = synth.MIXTRAL_8X7B
        gus, dns = [], []
        mod = None
        for e in range(shape.num_experts):                      # quantise expert by expert to bound memory
            gu, dn = synth.moe_weights(shape, seed=0, experts=range(e, e + 1))
            m1 = SmoothQuantPackedMoeExperts(gu.to(dev), dn.to(dev), torch.nn.SiLU(), expert_range=(e, e + 1),
                                             num_experts=shape.num_experts)
            gus.append((m1.gate_up_proj, m1.gate_up_proj_scale))
            dns.append((m1.down_proj, m1.down_proj_scale))
            mod = m1
        mod.gate_up_proj = torch.cat([g[0] for g in gus])
        mod.gate_up_proj_scale = torch.cat([g[1] for g in gus])
        mod.down_proj = torch.cat([d[0] for d in dns])
        mod.down_proj_scale = torch.cat([d[1] for d in dns])
        mod.expert_range = (0, shape.num_experts)
        del gus, dns
        hs = synth.normal_activation(shape.tokens, shape.hidden, seed=0).to(dev)
        idx, wts = ops.moe_router_topk(synth.router_logits(shape.tokens, shape.num_experts, seed=0).to(dev), 2)
        t = timed(lambda: mod(hs, idx, wts), 5, warm=2)
        ops.check_device_errors()
        opsn = 2 * (2 * shape.tokens) * shape.hidden * 2 * shape.ffn + 2 * (2 * shape.tokens) * shape.ffn * shape.hidden
        emit(suite="moe_w8a8", tokens=shape.tokens, ms=t * 1e3, tokens_per_s=shape.tokens / t, tops=opsn / t / 1e12)


def main():
    global POOL_SETS, FUSE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--e2e-call", default="many", choices=["many", "single", "single_zero_copy"],
                    help="end-to-end leg: one forward_host_many call per step (default), one forward_host call per "
                         "linear, or the latter with the kernels storing straight into the pinned output")
    ap.add_argument("--pool-sets", type=int, default=POOL_SETS, help="layer sets in the weight pool")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch for the decode linears")
    ap.add_argument("--fuse", type=int, default=1,
                    help="hold q/k/v and gate/up as row-concatenated weights (4 launches per step instead of 7)")
    ap.add_argument("--concurrent", type=int, default=1,
                    help="run q/k/v and gate/up of a layer on parallel streams inside the captured step")
    ap.add_argument("--moe", type=int, default=1, help="also measure the expert-parallel MoE layer (extra key)")
    ap.add_argument("--tp", type=int, default=1, help="on N > 1: also measure the tensor-parallel 70B-shaped linears (extra keys)")
    ap.add_argument("--configs", type=int, default=1, help="on N = 1: also measure the other configs (extra key)")
    ap.add_argument("--suite", default="", help="comma list of extra per-kernel lines: decode,prefill,w8a8,moe,all")
    ap.add_argument("--suite-only", action="store_true", help="skip the headline workload")
    ap.add_argument("--decode-kernel", default="default", choices=["default", "auto", "umma", "mma_sync"],
                    help="kernel behind the M <= 16 decode linears (default: the library's default)")
    ap.add_argument("--decode-m", default="1,16", help="token counts of the decode suite")
    ap.add_argument("--suite-pdl", type=int, default=0,
                    help="decode suite: launch the chain with programmatic dependent launch (adds \"pdl\": 1 to the line)")
    ap.add_argument("--decode-shapes", default="", help="restrict the decode suite, e.g. 8192x28672,4096x4096 (NxK)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    POOL_SETS = max(2, args.pool_sets)
    FUSE = bool(args.fuse)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        if args.decode_kernel != "default":
            from mindpipe_b200 import ops as _ops
            _ops.set_decode_kernel(args.decode_kernel)
        if not args.suite_only:
            run_ours(args, rank, world, local_rank)
        if args.suite and rank == 0:
            run_suite(args, local_rank)


if __name__ == "__main__":
    main()
