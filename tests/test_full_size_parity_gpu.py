"""Parity at the full sizes of the 70B-shaped W4A16 linears and of the Mixtral-shaped W8A8 MoE layer, and
bit-exactness of the dequantised weight INSIDE every forward kernel (through the C ABI).

* W4A16 forward = F.linear(x, pseudo_quantize_tensor(W)) (awq/quantize/quantizer.py:63-130): group
  quantisation is per output row, so the oracle quantises a seeded sample of rows only and the matching
  output columns are compared (relative Frobenius error <= 1e-2), for every kernel choice, so that the
  grids these shapes get (halved K-split clusters, the persistent tcgen05 grid, the split-K tensor-core
  GEMM above 16 rows) are the ones checked.
* MoE = SmoothQuantPackedMoeExperts.forward (smoothquant/fake_quant.py:165-191): every output row depends
  on one token and its two experts, so the oracle runs on a seeded sample of tokens.
* One-hot activation rows return single weights: y[m, n] must equal f16((u - z) * s) bit for bit.
"""
import numpy as np
import pytest
import torch

from mindpipe_b200 import synth
from oracle import pseudo_quant as O

pytestmark = pytest.mark.gpu
TOL = 1e-2          # relative Frobenius error of fp16 outputs


@pytest.fixture(scope="module")
def ops():
    from mindpipe_b200 import ops as _ops
    yield _ops
    _ops.check_device_errors()


# ------------------------------------------------------------------ config 5: Llama-2-70B-shaped linears
_CFG5 = {}


def _cfg5_case(ops, n, k):
    """Weights of one 70B-shaped linear (seeded), quantised on the GPU, plus the oracle's dequantised
    weights for 256 sampled rows."""
    key = (n, k)
    if key not in _CFG5:
        _CFG5.clear()                                      # one shape resident at a time
        w = synth.normal_weight(n, k, seed=50, index=n % 97)
        packed, scale, zero, _ = ops.w4a16_quantize(w.cuda(), 128)
        sz = ops.w4a16_prepare(scale, zero, k)
        rows = np.sort(np.random.default_rng(n * 31 + k).choice(n, 256, replace=False))
        wdq_rows, _, _, u = O.w4_group_asym_quantize(w[rows].numpy(), 128)
        # the sampled rows' packed codes are the oracle's (bit-exact), so the forward is compared on the
        # same weights the reference would multiply with
        assert np.array_equal(packed[torch.from_numpy(rows).cuda()].cpu().numpy(), O.pack_int4_unsigned(u))
        _CFG5[key] = (packed, sz, rows, wdq_rows)
    return _CFG5[key]


@pytest.mark.parametrize("kernel", ["mma_sync", "umma", "auto"])
@pytest.mark.parametrize("m", [1, 8, 64])
@pytest.mark.parametrize("n,k", [(28672, 8192), (8192, 28672), (1024, 8192), (8192, 8192)])
def test_cfg5_llama2_70b_shapes_row_sample(ops, n, k, m, kernel):
    packed, sz, rows, wdq_rows = _cfg5_case(ops, n, k)
    x = synth.normal_activation(m, k, seed=51, index=m)
    if m <= 16:
        ws = ops.new_workspace(max(ops.w4a16_decode_workspace_bytes(m, n, k), 5 << 20), "cuda")
        y = ops.w4a16_linear_decode(x.cuda(), packed, sz, workspace=ws, options=ops.decode_options(kernel=kernel))
    else:
        if kernel != "auto":
            pytest.skip("above 16 rows the dispatching entry picks the split-K tensor-core GEMM")
        y = ops.w4a16_linear(x.cuda(), packed, sz)
    ops.check_device_errors()
    ref = O.linear_f16(x.numpy(), wdq_rows)
    got = y[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    assert O.rel_frobenius(got, ref) <= TOL


# ------------------------------------------------------------------ config 4: Mixtral-8x7B-shaped MoE layer
def test_cfg4_mixtral_moe_full_size_token_sample(ops):
    from mindpipe_b200.modules import SmoothQuantPackedMoeExperts
    shape = synth.MIXTRAL_8X7B
    parts, fake = [], {}
    hs = synth.normal_activation(shape.tokens, shape.hidden, seed=0)
    logits = synth.router_logits(shape.tokens, shape.num_experts, seed=0)
    idx, wts = ops.moe_router_topk(logits.cuda(), shape.top_k)
    sample = np.sort(np.random.default_rng(4).choice(shape.tokens, 64, replace=False))
    idx_s = idx.cpu().numpy()[sample].astype(np.int64)
    for e in range(shape.num_experts):                     # expert by expert: bounded host and device memory
        gu, dn = synth.moe_weights(shape, seed=0, experts=range(e, e + 1))
        parts.append(SmoothQuantPackedMoeExperts(gu.cuda(), dn.cuda(), torch.nn.SiLU(), expert_range=(e, e + 1),
                                                 num_experts=shape.num_experts))
        if (idx_s == e).any():                             # fake-quantised weights of the experts the sample hits
            fake[e] = (O.absmax_quant_last_dim(gu[0].numpy())[0], O.absmax_quant_last_dim(dn[0].numpy())[0])
    mod = parts[0]
    mod.gate_up_proj = torch.cat([p.gate_up_proj for p in parts])
    mod.gate_up_proj_scale = torch.cat([p.gate_up_proj_scale for p in parts])
    mod.down_proj = torch.cat([p.down_proj for p in parts])
    mod.down_proj_scale = torch.cat([p.down_proj_scale for p in parts])
    mod.expert_range = (0, shape.num_experts)
    del parts
    out = mod(hs.cuda(), idx, wts)
    ops.check_device_errors()
    # the reference forward on the sampled tokens only (experts the sample never hits stay zero)
    guf = np.zeros((shape.num_experts, 2 * shape.ffn, shape.hidden), dtype=np.float16)
    dnf = np.zeros((shape.num_experts, shape.hidden, shape.ffn), dtype=np.float16)
    for e, (g, d) in fake.items():
        guf[e], dnf[e] = g, d
    ref = O.moe_experts_forward(hs.numpy()[sample], idx_s, wts.cpu().numpy()[sample], guf, dnf)
    got = out[torch.from_numpy(sample).cuda()].cpu().numpy()
    assert O.rel_frobenius(got, ref) <= TOL


# ------------------------------------------------------------------ dequantised weights inside the forward kernels
def _one_hot_case(ops, n, k, group, seed):
    w = synth.normal_weight(n, k, seed=seed, index=1).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, group)
    wdq = ops.w4a16_dequant(packed, scale, zero, n, k)           # bit-exact against the oracle elsewhere
    return packed, ops.w4a16_prepare(scale, zero, k), wdq


def _identity_rows(m, k, k0):
    x = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    x[torch.arange(m), k0 + torch.arange(m)] = 1.0
    return x


@pytest.mark.parametrize("kernel,m", [("mma_sync", 16), ("mma_sync", 9), ("umma", 16), ("umma", 3), ("mma_sync", 8),
                                      ("mma_sync", 1)])
def test_forward_kernels_multiply_with_the_reference_weights_bit_for_bit(ops, kernel, m):
    """x = rows of the identity, so y[i, n] is the kernel's own weight (n, k0 + i) rounded to fp16.  The
    9-16 token mma.sync kernel and the tcgen05 kernel expand every weight to f16((u - z) * s) before the
    tensor core; the mma.sync kernel for up to 8 tokens applies s and z to group sums in fp32, which for a
    single weight is s * (u - z) rounded to fp16 once -- the same value (sums of several weights differ
    from the reference by its per-weight rounding, inside the 1e-2 bound checked elsewhere)."""
    n, k = 384, 1024
    packed, sz, wdq = _one_hot_case(ops, n, k, 128, seed=4)
    ws = ops.new_workspace(5 << 20, "cuda")
    for k0 in (0, 5, 130, k - m):
        y = ops.w4a16_linear_decode(_identity_rows(m, k, k0), packed, sz, workspace=ws,
                                    options=ops.decode_options(kernel=kernel))
        assert torch.equal(y.view(torch.int16), wdq[:, k0:k0 + m].t().contiguous().view(torch.int16))


def test_register_streaming_decode_kernels_bit_for_bit(ops):
    """Shapes the TMA-fed kernel does not take (a group size that neither divides nor is a multiple of 256)
    go to the cluster kernel; an explicit K split goes to the workspace kernel."""
    n, k, group = 264, 1536, 384
    packed, sz, wdq = _one_hot_case(ops, n, k, group, seed=6)
    for m in (4, 16):
        for k0 in (0, 383, k - m):
            x = _identity_rows(m, k, k0)
            ref = wdq[:, k0:k0 + m].t().contiguous().view(torch.int16)
            assert torch.equal(ops.w4a16_linear_decode(x, packed, sz).view(torch.int16), ref)
            assert torch.equal(ops.w4a16_linear_decode(x, packed, sz, k_split=3).view(torch.int16), ref)


@pytest.mark.parametrize("m,n,k", [(64, 512, 1024), (128, 256, 512), (200, 512, 1024), (320, 512, 512)])
def test_prefill_kernels_bit_for_bit(ops, m, n, k):
    """The tcgen05 GEMM in its one-CTA forms (up to 128 and up to 256 rows, with and without split-K) and in
    its CTA-pair form (more than 256 rows): identity rows return the dequantised weights exactly."""
    packed, sz, wdq = _one_hot_case(ops, n, k, 128, seed=8)
    for k0 in (0, k - m):
        y = ops.w4a16_linear_prefill(_identity_rows(m, k, k0), packed, sz)
        assert torch.equal(y.view(torch.int16), wdq[:, k0:k0 + m].t().contiguous().view(torch.int16))
