"""The tcgen05 decode kernel (dequantised weights as the tensor-memory operand) against the oracle's
F.linear(x, Wdq) (awq/quantize/quantizer.py:109-130 with the weights of :63-105) and against the
mma.sync kernel, through the C ABI."""
import numpy as np
import pytest
import torch

from mindpipe_b200 import synth
from oracle import pseudo_quant as O

pytestmark = pytest.mark.gpu
TOL = 1e-2          # relative Frobenius error of fp16 outputs
TOL_KERNELS = 2e-3  # two fp32-accumulating kernels on identical fp16 weights: summation order + one fp16 rounding


@pytest.fixture
def umma():
    from mindpipe_b200 import ops
    prev = ops.set_decode_kernel("umma")
    yield ops
    ops.check_device_errors()
    ops.set_decode_kernel(prev)


def _case(ops, n, k, m, group=128, seed=0, bias=False):
    w = synth.normal_weight(n, k, seed=seed, index=1).numpy()
    x = synth.normal_activation(m, k, seed=seed, index=2).numpy()
    b = (synth.normal_activation(1, n, seed=seed, index=3).numpy()[0] * np.float16(0.1)).astype(np.float16) if bias else None
    packed, scale, zero, _ = ops.w4a16_quantize(torch.from_numpy(w).cuda(), group)
    wdq = ops.w4a16_dequant(packed, scale, zero, n, k).cpu().numpy()
    sz = ops.w4a16_prepare(scale, zero, k)
    xd = torch.from_numpy(x).cuda()
    bd = None if b is None else torch.from_numpy(b).cuda()
    y = ops.w4a16_linear_decode(xd, packed, sz, bd)
    torch.cuda.synchronize()
    ref = O.linear_f16(x, wdq, b)
    return y, ref, (xd, packed, sz, bd)


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 15, 16])
def test_umma_decode_all_row_counts(umma, m):
    y, ref, _ = _case(umma, 256, 1024, m)
    assert y.shape == ref.shape
    assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("n,k,group", [(8, 128, 128), (40, 256, 64), (72, 384, 32), (264, 1280, 128), (64, 256, 256),
                                       (128, 1024, 512), (136, 384, 64)])
def test_umma_decode_ragged_shapes_and_groups(umma, n, k, group):
    for m in (1, 16):
        y, ref, _ = _case(umma, n, k, m, group=group, bias=True)
        assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008), (12288, 4096)])
@pytest.mark.parametrize("m", [1, 16])
def test_umma_decode_llama_shapes_and_agreement_with_mma_sync(umma, n, k, m):
    y, ref, (xd, packed, sz, bd) = _case(umma, n, k, m, seed=1)
    assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL
    umma.set_decode_kernel("mma_sync")
    y2 = umma.w4a16_linear_decode(xd, packed, sz, bd)
    umma.set_decode_kernel("umma")
    # M > 8 on the mma.sync kernel multiplies the same fp16 weights: only the summation order differs
    assert O.rel_frobenius(y.cpu().numpy(), y2.cpu().numpy()) <= TOL_KERNELS


def test_umma_decode_repeat_calls_identical(umma):
    y0, _, (xd, packed, sz, bd) = _case(umma, 512, 8192, 16, seed=3)
    for _ in range(5):
        assert torch.equal(umma.w4a16_linear_decode(xd, packed, sz, bd), y0)   # fixed-order cluster sum


def test_umma_decode_linearity_70b_shape(umma):
    """Size-independent check at a 70B shape: f(2x) = 2 f(x) -- scaling by two commutes with every rounding
    except that of an output in the fp16 subnormal range, hence one subnormal step (2^-24) of slack."""
    n, k = 8192, 8192
    w = synth.normal_weight(n, k, seed=5, index=1).cuda()
    packed, scale, zero, _ = umma.w4a16_quantize(w, 128)
    sz = umma.w4a16_prepare(scale, zero, k)
    x = synth.normal_activation(16, k, seed=5, index=2).cuda()
    y1 = umma.w4a16_linear_decode(x, packed, sz)
    y2 = umma.w4a16_linear_decode(x * 2, packed, sz)
    assert (y2.float() - 2 * y1.float()).abs().max().item() <= 2.0 ** -24
    rows = torch.arange(0, n, 257, device="cuda")
    wdq = umma.w4a16_dequant(packed, scale, zero, n, k)[rows].float()
    ref = (x.float() @ wdq.T).cpu().numpy()
    assert O.rel_frobenius(y1[:, rows].float().cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("kind", ["umma", "mma_sync"])
def test_back_to_back_launches_under_programmatic_dependent_launch(kind):
    """A chain of decode launches sharing one workspace, each allowed to start fetching its weights while the
    previous one finishes (mp_set_programmatic_launch): same bits as the serialised chain."""
    from mindpipe_b200 import _lib, ops
    prev_kind = ops.set_decode_kernel(kind)
    lib = _lib.load()
    try:
        shapes = [(1024, 2048), (512, 4096), (2048, 1024)]
        x = {k: synth.normal_activation(16, k, seed=9, index=k).cuda() for k in {k for _, k in shapes}}
        mods = []
        for i, (n, k) in enumerate(shapes):
            w = synth.normal_weight(n, k, seed=9, index=i).cuda()
            packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
            mods.append((packed, ops.w4a16_prepare(scale, zero, k), k))
        ws = ops.new_workspace(max(ops.w4a16_decode_workspace_bytes(16, n, k) for n, k in shapes), "cuda")

        def chain():
            outs = []
            for _ in range(3):
                for packed, sz, k in mods:
                    outs.append(ops.w4a16_linear_decode(x[k], packed, sz, workspace=ws))
            torch.cuda.synchronize()
            return outs

        base = chain()
        before = lib.mp_set_programmatic_launch(1)
        try:
            overlapped = chain()
        finally:
            lib.mp_set_programmatic_launch(before)
        ops.check_device_errors()
        for a, b in zip(base, overlapped):
            assert torch.equal(a, b)
    finally:
        ops.set_decode_kernel(prev_kind)


# ---- 17..64 rows: the same kernel with a 32- or 64-token activation tile, chosen per call ----
def _wide_case(ops, n, k, m, group=128, seed=0, bias=False):
    w = synth.normal_weight(n, k, seed=seed, index=1).numpy()
    x = synth.normal_activation(m, k, seed=seed, index=2).numpy()
    b = (synth.normal_activation(1, n, seed=seed, index=3).numpy()[0] * np.float16(0.1)).astype(np.float16) if bias else None
    packed, scale, zero, _ = ops.w4a16_quantize(torch.from_numpy(w).cuda(), group)
    wdq = ops.w4a16_dequant(packed, scale, zero, n, k)
    sz = ops.w4a16_prepare(scale, zero, k)
    xd = torch.from_numpy(x).cuda()
    bd = None if b is None else torch.from_numpy(b).cuda()
    ws = ops.new_workspace(20 << 20, "cuda")                # 64-token partial tiles: 16 KB + 296 x 2 x 32 KB
    y = ops.w4a16_linear_decode(xd, packed, sz, bd, workspace=ws, options=ops.decode_options(kernel="umma"))
    torch.cuda.synchronize()
    return y, O.linear_f16(x, wdq.cpu().numpy(), b), (xd, packed, sz, bd, ws, wdq)


@pytest.mark.parametrize("m", [17, 24, 32, 33, 48, 64])
def test_umma_wide_tile_all_row_counts(m):
    from mindpipe_b200 import ops
    y, ref, _ = _wide_case(ops, 256, 1024, m, bias=True)
    ops.check_device_errors()
    assert y.shape == ref.shape
    assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("n,k,group", [(40, 256, 64), (72, 384, 32), (264, 1280, 128), (128, 1024, 512), (4104, 512, 128)])
def test_umma_wide_tile_ragged_shapes_and_groups(n, k, group):
    from mindpipe_b200 import ops
    for m in (20, 64):
        y, ref, _ = _wide_case(ops, n, k, m, group=group, bias=True)
        ops.check_device_errors()
        assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("n,k", [(4096, 4096), (22016, 4096), (4096, 11008)])
@pytest.mark.parametrize("m", [32, 64])
def test_umma_wide_tile_llama_shapes_and_agreement_with_the_gemm(n, k, m):
    from mindpipe_b200 import ops
    y, ref, (xd, packed, sz, bd, ws, _) = _wide_case(ops, n, k, m, seed=1)
    ops.check_device_errors()
    assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL
    y2 = ops.w4a16_linear_prefill(xd, packed, sz, bd)      # same fp16 weights, another summation order
    assert O.rel_frobenius(y.cpu().numpy(), y2.cpu().numpy()) <= TOL_KERNELS
    for _ in range(3):                                      # fixed-order fix-up: identical from run to run
        again = ops.w4a16_linear_decode(xd, packed, sz, bd, workspace=ws, options=ops.decode_options(kernel="umma"))
        assert torch.equal(again, y)
    assert int(ws[:16384].view(torch.int32).abs().sum().item()) == 0       # arrival counters re-armed


@pytest.mark.parametrize("m", [32, 64])
def test_umma_wide_tile_one_hot_rows_bit_for_bit(m):
    from mindpipe_b200 import ops
    n, k = 384, 1024
    w = synth.normal_weight(n, k, seed=4, index=1).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    wdq = ops.w4a16_dequant(packed, scale, zero, n, k)
    sz = ops.w4a16_prepare(scale, zero, k)
    ws = ops.new_workspace(20 << 20, "cuda")
    for k0 in (0, 5, 130, k - m):
        x = torch.zeros((m, k), dtype=torch.float16, device="cuda")
        x[torch.arange(m), k0 + torch.arange(m)] = 1.0
        y = ops.w4a16_linear_decode(x, packed, sz, workspace=ws, options=ops.decode_options(kernel="umma"))
        assert torch.equal(y.view(torch.int16), wdq[:, k0:k0 + m].t().contiguous().view(torch.int16))
    ops.check_device_errors()
