"""GPU parity of the tcgen05 int8 GEMM (through the C ABI).

int32 accumulators: bit-exact against exact integer matmul of the same codes
(computed in float64, exact below 2^53).  fp16 outputs: relative Frobenius
error <= 1e-2 against the reference's fake-quant forward as restated by the
oracle (``SmoothQuantLinear.forward``); against the same-arithmetic int
pipeline of the oracle the outputs agree to fp16 rounding.
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


def exact_acc(qx, qw):
    return (qx.astype(np.float64) @ qw.astype(np.float64).T).astype(np.int64)


def rand_i8(shape, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(-127, 128, size=shape, dtype=np.int8)


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 128),      # one tile, one k-block
    (128, 128, 512),      # k loop, ring wrap-around (4 k-blocks, 6 stages)
    (128, 256, 1024),     # 8 k-blocks: every stage reused
    (256, 384, 256),      # several tiles per CTA? no: several CTAs
    (100, 72, 144),       # ragged M, N, K (K % 16 == 0)
    (1, 8, 16),           # smallest legal problem
    (300, 1000, 4096),
])
def test_int32_accumulators_bit_exact(m, n, k):
    from mindpipe_b200 import ops
    qx, qw = rand_i8((m, k), 1), rand_i8((n, k), 2)
    acc = ops.w8a8_gemm_i32(dev(qx), dev(qw))
    ops.check_device_errors()
    assert np.array_equal(acc.cpu().numpy().astype(np.int64), exact_acc(qx, qw))


def test_int32_many_tiles_per_cta_and_both_tmem_buffers():
    """More tiles than SMs: every CTA walks several tiles, alternating accumulator buffers."""
    from mindpipe_b200 import ops
    m, n, k = 2048, 4096, 256          # 16 x 16 = 256 tiles of 128 x 256 over 148 CTAs
    qx, qw = rand_i8((m, k), 3), rand_i8((n, k), 4)
    acc = ops.w8a8_gemm_i32(dev(qx), dev(qw))
    ops.check_device_errors()
    assert np.array_equal(acc.cpu().numpy().astype(np.int64), exact_acc(qx, qw))


@pytest.mark.parametrize("m,n,k", [
    (2304, 2304, 128),     # 9 x 9 pair tiles on 74 CTA pairs: one k-block, some pairs take two tiles
    (2100, 2500, 384),     # ragged M and N: the second CTA of the last pair row is partly / fully out of range
    (4096, 4096, 1024),    # 256 pair tiles, ring of 6 stages reused across tiles, both accumulator buffers
])
def test_int32_cta_pair_form_bit_exact(m, n, k):
    """Shapes with >= 74 tiles of 256 x 256 run the two-CTA (cta_group::2) kernel."""
    from mindpipe_b200 import ops
    qx, qw = rand_i8((m, k), 5), rand_i8((n, k), 6)
    acc = ops.w8a8_gemm_i32(dev(qx), dev(qw))
    ops.check_device_errors()
    assert np.array_equal(acc.cpu().numpy().astype(np.int64), exact_acc(qx, qw))


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 1024, 2048), (64, 4096, 1024), (200, 512, 4096), (16, 4096, 14336)])
def test_split_k_small_batches_change_no_bit(m, n, k):
    """Few output tiles: K is cut into slices whose int32 partial tiles are added by a second kernel.
    Integer sums are order independent and the scale epilogue is the same arithmetic, so the result is
    bit-identical to the unsplit kernel (called with a null workspace)."""
    from mindpipe_b200 import _lib, ops
    lib = _lib.load()
    assert lib.mp_w8a8_gemm_workspace_bytes(m, n, k) > 0
    qx, qw = dev(rand_i8((m, k), 7)), dev(rand_i8((n, k), 8))
    rng = np.random.default_rng(9)
    sx = dev(rng.uniform(0.01, 0.1, m).astype(np.float32))
    sw = dev(rng.uniform(0.001, 0.01, n).astype(np.float32))
    bias = dev(rng.standard_normal(n).astype(np.float16))
    y = ops.w8a8_gemm(qx, sx, qw, sw, bias)
    ops.check_device_errors()
    y1 = torch.empty_like(y)
    st = lib.mp_w8a8_gemm(qx.data_ptr(), sx.data_ptr(), qw.data_ptr(), sw.data_ptr(), bias.data_ptr(), y1.data_ptr(),
                          m, n, k, ops._error_word(qx.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    ops.check_device_errors()
    assert torch.equal(y, y1)
    acc = exact_acc(qx.cpu().numpy(), qw.cpu().numpy()).astype(np.float32)
    want = (acc * sx.cpu().numpy()[:, None] * sw.cpu().numpy()[None, :] + bias.cpu().numpy().astype(np.float32))
    assert O.rel_frobenius(y.cpu().numpy(), want.astype(np.float16)) <= 1e-3


def _w8a8_case(m, n, k, seed, bias=False):
    from mindpipe_b200 import ops
    x = synth.outlier_activation(m, k, seed=seed, index=100).numpy()
    w = synth.normal_weight(n, k, seed=seed, index=0).numpy()
    b = (synth.normal_activation(1, n, seed=seed, index=7).numpy()[0] * np.float16(0.1)).astype(np.float16) if bias else None
    wfake, qw, sw = O.absmax_quant_last_dim(w)
    qx_d, sx_d, _ = ops.act_quant_per_token(dev(x))
    qw_d, sw_d, _ = ops.act_quant_per_token(dev(w))            # per-channel weights: the same arithmetic
    assert np.array_equal(qw_d.cpu().numpy(), qw)
    y = ops.w8a8_gemm(qx_d, sx_d, qw_d, sw_d, None if b is None else dev(b))
    ops.check_device_errors()
    return x, wfake, qw, sw, b, qx_d, sx_d, y.cpu().numpy()


@pytest.mark.parametrize("m,n,k", [(64, 128, 256), (333, 520, 1024), (512, 1024, 4096)])
def test_w8a8_fp16_output_vs_reference_forward(m, n, k):
    x, wfake, qw, sw, b, qx_d, sx_d, y = _w8a8_case(m, n, k, seed=m, bias=True)
    ref = O.smoothquant_linear_forward(x, wfake, b)                 # the reference's fake-quant forward
    assert O.rel_frobenius(y, ref) <= TOL
    same = O.w8a8_int_forward(qx_d.cpu().numpy(), sx_d.cpu().numpy(), qw, sw, b)
    assert O.rel_frobenius(y, same) <= 1e-3


def test_w8a8_cfg3_attention_proj_full_size():
    """Config 3, 4096x4096 at M=4096: int32 accumulators on a row sample, fp16 output on all rows."""
    from mindpipe_b200 import ops
    m = n = k = 4096
    x, wfake, qw, sw, b, qx_d, sx_d, y = _w8a8_case(m, n, k, seed=0)
    acc = ops.w8a8_gemm_i32(qx_d, dev(qw))
    ops.check_device_errors()
    qx = qx_d.cpu().numpy()
    _, codes, _ = O.absmax_quant_last_dim(x)
    assert np.array_equal(qx, codes)                                # int8 activations bit-exact
    rows = np.random.default_rng(0).choice(m, 256, replace=False)
    assert np.array_equal(acc.cpu().numpy()[rows].astype(np.int64), exact_acc(qx[rows], qw))
    ref = O.smoothquant_linear_forward(x[rows], wfake)
    assert O.rel_frobenius(y[rows], ref) <= TOL


@pytest.mark.parametrize("n,k", [(1024, 4096), (14336, 4096), (4096, 14336)])
def test_w8a8_cfg3_other_shapes_row_sample(n, k):
    m = 4096
    x, wfake, qw, sw, b, qx_d, sx_d, y = _w8a8_case(m, n, k, seed=1)
    rows = np.random.default_rng(1).choice(m, 64, replace=False)
    ref = O.smoothquant_linear_forward(x[rows], wfake)
    assert O.rel_frobenius(y[rows], ref) <= TOL


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (16, 1024, 14336), (300, 512, 1024), (4096, 1024, 4096)])
def test_w8a8_linear_under_programmatic_dependent_launch_same_bits(m, n, k):
    """Per-token quant -> GEMM (-> split-K reduce for small batches), each launch allowed to be scheduled before
    its predecessor has finished (every kernel waits on the device): same bits as the serialised launches, eagerly
    and as a replayed CUDA graph of three forwards."""
    from mindpipe_b200 import _lib, ops
    from mindpipe_b200.modules import SmoothQuantLinear
    lin = torch.nn.Linear(k, n, bias=True).half().cuda()
    mod = SmoothQuantLinear.from_float(lin, quantize_output=(m == 300))
    x = synth.outlier_activation(m, k, seed=17).cuda()
    base = mod(x)
    lib = _lib.load()
    before = lib.mp_set_programmatic_launch(1)
    try:
        for _ in range(3):
            assert torch.equal(mod(x), base)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            mod(x)
            with torch.cuda.graph(graph, stream=side):
                outs = [mod(x) for _ in range(3)]
            graph.replay()
            graph.replay()
        side.synchronize()
        for o in outs:
            assert torch.equal(o, base)
    finally:
        lib.mp_set_programmatic_launch(before)
    ops.check_device_errors()


def test_smoothquant_linear_module_matches_reference_golden(golden):
    """SmoothQuantLinear twin (int8 weights) vs the reference module's outputs on the golden case."""
    from mindpipe_b200 import ops
    from mindpipe_b200.modules import SmoothQuantLinear, W8A8DynamicLinearMethod
    g = golden("w8a8_small.npz")
    lin = torch.nn.Linear(256, 16, bias=True).half().cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(g["w"]))
        lin.bias.copy_(dev(g["bias"]))
    m = SmoothQuantLinear.from_float(lin)
    assert m.weight.dtype == torch.int8
    assert np.array_equal(m.dequantize().cpu().numpy(), g["w_fake"])      # values (int8 drops the sign of -0.0)
    y = m(dev(g["x"]))
    ops.check_device_errors()
    assert O.rel_frobenius(y.cpu().numpy(), g["y"]) <= TOL
    mq = SmoothQuantLinear.from_float(lin, quantize_output=True)
    assert O.rel_frobenius(mq(dev(g["x"])).cpu().numpy(), g["y_outq"]) <= TOL
    y3 = m(dev(g["x"]).reshape(1, 7, 256))
    assert y3.shape == (1, 7, 16)
    # linear-method entry: tensor input, (codes, scale) tuple input, return_scale, int32 passthrough
    method = W8A8DynamicLinearMethod()
    layer = type("Layer", (), {})()
    layer.weight, layer.weight_scale = m.weight, m.weight_scale.clone()
    method.process_weights_after_loading(layer)
    out = method.apply(layer, dev(g["x"]), bias=m.bias)
    assert torch.equal(out, y)
    q, s, _ = ops.act_quant_per_token(dev(g["x"]))
    layer._ascend_quant_config = {"output_dtype": torch.float16, "return_scale": True}
    out2, s2 = method.apply(layer, (q, s), bias=m.bias)
    assert torch.equal(out2, y) and torch.equal(s2, s)
    layer._ascend_quant_config = {"output_dtype": torch.int32}
    acc = method.apply(layer, (q, s))
    assert np.array_equal(acc.cpu().numpy(), O.int32_accumulate(q.cpu().numpy(), m.weight.cpu().numpy()))


def test_omniquant_affine_quant_bit_exact(golden):
    """Asymmetric per-row quantiser vs the reference's UniformAffineQuantizer (golden) and the oracle."""
    from mindpipe_b200 import ops
    g = golden("omniquant_small.npz")
    for key in ("x", "w"):
        q, s, z, rs, f = ops.affine_quant_per_row(dev(g[key]), want_fake=True)
        fake, codes, sc, zp = O.affine_quant_last_dim(g[key])
        assert np.array_equal(q.cpu().numpy(), codes)
        assert np.array_equal(s.cpu().numpy(), sc.astype(np.float32).reshape(-1))
        assert np.array_equal(z.cpu().numpy(), zp.astype(np.float32).reshape(-1))
        assert np.array_equal(rs.cpu().numpy(), codes.astype(np.int64).sum(axis=1).astype(np.int32))
        assert np.array_equal(f.cpu().numpy(), g[key + "_fake"])
    x = synth.outlier_activation(300, 4096, seed=3).numpy()
    q, s, z, rs, _ = ops.affine_quant_per_row(dev(x))
    _, codes, sc, zp = O.affine_quant_last_dim(x)
    assert np.array_equal(q.cpu().numpy(), codes) and np.array_equal(z.cpu().numpy(), zp.astype(np.float32).reshape(-1))


@pytest.mark.parametrize("m,n,k", [(7, 16, 256), (300, 520, 1024), (1024, 1024, 4096)])
def test_omniquant_quantlinear_twin(golden, m, n, k):
    from mindpipe_b200 import ops
    from mindpipe_b200.modules import QuantLinear
    if (m, n, k) == (7, 16, 256):
        g = golden("omniquant_small.npz")
        x, w, b, ref = g["x"], g["w"], g["bias"], g["y"]               # outputs of the reference module itself
    else:
        x = synth.outlier_activation(m, k, seed=m).numpy()
        w = synth.normal_weight(n, k, seed=m, index=0).numpy()
        b = None
        ref = O.omniquant_linear_forward(x, w)
    lin = torch.nn.Linear(k, n, bias=b is not None).half().cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(w))
        if b is not None:
            lin.bias.copy_(dev(b))
    mod = QuantLinear(lin, weight_quant_params={"n_bits": 8, "symmetric": False, "dynamic_method": "per_channel"},
                      act_quant_params={"n_bits": 8, "symmetric": False, "dynamic_method": "per_token"})
    assert np.array_equal(mod.dequantize().cpu().numpy(), O.affine_quant_last_dim(w)[0])
    y = mod(dev(x))
    ops.check_device_errors()
    assert O.rel_frobenius(y.cpu().numpy(), ref) <= TOL
    # exact integer identity of the zero-point correction, checked through a unit-scale call
    q, s, z, rs, _ = ops.affine_quant_per_row(dev(x))
    ones_m = torch.ones_like(s)
    ones_n = torch.ones_like(mod.scales)
    yi = ops.w8a8_affine_gemm(q[:4].contiguous(), ones_m[:4].contiguous(), z[:4].contiguous(), rs[:4].contiguous(),
                              mod.weight[:8].contiguous(), ones_n[:8].contiguous(), mod.zeros[:8].contiguous(),
                              mod.weight_rowsum[:8].contiguous())
    exact = (q[:4].cpu().numpy().astype(np.int64) - z[:4].cpu().numpy().astype(np.int64)[:, None]) @ \
            (mod.weight[:8].cpu().numpy().astype(np.int64) - mod.zeros[:8].cpu().numpy().astype(np.int64)[:, None]).T
    assert np.allclose(yi.float().cpu().numpy(), exact.astype(np.float16).astype(np.float32), rtol=2e-3, atol=1.0)
