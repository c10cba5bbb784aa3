"""GPU parity of the W8A8 pieces against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

from mindpipe_b200 import synth
from oracle import pseudo_quant as O

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def _check_quant(x16: np.ndarray):
    from mindpipe_b200 import ops
    q, s, f = ops.act_quant_per_token(dev(x16), want_codes=True, want_fake=True)
    fake, codes, sc = O.absmax_quant_last_dim(x16)
    assert np.array_equal(q.cpu().numpy(), codes)                                  # int8 codes bit-exact
    assert np.array_equal(s.cpu().numpy(), sc.astype(np.float32).reshape(s.shape))  # fp16 scale, widened
    assert np.array_equal(bits(f.cpu().numpy()), bits(fake))


def test_act_quant_golden(golden):
    g = golden("w8a8_small.npz")
    _check_quant(g["x"])            # includes an all-zero token and x20 outlier channels
    from mindpipe_b200 import ops
    _, _, f = ops.act_quant_per_token(dev(g["x"]), want_codes=False, want_fake=True)
    assert np.array_equal(bits(f.cpu().numpy()), bits(g["x_fake"]))
    _, _, wf = ops.act_quant_per_token(dev(g["w"]), want_codes=False, want_fake=True)
    assert np.array_equal(bits(wf.cpu().numpy()), bits(g["w_fake"]))   # per-channel weights: same arithmetic


@pytest.mark.parametrize("m,k", [(1, 8), (3, 64), (5, 1000), (17, 4096), (4, 14336), (2, 28672)])
def test_act_quant_shapes(m, k):
    _check_quant(synth.outlier_activation(m, k, seed=m, index=k).numpy())


def test_act_quant_cfg3_full_size():
    """Config 3: X[4096,4096] fp16 N(0,1), 1 % of channels x20, per-token dynamic int8."""
    _check_quant(synth.outlier_activation(4096, 4096, seed=0, index=100).numpy())


@pytest.mark.parametrize("k", [4096, 8192])
@pytest.mark.parametrize("amax", [1e-6, 1e-4, 0.004, 0.00775, 0.0079, 0.0371, 1.0, 1.9995, 3.1416, 77.25, 1000.0, 65504.0])
def test_act_quant_every_fp16_value(amax, k):
    """Every finite fp16 value of magnitude <= amax, quantised against the scale amax pins: the kernel's
    division-free routes (packed f16x2 for ordinary scales, fp32 for tiny ones) must give the code the IEEE
    division gives, for all of them."""
    allv = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    a16 = np.float16(amax)
    vals = allv[np.isfinite(allv) & (np.abs(allv.astype(np.float32)) <= np.float32(a16))]
    per_row = k - 1
    rows = -(-vals.size // per_row)
    x = np.zeros((rows, k), np.float16)
    x[:, 0] = a16
    flat = np.zeros(rows * per_row, np.float16)
    flat[:vals.size] = vals
    x[:, 1:] = flat.reshape(rows, per_row)
    _check_quant(x)


def test_act_quant_3d_and_empty():
    from mindpipe_b200 import ops
    x = synth.normal_activation(6, 256, seed=1).reshape(2, 3, 256).cuda()
    q, s, _ = ops.act_quant_per_token(x)
    assert q.shape == (2, 3, 256) and s.shape == (2, 3)
    q, s, _ = ops.act_quant_per_token(torch.zeros(0, 64, dtype=torch.float16, device="cuda"))
    assert q.shape == (0, 64) and s.shape == (0,)


@pytest.mark.parametrize("m,h", [(5, 256), (33, 4096), (4, 8192), (2, 14336)])
def test_add_rmsnorm_quant_vs_composed_oracle(m, h):
    """Fused residual add + RMSNorm + quant.  The new residual is bit-exact; codes may differ by one
    step where the fp32 reduction order moves rsqrt by an ulp (the reference has no CPU statement
    of this fused op, so the oracle is a composition of its pieces)."""
    from mindpipe_b200 import ops
    x = synth.normal_activation(m, h, seed=1, index=1).numpy()
    res = synth.outlier_activation(m, h, seed=1, index=2).numpy()
    gamma = (1.0 + 0.1 * synth.normal_activation(1, h, seed=1, index=3).numpy()[0]).astype(np.float16)
    res_d = dev(res.copy())
    q, s = ops.add_rmsnorm_quant(dev(x), res_d, dev(gamma), 1e-5)
    r_ref, codes, sc = O.add_rmsnorm_quant(x, res, gamma, 1e-5)
    assert np.array_equal(bits(res_d.cpu().numpy()), bits(r_ref))
    diff = np.abs(q.cpu().numpy().astype(np.int32) - codes.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3
    assert np.allclose(s.cpu().numpy(), sc.astype(np.float32).reshape(-1), rtol=2e-3)
    # the pair feeds the W8A8 linear directly
    from mindpipe_b200.modules import SmoothQuantLinear
    lin = torch.nn.Linear(h, 64, bias=False).half().cuda()
    mod = SmoothQuantLinear.from_float(lin)
    y = mod((q, s))
    assert y.shape == (m, 64)
    ops.check_device_errors()
