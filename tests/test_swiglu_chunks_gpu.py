"""The dense chunked gate/up + SwiGLU + re-quant op (the reference's ``grouped_swiglu_loop_out``,
acceleration/custom_ops/qwen2_5_vl/aclnn_grouped_swiglu_out_bridge.cpp:157-273) against the oracle's
composition of the same steps: int32 accumulation (exact), ``acc * s_token * s_channel`` rounded to fp16,
``silu(gate) * up`` in fp16, per-token abs-max quantisation (smoothquant/fake_quant.py:22-31).

Bar: the integer accumulators are exact, so gate and up are the oracle's bits; SiLU on the GPU uses the
hardware exponential and its fp16 result can differ from the oracle's in the last bit on a small share of
elements.  Hence scales agree within one fp16 step, codes within one code with at most 1% of them off, and
the dequantised product ``codes * scale`` within 1e-2 relative Frobenius error.
"""
import numpy as np
import pytest
import torch

from mindpipe_b200 import synth
from oracle import pseudo_quant as O

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def ops():
    from mindpipe_b200 import ops as _ops
    yield _ops
    _ops.check_device_errors()


def _case(t, h, c, chunks, seed):
    """Reference-side tensors: codes and scales of x, and the batched ``[chunks, H, 2C]`` weight with its
    per-chunk views, as the runtime hands them to the op."""
    x = synth.normal_activation(t, h, seed=seed)
    _, xq, xs = O.absmax_quant_last_dim(x.numpy())
    w = torch.cat([synth.normal_weight(2 * c, h, seed=seed, index=10 + i)[None] for i in range(chunks)])
    _, wq, ws = O.absmax_quant_last_dim(w.numpy())                  # [chunks, 2C, H] codes, [chunks, 2C, 1] scales
    batched_weight = torch.from_numpy(wq).transpose(1, 2).contiguous()           # [chunks, H, 2C]
    batched_scale = torch.from_numpy(ws[..., 0].astype(np.float32)).contiguous()   # [chunks, 2C]
    return xq, xs[:, 0].astype(np.float32), wq, ws[..., 0].astype(np.float32), batched_weight, batched_scale


def _oracle(xq, xs, wq, ws, rows):
    """codes [chunks, rows, C], scales [chunks, rows] for the sampled token rows."""
    qs, ss = [], []
    for ch in range(wq.shape[0]):
        acc = (xq[rows].astype(np.float64) @ wq[ch].astype(np.float64).T).astype(np.float32)   # exact: |acc| < 2^53
        gu = (acc * xs[rows, None] * ws[ch][None, :]).astype(np.float16)
        c = gu.shape[1] // 2
        h = (O.silu_f16(gu[:, :c]) * gu[:, c:]).astype(np.float16)
        _, q, s = O.absmax_quant_last_dim(h)
        qs.append(q)
        ss.append(s[:, 0].astype(np.float32))
    return np.stack(qs), np.stack(ss)


def _check(got_q, got_s, ref_q, ref_s):
    assert np.all(np.abs(got_s - ref_s) <= ref_s * 2.0 ** -10 + 1e-12)
    diff = np.abs(got_q.astype(np.int32) - ref_q.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() <= 0.01
    assert O.rel_frobenius(got_q * got_s[..., None], ref_q * ref_s[..., None]) <= TOL


def _run(ops, t, h, c, chunks, seed, via_torch_op=False):
    xq, xs, wq, ws, bw, bs = _case(t, h, c, chunks, seed)
    dev = lambda a: (a if torch.is_tensor(a) else torch.from_numpy(a)).cuda()
    bw_d, bs_d = dev(bw), dev(bs)
    args = (dev(xq), [bw_d[i:i + 1] for i in range(chunks)], bw_d, torch.tensor([t], dtype=torch.int64, device="cuda"),
            [bs_d[i:i + 1] for i in range(chunks)], bs_d, dev(xs), 64, 0)
    if via_torch_op:
        from mindpipe_b200.custom_ops import load_and_register
        q, s = load_and_register().grouped_swiglu_loop_out(*args)
    else:
        q, s = ops.grouped_swiglu_loop_out(*args)
    ops.check_device_errors()
    assert tuple(q.shape) == (chunks, t, c) and q.dtype == torch.int8
    assert tuple(s.shape) == (chunks, t) and s.dtype == torch.float32
    return xq, xs, wq, ws, q.cpu().numpy(), s.cpu().numpy()


@pytest.mark.parametrize("t,h,c,chunks", [(300, 512, 256, 3), (1, 256, 128, 2), (256, 128, 384, 1), (513, 384, 144, 4)])
def test_loop_out_matches_oracle_composition(ops, t, h, c, chunks):
    xq, xs, wq, ws, q, s = _run(ops, t, h, c, chunks, seed=t + c)
    ref_q, ref_s = _oracle(xq, xs, wq, ws, np.arange(t))
    _check(q, s, ref_q, ref_s)


def test_loop_out_under_programmatic_dependent_launch_same_bits(ops):
    """The op's three launches chained (each kernel waits for its predecessor on the device): the bits of the
    serialised launches."""
    from mindpipe_b200 import _lib
    base = _run(ops, 300, 512, 256, 3, seed=77)
    lib = _lib.load()
    before = lib.mp_set_programmatic_launch(1)
    try:
        for _ in range(3):
            got = _run(ops, 300, 512, 256, 3, seed=77)
            assert np.array_equal(got[4], base[4]) and np.array_equal(got[5], base[5])
    finally:
        lib.mp_set_programmatic_launch(before)


def test_loop_out_qwen25_vl_7b_shape_token_sample(ops):
    """Hidden 3584, four chunks of 4736 (scripts/repro/verify_qwen25_vl_w8a8_loop_out_hybrid.py:17-19), a ragged
    token count; the oracle runs on a seeded sample of tokens (each output row depends on its own token only)."""
    t, h, c, chunks = 777, 3584, 4736, 4
    xq, xs, wq, ws, q, s = _run(ops, t, h, c, chunks, seed=25, via_torch_op=True)
    rows = np.sort(np.random.default_rng(7).choice(t, 48, replace=False))
    ref_q, ref_s = _oracle(xq, xs, wq, ws, rows)
    _check(q[:, rows], s[:, rows], ref_q, ref_s)


def test_loop_out_reference_layout_equals_kernel_layout(ops):
    """The reference's ``[chunks, H, 2C]`` weight (transposed once and cached by the wrapper) and the kernel's own
    ``[chunks, 2C, H]`` layout give the same bits."""
    t, h, c, chunks = 200, 256, 256, 2
    xq, xs, wq, ws, q, s = _run(ops, t, h, c, chunks, seed=3)
    lib_w = torch.from_numpy(wq).cuda()
    lib_s = torch.from_numpy(ws).cuda()
    q2, s2 = ops.w8a8_gate_up_swiglu_requant(torch.from_numpy(xq).cuda(), torch.from_numpy(xs).cuda(), lib_w, lib_s)
    assert np.array_equal(q2.cpu().numpy(), q) and np.array_equal(s2.cpu().numpy(), s)


def test_loop_out_argument_checks(ops):
    xq, xs, wq, ws, bw, bs = _case(4, 128, 64, 2, seed=1)
    bw_d, bs_d = bw.cuda(), bs.cuda()
    x = torch.from_numpy(xq).cuda()
    sx = torch.from_numpy(xs).cuda()
    gl = torch.tensor([4], dtype=torch.int64, device="cuda")
    views, sviews = [bw_d[i:i + 1] for i in range(2)], [bs_d[i:i + 1] for i in range(2)]
    with pytest.raises(RuntimeError):
        ops.grouped_swiglu_loop_out(x, [], bw_d, gl, [], bs_d, sx, 64, 0)
    with pytest.raises(RuntimeError):
        ops.grouped_swiglu_loop_out(x, views[:1], bw_d, gl, sviews[:1], bs_d, sx, 64, 0)
    with pytest.raises(RuntimeError):
        ops.grouped_swiglu_loop_out(x, views, bw_d, gl.to(torch.int32), sviews, bs_d, sx, 64, 0)
    with pytest.raises(RuntimeError):
        ops.grouped_swiglu_loop_out(x, views, bw_d, gl, sviews, bs_d, sx[:3], 64, 0)
