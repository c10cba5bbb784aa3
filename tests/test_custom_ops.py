"""The torch.library registration: fake implementations on CPU, real ones on the GPU."""
import pytest
import torch


def test_registration_is_idempotent_and_fake_impls_give_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    from mindpipe_b200.custom_ops import load_and_register
    ns = load_and_register()
    assert load_and_register() is ns
    with FakeTensorMode():
        x = torch.empty(2, 5, 256, dtype=torch.float16)
        y = ns.w4a16_linear(x, torch.empty(64, 32, dtype=torch.int32), torch.empty(2, 64, 2, dtype=torch.float16))
        assert y.shape == (2, 5, 64) and y.dtype == torch.float16
        q, s = ns.act_quant_per_token(x)
        assert q.shape == x.shape and q.dtype == torch.int8 and s.shape == (2, 5) and s.dtype == torch.float32
        y = ns.w8a8_linear(x, torch.empty(48, 256, dtype=torch.int8), torch.empty(48, 1, dtype=torch.float16))
        assert y.shape == (2, 5, 48)
        y = ns.w8a8_gemm(torch.empty(7, 256, dtype=torch.int8), torch.empty(7), torch.empty(48, 256, dtype=torch.int8),
                         torch.empty(48))
        assert y.shape == (7, 48) and y.dtype == torch.float16
        h = torch.empty(9, 128, dtype=torch.float16)
        out = ns.moe_w8a8_experts(h, torch.empty(9, 2, dtype=torch.int32), torch.empty(9, 2, dtype=torch.float16),
                                  torch.empty(4, 512, 128, dtype=torch.int8), torch.empty(4, 512),
                                  torch.empty(4, 128, 256, dtype=torch.int8), torch.empty(4, 128))
        assert out.shape == h.shape
        bw, bs = torch.empty(4, 128, 96, dtype=torch.int8), torch.empty(4, 96)
        q, s = ns.grouped_swiglu_loop_out(torch.empty(9, 128, dtype=torch.int8), [bw[i:i + 1] for i in range(4)], bw,
                                          torch.empty(1, dtype=torch.int64), [bs[i:i + 1] for i in range(4)], bs,
                                          torch.empty(9), 64, 0)
        assert q.shape == (4, 9, 48) and q.dtype == torch.int8 and s.shape == (4, 9) and s.dtype == torch.float32


def test_loop_out_argument_checks_precede_any_device_work():
    """The bridge's checks (aclnn_grouped_swiglu_out_bridge.cpp:166-199) fire on the host before a kernel is
    looked up, so they can be exercised without a GPU."""
    from mindpipe_b200 import ops
    bw, bs = torch.zeros(2, 128, 96, dtype=torch.int8), torch.zeros(2, 96)
    x, xs, gl = torch.zeros(4, 128, dtype=torch.int8), torch.zeros(4), torch.tensor([4], dtype=torch.int64)
    views, sviews = [bw[i:i + 1] for i in range(2)], [bs[i:i + 1] for i in range(2)]
    with pytest.raises(RuntimeError, match="non-empty"):
        ops.grouped_swiglu_loop_out(x, [], bw, gl, [], bs, xs, 64, 0)
    with pytest.raises(RuntimeError, match="chunk count"):
        ops.grouped_swiglu_loop_out(x, views[:1], bw, gl, sviews[:1], bs, xs, 64, 0)
    with pytest.raises(RuntimeError, match="int8"):
        ops.grouped_swiglu_loop_out(x.float(), views, bw, gl, sviews, bs, xs, 64, 0)
    with pytest.raises(RuntimeError, match="x_scale"):
        ops.grouped_swiglu_loop_out(x, views, bw, gl, sviews, bs, xs[:3], 64, 0)
    with pytest.raises(RuntimeError, match="group_list"):
        ops.grouped_swiglu_loop_out(x, views, bw, gl.to(torch.int32), sviews, bs, xs, 64, 0)
    with pytest.raises(ValueError, match="CUDA tensor"):          # everything valid: stops at "there is no CPU path"
        ops.grouped_swiglu_loop_out(x, views, bw, gl, sviews, bs, xs, 64, 0)


@pytest.mark.gpu
def test_ops_run_eager_and_under_torch_compile():
    from mindpipe_b200 import ops, synth
    from mindpipe_b200.custom_ops import load_and_register
    ns = load_and_register()
    w = synth.normal_weight(256, 512, seed=0).cuda()
    x = synth.normal_activation(4, 512, seed=0).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    sz = ops.w4a16_prepare(scale, zero, 512)
    eager = ns.w4a16_linear(x, packed, sz)
    assert torch.equal(eager, ops.w4a16_linear_decode(x, packed, sz))

    def f(a):
        return ns.w4a16_linear(a, packed, sz) * 2

    compiled = torch.compile(f, fullgraph=True)
    assert torch.equal(compiled(x), eager * 2)
    qw, sw, _ = ops.act_quant_per_token(w)
    y = ns.w8a8_linear(x, qw, sw.reshape(-1, 1).half())
    q, s = ns.act_quant_per_token(x)
    assert torch.equal(y, ops.w8a8_gemm(q, s, qw, sw))
    ops.check_device_errors()
