"""GPU parity of the W4A16 path against the CPU oracle (through the C ABI).

Bit-exact: packed codes, scales, zero points, dequantised weights.
fp16 outputs: relative Frobenius error <= 1e-2 against the oracle's
``F.linear(x, Wdq)`` (observed ~1e-3).
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


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def quantize_both(w16: np.ndarray, group=128):
    from mindpipe_b200 import ops
    packed, scale, zero, g = ops.w4a16_quantize(dev(w16), group)
    wdq, s, z, u = O.w4_group_asym_quantize(w16, group)
    return (packed, scale, zero, g), (wdq, s, z, u)


@pytest.mark.parametrize("key", ["w", "w_ragged", "w_const"])
def test_quantize_golden_bit_exact(golden, key):
    g = golden("w4a16_small.npz")
    w = g[key]
    (packed, scale, zero, gs), (wdq, s, z, u) = quantize_both(w)
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4_unsigned(u))
    assert np.array_equal(bits(scale.cpu().numpy()), bits(s))
    assert np.array_equal(zero.cpu().numpy(), O.pack_int4_unsigned(z.astype(np.uint8)))
    from mindpipe_b200 import ops
    back = ops.w4a16_dequant(packed, scale, zero, w.shape[0], w.shape[1])
    assert np.array_equal(bits(back.cpu().numpy()), bits(g[key.replace("w", "wdq", 1)]))


def test_quantize_dequant_cfg1_full_size_bit_exact():
    """Config 1: W[4096,4096] ~ N(0,0.02), seed 0, asymmetric int4 g128."""
    from mindpipe_b200 import ops
    w = synth.normal_weight(4096, 4096, seed=0, index=0).numpy()
    (packed, scale, zero, gs), (wdq, s, z, u) = quantize_both(w)
    assert gs == 128
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4_unsigned(u))
    assert np.array_equal(bits(scale.cpu().numpy()), bits(s))
    assert np.array_equal(zero.cpu().numpy(), O.pack_int4_unsigned(z.astype(np.uint8)))
    back = ops.w4a16_dequant(packed, scale, zero, 4096, 4096)
    assert np.array_equal(bits(back.cpu().numpy()), bits(wdq))


def test_symmetric_export_format_dequant(golden):
    """The reference's exported format: signed codes stored +8, no zero-point tensor."""
    from mindpipe_b200 import ops
    g = golden("int4_pack.npz")
    out = ops.w4a16_dequant(dev(g["q_packed"]), dev(g["scale"]), None, 6, 40)
    assert np.array_equal(bits(out.cpu().numpy()), bits(g["q_dequant_f32"].astype(np.float16)))
    a = golden("gptq_artifact.npz")
    out = ops.w4a16_dequant(dev(a["packed"]), dev(a["scale"].astype(np.float16)), None, 16, 64)
    ref = O.w4_dequant(a["packed"], a["scale"].astype(np.float16), None, 16, 64, 32)
    assert np.array_equal(bits(out.cpu().numpy()), bits(ref))


def _linear_case(n, k, m, group=128, seed=0, bias=False, k_split=0):
    from mindpipe_b200 import ops
    w = synth.normal_weight(n, k, seed=seed, index=1).numpy()
    x = synth.normal_activation(m, k, seed=seed, index=2).numpy()
    b = (synth.normal_activation(1, n, seed=seed, index=3).numpy()[0] * np.float16(0.1)).astype(np.float16) if bias else None
    (packed, scale, zero, gs), (wdq, s, z, u) = quantize_both(w, group)
    sz = ops.w4a16_prepare(scale, zero, k)
    y = ops.w4a16_linear_decode(dev(x), packed, sz, None if b is None else dev(b), k_split=k_split)
    torch.cuda.synchronize()
    ref = O.linear_f16(x, wdq, b)
    return y.cpu().numpy(), ref


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64])
def test_decode_small_all_row_counts(m):
    y, ref = _linear_case(96, 512, m)
    assert y.shape == ref.shape
    assert O.rel_frobenius(y, ref) <= TOL


@pytest.mark.parametrize("n,k,group", [(8, 128, 128), (40, 256, 64), (72, 384, 32), (264, 1280, 128), (64, 256, 256)])
def test_decode_ragged_shapes_and_groups(n, k, group):
    for m in (1, 16):
        y, ref = _linear_case(n, k, m, group=group, bias=True)
        assert O.rel_frobenius(y, ref) <= TOL


@pytest.mark.parametrize("k_split", [1, 2, 3, 8])
def test_decode_explicit_k_split_and_bias(k_split):
    y, ref = _linear_case(128, 2048, 5, bias=True, k_split=k_split)
    assert O.rel_frobenius(y, ref) <= TOL


@pytest.mark.parametrize("m", [1, 16])
def test_decode_cfg1_full_size(m):
    """Config 1: 4096x4096, M in {1,16}, seed 0."""
    y, ref = _linear_case(4096, 4096, m, seed=0)
    assert O.rel_frobenius(y, ref) <= TOL


@pytest.mark.parametrize("n,k", [(11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("m", [1, 16])
def test_decode_cfg2_mlp_shapes(n, k, m):
    y, ref = _linear_case(n, k, m, seed=1)
    assert O.rel_frobenius(y, ref) <= TOL


def test_decode_repeat_calls_identical_and_workspace_rearmed():
    from mindpipe_b200 import ops
    w = synth.normal_weight(256, 4096, seed=3, index=1)
    x = synth.normal_activation(16, 4096, seed=3, index=2).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w.cuda(), 128)
    sz = ops.w4a16_prepare(scale, zero, 4096)
    y0 = ops.w4a16_linear_decode(x, packed, sz)
    for _ in range(5):
        y = ops.w4a16_linear_decode(x, packed, sz)
        assert torch.equal(y, y0)          # fixed-order split-K sum: run-to-run identical


def test_decode_linearity_property_full_size():
    """Size-independent check at a 70B shape: f(2x) = 2 f(x) to within one fp16 rounding of the output."""
    from mindpipe_b200 import ops
    n, k = 8192, 8192
    w = synth.normal_weight(n, k, seed=5, index=1).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    sz = ops.w4a16_prepare(scale, zero, k)
    x = synth.normal_activation(8, k, seed=5, index=2).cuda()
    y = ops.w4a16_linear_decode(x, packed, sz)
    y2 = ops.w4a16_linear_decode(x * 2, packed, sz)
    # scaling by a power of two is exact end to end except for two roundings that are not scale
    # invariant: outputs in the fp16 subnormal range (spacing 2^-24), and, in the folded kernel, the
    # few activations below 2^-10, whose 1/16 multiple is subnormal (an absolute error of a few 1e-7
    # in an output of magnitude ~1).  Either moves an output by at most one fp16 unit in the last
    # place, or by 2^-19 absolutely where the output itself is a near-cancellation.
    gap = (y2.float() - 2 * y.float()).abs()
    assert bool((gap <= 2.0 ** -10 * (2 * y.float()).abs() + 2.0 ** -19).all())
    assert (gap > 0).float().mean().item() < 0.01
    ref = (x.float() @ ops.w4a16_dequant(packed, scale, zero, n, k).float().T)
    err = (y.float() - ref).norm() / ref.norm()
    assert err.item() <= TOL


def test_module_forward_matches_reference_forward(golden):
    """VllmPackedInt4Linear.forward == F.linear(x, pseudo_quantize_tensor(W)) on the golden case."""
    from mindpipe_b200.modules import VllmPackedInt4Linear
    g = golden("w4a16_small.npz")
    lin = torch.nn.Linear(384, 24, bias=False).half().cuda()
    with torch.no_grad():
        lin.weight.copy_(dev(g["w"]))
    m = VllmPackedInt4Linear.from_float(lin)
    assert np.array_equal(bits(m.dequantize().cpu().numpy()), bits(g["wdq"]))
    y = m(dev(g["x"]))
    assert O.rel_frobenius(y.cpu().numpy(), g["y"]) <= TOL
    y3 = m(dev(g["x"]).reshape(1, 5, 384))
    assert y3.shape == (1, 5, 24)
    big = m(dev(np.tile(g["x"], (20, 1))))          # M = 100 goes through 64-row slabs
    assert O.rel_frobenius(big.cpu().numpy()[:5], g["y"]) <= TOL


@pytest.mark.parametrize("m", [1, 16])
def test_host_buffer_entry_matches_device_entry(m):
    """The host-buffer form (H2D copy, kernel, D2H copy on one stream) gives the device entry's bits."""
    from mindpipe_b200.modules import VllmPackedInt4Linear
    n, k = 512, 1024
    lin = torch.nn.Linear(k, n, bias=True).half().cuda()
    mod = VllmPackedInt4Linear.from_float(lin)
    x_host = synth.normal_activation(m, k, seed=3, index=m).pin_memory()
    y_host = torch.empty((m, n), dtype=torch.float16).pin_memory()
    side = torch.cuda.Stream()
    for it in range(4):               # 2nd call: staging buffers reused; 3rd, 4th: the validated raw call, own stream
        y_host.zero_()
        out = mod.forward_host(x_host, y_host, stream=side if it == 3 else None)
        torch.cuda.synchronize()
        assert out is y_host
        assert torch.equal(y_host, mod(x_host.cuda()).cpu())
    with pytest.raises(ValueError):
        mod.forward_host(x_host.cuda(), y_host)
    with pytest.raises(RuntimeError):
        mod.forward_host(synth.normal_activation(17, k, seed=3).pin_memory())


def test_zero_copy_output_of_the_host_buffer_entry():
    """Repeated host-buffer calls store the result into the pinned output through its device-side address; the
    staged form (kernel into a device buffer, then a D2H copy) gives the same bits.  Pageable memory has no such
    address and keeps the staged form."""
    import ctypes
    from mindpipe_b200 import _lib
    from mindpipe_b200.modules import VllmPackedInt4Linear
    lib = _lib.load()
    pinned = torch.empty(4096, dtype=torch.float16).pin_memory()
    alias = ctypes.c_void_p()
    assert lib.mp_host_buffer_device_alias(pinned.data_ptr(), pinned.numel() * 2, ctypes.byref(alias)) == 0
    assert alias.value
    pageable = torch.empty(4096, dtype=torch.float16)
    assert lib.mp_host_buffer_device_alias(pageable.data_ptr(), pageable.numel() * 2, ctypes.byref(alias)) != 0
    n, k = 1536, 2048
    mod = VllmPackedInt4Linear.from_float(torch.nn.Linear(k, n, bias=True).half().cuda())
    for m in (1, 5, 16):
        x_host = synth.normal_activation(m, k, seed=8, index=m).pin_memory()
        want = mod(x_host.cuda()).cpu()
        for zero_copy in (True, False):
            y_host = torch.empty((m, n), dtype=torch.float16).pin_memory()
            for _ in range(3):                      # the second and third call run the remembered form
                y_host.zero_()
                mod.forward_host(x_host, y_host, zero_copy_output=zero_copy)
                torch.cuda.synchronize()
                assert torch.equal(y_host, want)
        y_pageable = torch.empty((m, n), dtype=torch.float16)
        for _ in range(2):
            mod.forward_host(x_host, y_pageable)
            torch.cuda.synchronize()
            assert torch.equal(y_pageable, want)


def test_host_buffer_entry_on_a_shape_that_takes_the_workspace_kernel():
    """A gate/up-sized linear at 16 rows: the host-buffer call owns a workspace per stream, so the library picks the
    same kernel as for device-resident activations -- same bits, staged or stored straight into pinned memory, on
    two streams in turn."""
    from mindpipe_b200 import ops
    from mindpipe_b200.modules import VllmPackedInt4Linear
    n, k, m = 22016, 4096, 16
    assert ops.w4a16_decode_kernel_choice(m, n, k) == "umma"
    w = synth.normal_weight(n, k, seed=6, index=1).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    mod = VllmPackedInt4Linear(packed_weight=packed, scale=scale, bias=None, in_features=k, out_features=n,
                               zero_point=zero)
    x_host = synth.normal_activation(m, k, seed=6, index=2).pin_memory()
    want = mod(x_host.cuda()).cpu()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for zero_copy in (True, False):
        y_hosts = [torch.empty((m, n), dtype=torch.float16).pin_memory() for _ in streams]
        for _ in range(3):
            for s_, y_host in zip(streams, y_hosts):
                y_host.zero_()
                mod.forward_host(x_host, y_host, stream=s_, zero_copy_output=zero_copy)
            torch.cuda.synchronize()
            for y_host in y_hosts:
                assert torch.equal(y_host, want)
    ops.check_device_errors()


def test_forward_host_many_matches_the_single_calls():
    """Several independent linears in one library call (copies in, kernels back to back, copies out): the bits of
    the one-by-one calls, with and without programmatic dependent launch, and again after one module's scales
    changed under the recorded call."""
    from mindpipe_b200 import _lib, ops
    from mindpipe_b200.modules import VllmPackedInt4Linear, forward_host_many
    shapes = [(768, 1024), (22016, 4096), (512, 2048), (4096, 4096)]
    mods, xs, ys, want = [], [], [], []
    for i, (n, k) in enumerate(shapes):
        w = synth.normal_weight(n, k, seed=14, index=i).cuda()
        packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
        mods.append(VllmPackedInt4Linear(packed_weight=packed, scale=scale, bias=None, in_features=k, out_features=n,
                                         zero_point=zero))
        xs.append(synth.normal_activation(16, k, seed=14, index=10 + i).pin_memory())
        ys.append(torch.empty((16, n), dtype=torch.float16).pin_memory())
        want.append(mods[-1](xs[-1].cuda()).cpu())
    side = torch.cuda.Stream()
    lib = _lib.load()
    for chained in (0, 1):
        before = lib.mp_set_programmatic_launch(chained)
        try:
            for _ in range(3):
                for y in ys:
                    y.zero_()
                out = forward_host_many(mods, xs, ys, stream=side)
                side.synchronize()
                assert out is ys
                for y, w_ in zip(ys, want):
                    assert torch.equal(y, w_)
        finally:
            lib.mp_set_programmatic_launch(before)
    mods[0].weight_scale.mul_(2)                      # the recorded call's derived buffer is stale now
    want0 = mods[0](xs[0].cuda()).cpu()
    forward_host_many(mods, xs, ys, stream=side)
    side.synchronize()
    assert torch.equal(ys[0], want0) and torch.equal(ys[1], want[1])
    with pytest.raises(ValueError):
        forward_host_many([mods[0], mods[0]], xs[:2], ys[:2])
    ops.check_device_errors()


def test_derived_buffers_follow_load_state_dict_and_in_place_updates():
    """The kernel-side (scale, zero) layout and the remembered host calls are rebuilt when the scales change
    under the module: through ``load_state_dict`` (copies in place) and through a plain in-place write."""
    from mindpipe_b200.modules import VllmPackedInt4Linear
    n, k = 256, 512
    a = VllmPackedInt4Linear.from_float(torch.nn.Linear(k, n, bias=False).half().cuda())
    b = VllmPackedInt4Linear.from_float(torch.nn.Linear(k, n, bias=False).half().cuda())
    x = synth.normal_activation(4, k, seed=12).cuda()
    x_host, y_host = x.cpu().pin_memory(), torch.empty((4, n), dtype=torch.float16).pin_memory()
    want_b = b(x)
    assert not torch.equal(a(x), want_b)                   # derived buffer of a's own weights now exists
    a.forward_host(x_host, y_host)
    a.forward_host(x_host, y_host)                         # the remembered raw call
    a.load_state_dict(b.state_dict())
    assert torch.equal(a(x), want_b)
    a.forward_host(x_host, y_host)
    torch.cuda.synchronize()
    assert torch.equal(y_host.cuda(), want_b)
    a.weight_scale.mul_(2)                                 # in place: scales doubled, zero points kept
    assert torch.equal(a(x), VllmPackedInt4Linear(packed_weight=b.weight_packed, scale=b.weight_scale * 2, bias=None,
                                                  in_features=k, out_features=n,
                                                  zero_point=b.weight_zero_point)(x))


def test_errors_are_loud():
    from mindpipe_b200 import _lib, ops
    x = torch.zeros(1, 64, dtype=torch.float16, device="cuda")             # K = 64 is not a multiple of 128
    with pytest.raises(_lib.MindPipeKernelError, match="not supported"):
        ops.w4a16_linear_decode(x, torch.zeros(8, 8, dtype=torch.int32, device="cuda"),
                                torch.zeros(1, 8, 2, dtype=torch.float16, device="cuda"))
    with pytest.raises(TypeError):
        ops.w4a16_quantize(torch.zeros(8, 128, device="cuda"), 128)          # fp32 weight
    with pytest.raises(ValueError):
        ops.w4a16_linear_decode(x, torch.zeros(8, 16, dtype=torch.int32, device="cuda"),
                                torch.zeros(1, 8, 2, dtype=torch.float16, device="cuda"))


def test_split_k_scratch_errors_are_loud():
    """A scratch buffer that is too small is refused with the "workspace" status, never written past."""
    from mindpipe_b200 import _lib, ops
    lib = _lib.load()
    m, n, k = 64, 512, 2048
    need = lib.mp_w4a16_prefill_workspace_bytes(m, n, k)
    assert need > 0
    w = synth.normal_weight(n, k, seed=9, index=0).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    sz = ops.w4a16_prepare(scale, zero, k)
    x = synth.normal_activation(m, k, seed=9, index=1).cuda()
    with pytest.raises(_lib.MindPipeKernelError, match="workspace"):
        ops.w4a16_linear_prefill(x, packed, sz, workspace=torch.zeros(need - 16, dtype=torch.uint8, device="cuda"))
    y = ops.w4a16_linear_prefill(x, packed, sz, workspace=torch.zeros(need, dtype=torch.uint8, device="cuda"))
    assert torch.equal(y, ops.w4a16_linear_prefill(x, packed, sz))
    # int8 GEMM: same contract
    need8 = lib.mp_w8a8_gemm_workspace_bytes(16, 4096, 4096)
    assert need8 > 0
    qx = torch.zeros((16, 4096), dtype=torch.int8, device="cuda")
    qw = torch.zeros((4096, 4096), dtype=torch.int8, device="cuda")
    with pytest.raises(_lib.MindPipeKernelError, match="workspace"):
        ops.w8a8_gemm(qx, torch.ones(16, device="cuda"), qw, torch.ones(4096, device="cuda"),
                      workspace=torch.zeros(need8 // 2, dtype=torch.uint8, device="cuda"))
    ops.check_device_errors()


# ---------------------------------------------------------------- prefill (tcgen05) kernel
def _prefill_case(n, k, m, group=128, seed=0, bias=False, rows=None):
    from mindpipe_b200 import ops
    w = synth.normal_weight(n, k, seed=seed, index=1).numpy()
    x = synth.normal_activation(m, k, seed=seed, index=2).numpy()
    b = (synth.normal_activation(1, n, seed=seed, index=3).numpy()[0] * np.float16(0.1)).astype(np.float16) if bias else None
    (packed, scale, zero, gs), (wdq, s, z, u) = quantize_both(w, group)
    sz = ops.w4a16_prepare(scale, zero, k)
    y = ops.w4a16_linear_prefill(dev(x), packed, sz, None if b is None else dev(b))
    ops.check_device_errors()
    y = y.cpu().numpy()
    if rows is not None:
        return y[rows], O.linear_f16(x[rows], wdq, b)
    return y, O.linear_f16(x, wdq, b)


@pytest.mark.parametrize("m,n,k,group", [
    (128, 256, 64, 64),        # one tile, one k-block
    (128, 256, 512, 128),      # k loop beyond the ring depth
    (65, 256, 256, 128),       # ragged M
    (300, 520, 1024, 128),     # ragged M and N, several tiles
    (1024, 2048, 256, 64),     # more tiles than one wave of CTAs? (8 x 8 = 64) no; both TMEM buffers via 2 tiles/CTA below
    (2048, 4864, 128, 128),    # 16 x 19 = 304 tiles over 148 CTAs: every CTA walks 2-3 tiles
    (1, 8, 64, 64),
])
def test_prefill_vs_oracle(m, n, k, group):
    y, ref = _prefill_case(n, k, m, group=group, bias=True)
    assert y.shape == ref.shape
    assert O.rel_frobenius(y, ref) <= TOL


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_prefill_cfg2_m2048_row_sample(n, k):
    """Config 2 at M=2048: every output row is produced, a seeded sample of rows is checked."""
    rows = np.random.default_rng(n + k).choice(2048, 96, replace=False)
    y, ref = _prefill_case(n, k, 2048, seed=2, rows=rows)
    assert O.rel_frobenius(y, ref) <= TOL


@pytest.mark.parametrize("m,n,k", [(17, 256, 2048), (65, 256, 2048), (128, 512, 4096), (200, 1024, 1024),
                                   (256, 4096, 4096), (512, 1024, 2048), (700, 512, 1024)])
def test_prefill_split_k_small_batches(m, n, k):
    """Few output tiles: K is cut into slices (fp32 partial tiles + an ordered sum).  Same result as the
    unsplit kernel to fp32 summation order, run-to-run identical, and within tolerance of the oracle."""
    from mindpipe_b200 import _lib, ops
    assert _lib.load().mp_w4a16_prefill_workspace_bytes(m, n, k) > 0          # these shapes do split
    w = synth.normal_weight(n, k, seed=m, index=0).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    sz = ops.w4a16_prepare(scale, zero, k)
    x = synth.normal_activation(m, k, seed=m, index=1).cuda()
    bias = (synth.normal_activation(1, n, seed=m, index=2)[0] * 0.1).to(torch.float16).cuda()
    y = ops.w4a16_linear_prefill(x, packed, sz, bias)
    ops.check_device_errors()
    assert torch.equal(y, ops.w4a16_linear_prefill(x, packed, sz, bias))
    wdq = ops.w4a16_dequant(packed, scale, zero, n, k).float()
    ref = x.float() @ wdq.T + bias.float()
    assert ((y.float() - ref).norm() / ref.norm()).item() <= TOL
    # a null workspace turns the split off: one K slice per tile, same math
    y1 = torch.empty_like(y)
    st = _lib.load().mp_w4a16_linear_prefill(x.data_ptr(), packed.data_ptr(), sz.data_ptr(), bias.data_ptr(),
                                             y1.data_ptr(), m, n, k, 128, ops._error_word(x.device).data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
    assert st == 0
    assert ((y.float() - y1.float()).abs().max() / ref.abs().max()).item() <= 2e-3


def test_linear_dispatch_uses_prefill_above_16_rows(golden):
    from mindpipe_b200 import ops
    w = synth.normal_weight(256, 512, seed=4, index=1).cuda()
    x = synth.normal_activation(200, 512, seed=4, index=2).cuda()
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    sz = ops.w4a16_prepare(scale, zero, 512)
    y = ops.w4a16_linear(x, packed, sz)
    slabs = torch.cat([ops.w4a16_linear_decode(x[i:i + 64], packed, sz) for i in range(0, 200, 64)])
    ops.check_device_errors()
    err = (y.float() - slabs.float()).norm() / slabs.float().norm()
    assert err.item() <= 2e-3                      # tensor-core vs streaming kernel: same Wdq, different sum order
