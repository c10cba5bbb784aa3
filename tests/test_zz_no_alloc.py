"""The allocation-free decode entry point (collected last on purpose).

``mp_w4a16_linear_decode_static`` serves callers that cannot allocate device
memory -- a plugin inside another runtime's forward pass whose allocator is
closed to it, code running where ``cudaMalloc`` is off limits -- by keeping
the split-K scratch in a fixed array inside the library.  It must give the
results of the existing workspace entry point, call after call, although the
array still holds whatever the previous call left behind.
"""
import numpy as np
import pytest
import torch

from mindpipe_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-2          # relative Frobenius bound used by the W4A16 output tests


def _case(n, k, m, seed, bias):
    from mindpipe_b200 import ops
    w = synth.normal_weight(n, k, seed=seed, index=1).cuda()
    x = synth.normal_activation(m, k, seed=seed, index=2).cuda()
    b = (synth.normal_activation(1, n, seed=seed, index=3)[0] * 0.1).half().cuda() if bias else None
    packed, scale, zero, _ = ops.w4a16_quantize(w, 128)
    sz = ops.w4a16_prepare(scale, zero, k)
    return x, packed, sz, b


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


@pytest.mark.parametrize("n,k,m,bias", [(4096, 4096, 16, False), (1024, 2048, 5, True), (512, 11008, 33, False)])
def test_static_scratch_matches_workspace_entry_on_two_calls_in_a_row(n, k, m, bias):
    from mindpipe_b200 import ops
    x, packed, sz, b = _case(n, k, m, seed=n + m, bias=bias)
    ref = ops.w4a16_linear_decode(x, packed, sz, b, k_split=4)         # existing entry point, caller's workspace
    out = torch.empty_like(ref)
    first = ops.w4a16_linear_decode_static(x, packed, sz, b, out=out).clone()
    second = ops.w4a16_linear_decode_static(x, packed, sz, b, out=out)  # scratch still holds the first call's data
    torch.cuda.synchronize()
    assert _rel(first, ref) <= TOL
    assert _rel(second, ref) <= TOL
    assert torch.equal(first, second)                                  # fixed summation order: repeatable


def test_static_scratch_survives_a_different_shape_in_between():
    from mindpipe_b200 import ops
    xa, pa, sa, _ = _case(2048, 4096, 16, seed=1, bias=False)
    xb, pb, sb, _ = _case(256, 1024, 3, seed=2, bias=False)
    ya = ops.w4a16_linear_decode_static(xa, pa, sa)
    yb = ops.w4a16_linear_decode_static(xb, pb, sb)
    ya2 = ops.w4a16_linear_decode_static(xa, pa, sa)
    torch.cuda.synchronize()
    assert torch.equal(ya, ya2)
    assert _rel(yb, ops.w4a16_linear_decode(xb, pb, sb, k_split=2)) <= TOL


def test_static_scratch_rejects_sizes_beyond_its_array():
    from mindpipe_b200 import _lib, ops
    lib = _lib.load()
    assert lib.mp_w4a16_linear_decode_static_max_bytes() == 8 << 20
    # M=64, N=16384, K=1024: two K slices of 64 x 16384 fp32 partial sums are 8 MiB, plus the counters
    x = torch.zeros(64, 1024, dtype=torch.float16, device="cuda")
    packed = torch.zeros(16384, 1024 // 8, dtype=torch.int32, device="cuda")
    sz = torch.zeros(1024 // 128, 16384, 2, dtype=torch.float16, device="cuda")
    with pytest.raises(_lib.MindPipeKernelError, match="workspace"):
        ops.w4a16_linear_decode_static(x, packed, sz)
