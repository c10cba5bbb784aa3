"""Tensor-level wrappers over the C ABI.

Each function validates its tensors the way the reference's native bridge
does (defined, on the device, exact dtype, contiguous:
acceleration/custom_ops/qwen2_5_vl/aclnn_grouped_swiglu_out_bridge.cpp:101-109),
allocates the outputs with the input's device, and launches on the current
CUDA stream.  torch is used for memory and streams only; all arithmetic is in
the CUDA library.  Nothing here falls back to torch math.
"""
from __future__ import annotations

import threading

import torch

from . import _lib

_ws_lock = threading.Lock()
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _req(t: torch.Tensor, name: str, dtype, ndim: int | None = None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must be {ndim}D, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Zero-initialised scratch, one per (device, stream), grown on demand.

    The kernels that use it leave it zeroed where it has to be, so it is
    cleared only when it is (re)allocated.
    """
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    with _ws_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("scratch memory would be allocated during CUDA graph capture; "
                                   "pass a preallocated workspace= (see new_workspace)")
            ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            _workspaces[key] = ws
    return ws


def new_workspace(nbytes: int, device) -> torch.Tensor:
    """A zero-filled scratch buffer for callers that manage scratch themselves (CUDA graphs)."""
    return torch.zeros(max(int(nbytes), 1 << 16), dtype=torch.uint8, device=device)


def w4a16_decode_workspace_bytes(m: int, n: int, k: int, k_split: int = 0) -> int:
    return int(_lib.load().mp_w4a16_decode_workspace_bytes_ex(m, n, k, k_split))


# ------------------------------------------------------------------ W4A16
def w4a16_quantize(weight: torch.Tensor, group_size: int = 128):
    """Asymmetric int4 group quantisation + packing of ``weight[N,K]`` (fp16).

    Returns ``(weight_packed int32[N,K/8], weight_scale f16[N,G],
    weight_zero_point int32[N,ceil(G/8)], group_size_used)``.  When ``K`` is
    not a multiple of ``group_size`` one group spans the row, as the
    reference does (quantizer.py:67-68).
    """
    w = _req(weight, "weight", torch.float16, 2)
    n, k = w.shape
    g = group_size if (group_size > 0 and k % group_size == 0) else k
    groups = k // g
    packed = torch.empty((n, k // 8), dtype=torch.int32, device=w.device)
    scale = torch.empty((n, groups), dtype=torch.float16, device=w.device)
    zero = torch.empty((n, (groups + 7) // 8), dtype=torch.int32, device=w.device)
    st = _lib.load().mp_w4a16_quantize(w.data_ptr(), n, k, g, packed.data_ptr(), scale.data_ptr(),
                                       zero.data_ptr(), _stream())
    _lib.check(st, "w4a16_quantize", N=n, K=k, group=g)
    return packed, scale, zero, g


def w4a16_dequant(weight_packed, weight_scale, weight_zero_point, out_features: int, in_features: int):
    """fp16 ``[N,K]`` weights ``f16((u - z) * s)``; ``weight_zero_point=None`` means z = 8."""
    p = _req(weight_packed, "weight_packed", torch.int32, 2)
    s = _req(weight_scale, "weight_scale", torch.float16, 2)
    z = None if weight_zero_point is None else _req(weight_zero_point, "weight_zero_point", torch.int32, 2)
    n, k = int(out_features), int(in_features)
    if p.shape != (n, k // 8) or k % 8:
        raise ValueError(f"weight_packed shape {tuple(p.shape)} does not match ({n}, {k}//8)")
    groups = s.shape[1]
    if s.shape[0] != n or k % groups:
        raise ValueError(f"weight_scale shape {tuple(s.shape)} does not divide K={k}")
    out = torch.empty((n, k), dtype=torch.float16, device=p.device)
    st = _lib.load().mp_w4a16_dequant(p.data_ptr(), s.data_ptr(), _ptr(z), n, k, k // groups,
                                      out.data_ptr(), _stream())
    _lib.check(st, "w4a16_dequant", N=n, K=k, groups=groups)
    return out


def w4a16_prepare(weight_scale, weight_zero_point, in_features: int):
    """Group-major ``(scale, zero)`` fp16 pairs ``[G, N, 2]`` read by the GEMM kernels."""
    s = _req(weight_scale, "weight_scale", torch.float16, 2)
    z = None if weight_zero_point is None else _req(weight_zero_point, "weight_zero_point", torch.int32, 2)
    n, groups = s.shape
    k = int(in_features)
    sz = torch.empty((groups, n, 2), dtype=torch.float16, device=s.device)
    st = _lib.load().mp_w4a16_prepare(s.data_ptr(), _ptr(z), n, k, k // groups, sz.data_ptr(), _stream())
    _lib.check(st, "w4a16_prepare", N=n, K=k, groups=groups)
    return sz


def w4a16_linear_decode(x, weight_packed, scale_zero, bias=None, *, k_split: int = 0, workspace=None, out=None):
    """``y[M,N] = x[M,K] @ dequant(W)^T (+bias)`` for M <= 64 (decode shapes).

    ``workspace`` (uint8, zero-filled when created, not shared by calls that
    may overlap) defaults to a cached buffer per device and stream.
    """
    x2 = _req(x, "x", torch.float16, 2)
    p = _req(weight_packed, "weight_packed", torch.int32, 2)
    sz = _req(scale_zero, "scale_zero", torch.float16, 3)
    b = None if bias is None else _req(bias, "bias", torch.float16, 1)
    m, k = x2.shape
    n = p.shape[0]
    groups = sz.shape[0]
    if p.shape[1] * 8 != k or sz.shape[1] != n or k % groups:
        raise ValueError(f"shape mismatch: x{tuple(x2.shape)} packed{tuple(p.shape)} sz{tuple(sz.shape)}")
    lib = _lib.load()
    nbytes = lib.mp_w4a16_decode_workspace_bytes_ex(m, n, k, k_split)
    ws = _workspace(nbytes, x2.device) if workspace is None else _req(workspace, "workspace", torch.uint8, 1)
    y = torch.empty((m, n), dtype=torch.float16, device=x2.device) if out is None else _req(out, "out", torch.float16, 2)
    if y.shape != (m, n):
        raise ValueError(f"out must be [{m}, {n}]")
    st = lib.mp_w4a16_linear_decode_ex(x2.data_ptr(), p.data_ptr(), sz.data_ptr(), _ptr(b), y.data_ptr(),
                                       m, n, k, k // groups, ws.data_ptr(), ws.numel(), k_split, _stream())
    _lib.check(st, "w4a16_linear_decode", M=m, N=n, K=k, group=k // groups)
    return y


def w4a16_linear(x, weight_packed, scale_zero, bias=None):
    """W4A16 linear for any number of rows.

    Rows are processed in slabs of at most 64 by the weight-streaming kernel.
    """
    m = x.shape[0]
    if m <= 64:
        return w4a16_linear_decode(x, weight_packed, scale_zero, bias)
    outs = [w4a16_linear_decode(x[i:i + 64], weight_packed, scale_zero, bias) for i in range(0, m, 64)]
    return torch.cat(outs, dim=0)


# ------------------------------------------------------------------- W8A8
def act_quant_per_token(x, *, want_codes: bool = True, want_fake: bool = False):
    """Per-row symmetric int8 quantisation of ``x[..., K]`` (fp16).

    Returns ``(codes int8[...,K] | None, scale f32[...] | None, fake f16 | None)``.
    """
    xt = _req(x, "x", torch.float16)
    k = xt.shape[-1]
    m = xt.numel() // k
    q = torch.empty(xt.shape, dtype=torch.int8, device=xt.device) if want_codes else None
    s = torch.empty(xt.shape[:-1], dtype=torch.float32, device=xt.device) if want_codes else None
    f = torch.empty_like(xt) if want_fake else None
    if m == 0:
        return q, s, f
    st = _lib.load().mp_act_quant_per_token(xt.data_ptr(), m, k, _ptr(q), _ptr(s), _ptr(f), _stream())
    _lib.check(st, "act_quant_per_token", M=m, K=k)
    return q, s, f
