"""ctypes binding of ``libmindpipe_b200.so`` (the C ABI in ``include/mindpipe_b200.h``).

The library is loaded lazily, once, under a lock (the reference guards its
custom-op load the same way, acceleration/runtime_patches/vllm.patch:291-306).
There is no CPU fallback: if the shared library is missing or a symbol is
absent, loading raises.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_int, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmindpipe_b200.so"

_lock = threading.Lock()
_lib = None

# name -> (restype, argtypes); mirrors include/mindpipe_b200.h one to one.
_P, _I, _Z = c_void_p, c_int, c_size_t
_U = ctypes.c_uint
SIGNATURES = {
    "mp_abi_version": (_I, []),
    "mp_status_string": (c_char_p, [_I]),
    "mp_last_cuda_error": (_I, []),
    "mp_w4a16_quantize": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "mp_w4a16_dequant": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
    "mp_w4a16_prepare": (_I, [_P, _P, _I, _I, _I, _P, _P]),
    "mp_w4a16_decode_workspace_bytes": (_Z, [_I, _I, _I]),
    "mp_w4a16_decode_workspace_bytes_ex": (_Z, [_I, _I, _I, _I]),
    "mp_w4a16_linear_decode": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _P]),
    "mp_w4a16_linear_decode_ex": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _I, _P]),
    "mp_w4a16_linear_decode_opts": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _U, _P]),
    "mp_w4a16_rowparallel_push": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "mp_w4a16_rowparallel_finish": (_I, [_P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P]),
    "mp_w4a16_linear_decode_host": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "mp_host_buffer_device_alias": (_I, [_P, _Z, _P]),
    "mp_w4a16_linear_decode_host_ws": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _P]),
    "mp_w4a16_linear_decode_host_many": (_I, [_P, _I, _P]),
    "mp_w4a16_linear_prefill": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "mp_w4a16_prefill_workspace_bytes": (_Z, [_I, _I, _I]),
    "mp_w4a16_linear_prefill_ex": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _P, _P]),
    "mp_w4a16_linear_decode_static_max_bytes": (_Z, []),
    "mp_w4a16_linear_decode_static": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "mp_set_programmatic_launch": (_I, [_I]),
    "mp_set_decode_kernel": (_I, [_I]),
    "mp_w4a16_decode_kernel_choice": (_I, [_I, _I, _I, _I]),
    "mp_read_decode_error": (_I, [_P]),
    "mp_act_quant_per_token": (_I, [_P, _I, _I, _P, _P, _P, _P]),
    "mp_add_rmsnorm_quant": (_I, [_P, _P, _P, ctypes.c_float, _I, _I, _P, _P, _P]),
    "mp_w8a8_gemm": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "mp_w8a8_gemm_workspace_bytes": (_Z, [_I, _I, _I]),
    "mp_w8a8_gemm_ex": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _Z, _P, _P]),
    "mp_w8a8_gemm_i32": (_I, [_P, _P, _P, _I, _I, _I, _P, _P]),
    "mp_affine_quant_per_row": (_I, [_P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "mp_w8a8_affine_gemm": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "mp_moe_router_topk": (_I, [_P, _I, _I, _I, _P, _P, _P]),
    "mp_moe_plan_ints": (_Z, [_I, _I]),
    "mp_moe_padded_rows": (_I, [_I, _I]),
    "mp_moe_route_gather_quant": (_I, [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "mp_moe_expert_stage_workspace_bytes": (_Z, [_I, _I]),
    "mp_moe_expert_stage": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _Z, _P, _P]),
    "mp_moe_expert_stage_scatter": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _Z, _P, _P]),
    "mp_moe_combine": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "mp_moe_gemm1_swiglu": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _Z, _I, _P, _P]),
    "mp_moe_requant": (_I, [_P, _I, _I, _I, _P, _Z, _P]),
    "mp_moe_gemm2": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _Z, _I, _P, _P]),
    "mp_w8a8_gate_up_swiglu_requant_workspace_bytes": (_Z, [_I, _I, _I, _I]),
    "mp_w8a8_gate_up_swiglu_requant": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _Z, _P, _P]),
    "mp_gather_rows": (_I, [_P, _P, _I, _I, _P, _P]),
    "mp_peer_barrier": (_I, [_P, _I, _I, ctypes.c_uint, _P, _P]),
    "mp_peer_barrier_counted": (_I, [_P, _I, _I, _P, _P, _P]),
    "mp_peer_signal": (_I, [_P, _I, _I, _P, _P]),
    "mp_w8a8_rowparallel_finish": (_I, [_P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P]),
    "mp_peer_publish": (_I, [_P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _P]),
    "mp_w8a8_rowparallel_finish_parity": (_I, [_P, _P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P]),
    "mp_peer_allgather_recv_bytes": (_Z, [_I, _I, _I]),
    "mp_peer_allgather_push": (_I, [_P, _I, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P]),
    "mp_w4a16_rowparallel_recv_bytes": (_Z, [_I, _I, _I]),
    "mp_w4a16_rowparallel_finish_ll": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P]),
    "mp_moe_ep_plan_ints": (_Z, [_I, _I, _I]),
    "mp_moe_ep_plan": (_I, [_P, _I, _I, _I, _I, _P, _P]),
    "mp_moe_ep_barrier_plan": (_I, [_P, _P, _I, _I, _P, _I, _I, _P, _P, _P]),
    "mp_moe_ep_pull": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P]),
    "mp_moe_ep_push": (_I, [_P, _P, _I, _I, _I, _I, _P, _P]),
    "mp_moe_ep_pull_part": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P]),
    "mp_moe_ep_push_part": (_I, [_P, _P, _I, _I, _I, _I, _P, _I, _P]),
    "mp_moe_ep_push_signal": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P]),
    "mp_moe_combine_after_peers": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P]),
}


class HostLinear(ctypes.Structure):
    """``mp_host_linear`` of the C header: one entry of ``mp_w4a16_linear_decode_host_many``."""
    _fields_ = [("x_host_f16", c_void_p), ("x_stage_f16", c_void_p), ("packed_i32", c_void_p), ("sz_f16x2", c_void_p),
                ("bias_f16", c_void_p), ("y_stage_f16", c_void_p), ("y_host_f16", c_void_p),
                ("M", c_int), ("N", c_int), ("K", c_int), ("group", c_int),
                ("workspace", c_void_p), ("workspace_bytes", c_size_t)]


class MindPipeKernelError(RuntimeError):
    """A C-ABI call returned a negative status."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mindpipe_b200.build` "
                "(there is no fallback path for the quantized kernels)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is absent
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, op: str, **shapes) -> None:
    if status == 0:
        return
    lib = load()
    msg = lib.mp_status_string(status).decode()
    detail = ", ".join(f"{k}={v}" for k, v in shapes.items())
    extra = f", cudaError={lib.mp_last_cuda_error()}" if status == -5 else ""
    raise MindPipeKernelError(f"{op} failed with status {status} ({msg}{extra}); {detail}")
