"""Registration of the kernels as ``torch.ops.mindpipe_b200.*`` custom ops.

The reference installs its native op through a loader that compiles the
bridge, then registers an op with a real and a fake (meta) implementation so
that ``torch.compile(fullgraph=True)`` and graph capture see one opaque call
(acceleration/runtime_patches/vllm.patch:114-208 for the two implementations,
:291-306 for ``load_and_register``).  This module is the same slot for the
B200 library: ``load_and_register()`` is idempotent and locked, loads the
shared library (raising if it is missing) and defines

* ``mindpipe_b200::w4a16_linear(x, weight_packed, scale_zero, bias?) -> y``
* ``mindpipe_b200::act_quant_per_token(x) -> (codes, scale)``
* ``mindpipe_b200::w8a8_linear(x, weight, weight_scale, bias?) -> y``
* ``mindpipe_b200::w8a8_gemm(qx, x_scale, weight, weight_scale, bias?) -> y``
* ``mindpipe_b200::moe_w8a8_experts(hidden, top_k_index, top_k_weights, w13, w13_scale, w2, w2_scale) -> out``
* ``mindpipe_b200::grouped_swiglu_loop_out(x, weights, batched_weight, group_list, weight_scales,
  batched_weight_scale, x_scale, min_tokens, layer_idx) -> (codes, scales)`` -- the reference's own op name and
  argument list (vllm.patch:114-208)

Each fake implementation only computes output shapes and dtypes.
"""
from __future__ import annotations

import threading
from typing import List, Optional, Tuple

import torch

_lock = threading.Lock()
_registered = False
NAMESPACE = "mindpipe_b200"


def load_and_register():
    """Load the CUDA library and register the ops once; returns ``torch.ops.mindpipe_b200``."""
    global _registered
    if _registered:
        return getattr(torch.ops, NAMESPACE)
    with _lock:
        if _registered:
            return getattr(torch.ops, NAMESPACE)
        from . import _lib, ops
        _lib.load()                                   # no library, no ops: fail here, not at first call

        @torch.library.custom_op(f"{NAMESPACE}::w4a16_linear", mutates_args=())
        def w4a16_linear(x: torch.Tensor, weight_packed: torch.Tensor, scale_zero: torch.Tensor,
                         bias: Optional[torch.Tensor] = None) -> torch.Tensor:
            lead = x.shape[:-1]
            y = ops.w4a16_linear(x.reshape(-1, x.shape[-1]).contiguous(), weight_packed, scale_zero, bias)
            return y.reshape(*lead, weight_packed.shape[0])

        @w4a16_linear.register_fake
        def _(x, weight_packed, scale_zero, bias=None):
            return x.new_empty((*x.shape[:-1], weight_packed.shape[0]))

        @torch.library.custom_op(f"{NAMESPACE}::act_quant_per_token", mutates_args=())
        def act_quant_per_token(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
            q, s, _ = ops.act_quant_per_token(x.contiguous())
            return q, s

        @act_quant_per_token.register_fake
        def _(x):
            return x.new_empty(x.shape, dtype=torch.int8), x.new_empty(x.shape[:-1], dtype=torch.float32)

        @torch.library.custom_op(f"{NAMESPACE}::w8a8_gemm", mutates_args=())
        def w8a8_gemm(qx: torch.Tensor, x_scale: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                      bias: Optional[torch.Tensor] = None) -> torch.Tensor:
            return ops.w8a8_gemm(qx, x_scale, weight, weight_scale, bias)

        @w8a8_gemm.register_fake
        def _(qx, x_scale, weight, weight_scale, bias=None):
            return qx.new_empty((qx.shape[0], weight.shape[0]), dtype=torch.float16)

        @torch.library.custom_op(f"{NAMESPACE}::w8a8_linear", mutates_args=())
        def w8a8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                        bias: Optional[torch.Tensor] = None) -> torch.Tensor:
            lead = x.shape[:-1]
            q, s, _ = ops.act_quant_per_token(x.reshape(-1, x.shape[-1]).contiguous())
            y = ops.w8a8_gemm(q, s, weight, weight_scale.flatten().to(torch.float32).contiguous(), bias)
            return y.reshape(*lead, weight.shape[0])

        @w8a8_linear.register_fake
        def _(x, weight, weight_scale, bias=None):
            return x.new_empty((*x.shape[:-1], weight.shape[0]))

        @torch.library.custom_op(f"{NAMESPACE}::moe_w8a8_experts", mutates_args=())
        def moe_w8a8_experts(hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
                             w13: torch.Tensor, w13_scale: torch.Tensor, w2: torch.Tensor,
                             w2_scale: torch.Tensor) -> torch.Tensor:
            hs = hidden.reshape(-1, hidden.shape[-1]).contiguous()
            ids = top_k_index.reshape(hs.shape[0], -1).to(torch.int32).contiguous()
            wts = top_k_weights.reshape(hs.shape[0], -1).to(torch.float16).contiguous()
            e = w13.shape[0]
            routing = ops.moe_route_gather_quant(hs, ids, 0, e)
            d = ops.moe_expert_stage(routing.routed_q, routing.routed_scale, routing.plan, e, w13, w13_scale, w2,
                                     w2_scale)
            return ops.moe_combine(d, routing.dest_row, ids, wts, hs.shape[0]).reshape(hidden.shape)

        @moe_w8a8_experts.register_fake
        def _(hidden, top_k_index, top_k_weights, w13, w13_scale, w2, w2_scale):
            return torch.empty_like(hidden)

        @torch.library.custom_op(f"{NAMESPACE}::grouped_swiglu_loop_out", mutates_args=())
        def grouped_swiglu_loop_out(x: torch.Tensor, weights: List[torch.Tensor], batched_weight: torch.Tensor,
                                    group_list: torch.Tensor, weight_scales: List[torch.Tensor],
                                    batched_weight_scale: torch.Tensor, x_scale: torch.Tensor, min_tokens: int,
                                    layer_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
            return ops.grouped_swiglu_loop_out(x, weights, batched_weight, group_list, weight_scales,
                                               batched_weight_scale, x_scale, min_tokens, layer_idx)

        @grouped_swiglu_loop_out.register_fake
        def _(x, weights, batched_weight, group_list, weight_scales, batched_weight_scale, x_scale, min_tokens,
              layer_idx):
            if not weights or len(weights) != len(weight_scales):
                raise RuntimeError("loop-out requires equal non-empty weight lists")
            chunks = len(weights)
            if batched_weight.shape[0] != chunks or batched_weight_scale.shape[0] != chunks:
                raise RuntimeError("loop-out batched weight has an invalid chunk count")
            width = batched_weight_scale.shape[-1] // 2
            return (x.new_empty((chunks, x.shape[0], width), dtype=torch.int8),
                    x.new_empty((chunks, x.shape[0]), dtype=torch.float32))

        _registered = True
    return getattr(torch.ops, NAMESPACE)
