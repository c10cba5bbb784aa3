"""Real-quant twins of the reference's Linear modules.

The classes keep the reference's names, constructor arguments and buffer
names, but hold integer weights and run the sm_100a kernels:

* :class:`VllmPackedInt4Linear` -- the export-only module of
  algorithm/quantization/exporters/vllm.py:57-86 (its ``forward`` raises
  there).  Here it runs W4A16: packed little-nibble-first int4 codes, fp16
  group scales and, for the asymmetric format AWQ's ``pseudo_quantize_tensor``
  defines (algorithm/quantization/ptq/awq/source/awq/quantize/quantizer.py:
  63-105), a packed zero-point buffer.  Its results are those of the
  reference's W4A16 forward, ``F.linear(x, pseudo_quantize_tensor(W))``.
"""
from __future__ import annotations

import torch
from torch import nn

from . import ops


class VllmPackedInt4Linear(nn.Module):
    """W4A16 linear holding packed int4 weights.

    Buffers (names of the reference's export format, exporters/vllm.py:70-81):
    ``weight_packed`` int32 ``[N, K/8]``, ``weight_scale`` fp16 ``[N, K/g]``,
    ``weight_shape`` int64 ``[2] = (N, K)``, optional ``bias``; plus
    ``weight_zero_point`` int32 ``[N, ceil(K/g/8)]`` for the asymmetric
    format (absent = symmetric export, zero point 8).
    """

    def __init__(self, *, packed_weight: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None,
                 in_features: int, out_features: int, zero_point: torch.Tensor | None = None) -> None:
        super().__init__()
        self.register_buffer("weight_packed", packed_weight.detach().contiguous())
        self.register_buffer("weight_scale", scale.detach().to(torch.float16).contiguous())
        self.register_buffer("weight_shape", torch.tensor([out_features, in_features], dtype=torch.int64))
        if zero_point is not None:
            self.register_buffer("weight_zero_point", zero_point.detach().contiguous())
        else:
            self.weight_zero_point = None
        if bias is not None:
            self.register_buffer("bias", bias.detach().contiguous())
        else:
            self.bias = None
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        if self.weight_packed.dtype != torch.int32 or tuple(self.weight_packed.shape) != (
                self.out_features, (self.in_features + 7) // 8):
            raise ValueError(
                f"packed_weight must be int32 [{self.out_features}, {(self.in_features + 7) // 8}], got "
                f"{self.weight_packed.dtype} {tuple(self.weight_packed.shape)}")
        if self.weight_scale.dim() != 2 or self.weight_scale.shape[0] != self.out_features or (
                self.in_features % self.weight_scale.shape[1]):
            raise ValueError(f"scale shape {tuple(self.weight_scale.shape)} does not divide in_features")
        self.group_size = self.in_features // int(self.weight_scale.shape[1])
        self._scale_zero = None   # kernel-side layout, built on first use

    # -- construction -------------------------------------------------------
    @staticmethod
    @torch.no_grad()
    def from_float(module: nn.Linear, w_bit: int = 4, group_size: int = 128, zero_point: bool = True):
        """Quantise an ``nn.Linear`` on its (CUDA) device with the reference's AWQ arithmetic."""
        if not isinstance(module, nn.Linear):
            raise TypeError("from_float expects nn.Linear")
        if w_bit != 4 or not zero_point:
            raise ValueError("only asymmetric 4-bit group quantisation is implemented")
        w = module.weight.detach()
        if w.dtype != torch.float16:
            raise TypeError(f"expected an fp16 weight, got {w.dtype}")
        packed, scale, zeros, _ = ops.w4a16_quantize(w.contiguous(), group_size)
        return VllmPackedInt4Linear(packed_weight=packed, scale=scale,
                                    bias=None if module.bias is None else module.bias.detach().clone(),
                                    in_features=module.in_features, out_features=module.out_features,
                                    zero_point=zeros)

    # -- weights ------------------------------------------------------------
    def process_weights_after_loading(self) -> None:
        """Build the group-major (scale, zero) buffer the GEMM kernels read."""
        self._scale_zero = ops.w4a16_prepare(self.weight_scale, self.weight_zero_point, self.in_features)

    def dequantize(self) -> torch.Tensor:
        """fp16 ``[N, K]`` weights, bit-identical to the reference's fake-quant weight."""
        return ops.w4a16_dequant(self.weight_packed, self.weight_scale, self.weight_zero_point,
                                 self.out_features, self.in_features)

    def _apply(self, fn, *args, **kwargs):
        self._scale_zero = None          # moved/cast: rebuild lazily on the new device
        return super()._apply(fn, *args, **kwargs)

    # -- forward ------------------------------------------------------------
    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._scale_zero is None:
            self.process_weights_after_loading()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = ops.w4a16_linear(x2, self.weight_packed, self._scale_zero, self.bias)
        return y.reshape(*shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"w_bit=4, group_size={self.group_size}, asymmetric={self.weight_zero_point is not None}")
