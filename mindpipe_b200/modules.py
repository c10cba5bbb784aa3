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
        self._host_stage = {}     # (row count, stream) -> (x, y) device staging buffers of forward_host
        self._host_plans = {}     # (x_host ptr, y_host ptr, shape, stream, weight-side ptrs) -> raw call of forward_host
        self._derived_from = None  # (address, version) of every tensor _scale_zero was built from
        self.register_load_state_dict_post_hook(VllmPackedInt4Linear._state_loaded)

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
    def _weight_side_state(self):
        return tuple((t.data_ptr(), t._version) for t in (self.weight_scale, self.weight_zero_point) if t is not None)

    def process_weights_after_loading(self) -> None:
        """Build the group-major (scale, zero) buffer the GEMM kernels read."""
        self._scale_zero = ops.w4a16_prepare(self.weight_scale, self.weight_zero_point, self.in_features)
        self._derived_from = self._weight_side_state()
        self._host_plans = {}            # they hold the old buffer's address

    @staticmethod
    def _state_loaded(module, incompatible_keys) -> None:
        """``load_state_dict`` copied new scales / zero points into the buffers: the derived layout is stale."""
        module._scale_zero = None
        module._host_plans = {}

    def _ensure_prepared(self) -> None:
        """(Re)build the derived buffer when it is missing or when scales / zero points were replaced or
        written in place since it was built (tensor version counters catch ``copy_`` and friends)."""
        if self._scale_zero is None or self._derived_from != self._weight_side_state():
            self.process_weights_after_loading()

    def dequantize(self) -> torch.Tensor:
        """fp16 ``[N, K]`` weights, bit-identical to the reference's fake-quant weight."""
        return ops.w4a16_dequant(self.weight_packed, self.weight_scale, self.weight_zero_point,
                                 self.out_features, self.in_features)

    def _apply(self, fn, *args, **kwargs):
        self._scale_zero = None          # moved/cast: rebuild lazily on the new device
        self._host_stage = {}
        self._host_plans = {}
        return super()._apply(fn, *args, **kwargs)

    # -- forward ------------------------------------------------------------
    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._ensure_prepared()
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = ops.w4a16_linear(x2, self.weight_packed, self._scale_zero, self.bias)
        return y.reshape(*shape[:-1], self.out_features)

    def forward_host(self, x_host: torch.Tensor, y_host: torch.Tensor | None = None, stream=None,
                     zero_copy_output: bool = False) -> torch.Tensor:
        """Decode (<= 16 rows) on a CPU fp16 tensor, as the reference's CPU forward takes it: the H2D
        copy, the kernel and the D2H copy are enqueued on ``stream`` (default: the current stream) and
        the call returns at once; read ``y_host`` after synchronising.  Staging buffers are kept per row
        count and stream (calls on different streams may overlap, so they do not share staging), and a call
        that repeats an earlier one's buffers (same ``x_host`` / ``y_host`` storage, stream and weight-side
        tensors, as a serving loop with fixed pinned buffers does) skips the argument checks and goes
        straight to the library; with ``zero_copy_output`` such a repeated call also lets the kernel store the
        result into the pinned ``y_host`` directly (through its device-side address) instead of staging it and
        copying -- the same bits and one enqueue less, but the kernel's stores then cross PCIe: measured 3 % more
        throughput with several steps in flight and 17 % more latency for a lone call, hence off by default."""
        self._ensure_prepared()
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
        key = (x_host.data_ptr(), None if y_host is None else y_host.data_ptr(), tuple(x_host.shape), st,
               self.weight_packed.data_ptr(), self._scale_zero.data_ptr(),
               None if self.bias is None else self.bias.data_ptr(), zero_copy_output)
        plan = self._host_plans.get(key)
        if plan is not None:
            call, args, y_keep, shapes, _keep = plan
            status = call(*args, st)
            if status != 0:
                from . import _lib
                _lib.check(status, "w4a16_linear_decode_host", **shapes)
            return y_keep
        m = x_host.shape[0]
        stage = self._host_stage.get((m, st))
        if stage is None:
            dev = self.weight_packed.device
            # scratch of this (row count, stream) pair, when the library's choice for the shape needs one: calls on
            # one stream run in order, so they may share it
            ws = None
            if 0 < m <= 16 and ops.w4a16_decode_kernel_choice(m, self.out_features, self.in_features) == "umma":
                ws = ops.new_workspace(ops.w4a16_decode_workspace_bytes(m, self.out_features, self.in_features), dev)
            stage = (torch.empty((m, self.in_features), dtype=torch.float16, device=dev),
                     torch.empty((m, self.out_features), dtype=torch.float16, device=dev), ws)
            self._host_stage[(m, st)] = stage
        if stream is None:
            y = ops.w4a16_linear_decode_host(x_host, self.weight_packed, self._scale_zero, self.bias, y_host=y_host,
                                             x_stage=stage[0], y_stage=stage[1], workspace=stage[2])
        else:
            with torch.cuda.stream(stream):
                y = ops.w4a16_linear_decode_host(x_host, self.weight_packed, self._scale_zero, self.bias,
                                                 y_host=y_host, x_stage=stage[0], y_stage=stage[1], workspace=stage[2])
        if y_host is not None and x_host.is_pinned() and y_host.is_pinned():
            # validated once: remember the raw call (the tensors are kept alive by the plan)
            import ctypes
            from . import _lib
            y_out, y_copy = stage[1].data_ptr(), y_host.data_ptr()
            if zero_copy_output:
                # pinned memory is mapped into the device's address space: let the kernel store the result there
                # itself instead of a staging buffer plus a D2H copy (one call less per linear on the host)
                alias = ctypes.c_void_p()
                if _lib.load().mp_host_buffer_device_alias(y_host.data_ptr(), y_host.numel() * 2,
                                                           ctypes.byref(alias)) == 0 and alias.value:
                    y_out, y_copy = alias.value, None
            args = (x_host.data_ptr(), stage[0].data_ptr(), self.weight_packed.data_ptr(), self._scale_zero.data_ptr(),
                    None if self.bias is None else self.bias.data_ptr(), y_out, y_copy,
                    m, self.out_features, self.in_features, self.group_size,
                    None if stage[2] is None else stage[2].data_ptr(), 0 if stage[2] is None else stage[2].numel())
            if len(self._host_plans) >= 64:
                self._host_plans.clear()
            self._host_plans[key] = (_lib.load().mp_w4a16_linear_decode_host_ws, args, y_host,
                                     dict(M=m, N=self.out_features, K=self.in_features, group=self.group_size),
                                     (x_host, stage, self._scale_zero))
        return y

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"w_bit=4, group_size={self.group_size}, asymmetric={self.weight_zero_point is not None}")


_HOST_MANY_PLANS: dict = {}


def forward_host_many(linears, x_hosts, y_hosts, stream=None):
    """``forward_host`` of several independent ``VllmPackedInt4Linear`` modules on ONE stream in one library
    call: all H2D copies first, then the kernels back to back (so that under ``mp_set_programmatic_launch(1)`` each
    fetches its weights while the one before drains), then the D2H copies.  For linears that do not depend on one
    another -- the q/k/v or gate/up projections of a decoder layer.  ``x_hosts`` / ``y_hosts`` are pinned CPU fp16
    tensors, one pair per module (<= 16 rows); returns ``y_hosts``, valid once the stream is synchronised.  The
    first call with a given set of modules, buffers and stream goes through each module's own ``forward_host``
    (argument checks, staging and scratch buffers); repeats reuse the recorded call."""
    from . import _lib
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
    key = (st,) + tuple((id(m), x.data_ptr(), y.data_ptr(), x.shape[0]) for m, x, y in zip(linears, x_hosts, y_hosts))
    plan = _HOST_MANY_PLANS.get(key)
    if plan is not None:
        for m in linears:
            m._ensure_prepared()
        calls, derived, _keep = plan
        if all(m._scale_zero is z and m.weight_packed.data_ptr() == p and (None if m.bias is None else m.bias.data_ptr()) == b
               for m, (z, p, b) in zip(linears, derived)):
            status = _lib.load().mp_w4a16_linear_decode_host_many(calls, len(derived), st)
            if status != 0:
                _lib.check(status, "w4a16_linear_decode_host_many", count=len(derived))
            return y_hosts
    if not (len(linears) == len(x_hosts) == len(y_hosts)) or not linears:
        raise ValueError("forward_host_many takes one (x_host, y_host) pair per module")
    if len({id(m) for m in linears}) != len(linears):
        raise ValueError("a module may appear once per call (its staging buffers are per stream)")
    for m, x, y in zip(linears, x_hosts, y_hosts):
        if not isinstance(m, VllmPackedInt4Linear):
            raise TypeError("forward_host_many expects VllmPackedInt4Linear modules")
        if y is None or not x.is_pinned() or not y.is_pinned():
            raise ValueError("forward_host_many needs pinned x_host and y_host tensors")
        m.forward_host(x, y, stream=stream, zero_copy_output=False)      # validates; creates staging and scratch
    calls = (_lib.HostLinear * len(linears))()
    for c, m, x, y in zip(calls, linears, x_hosts, y_hosts):
        xs, ys, ws = m._host_stage[(x.shape[0], st)]
        c.x_host_f16, c.x_stage_f16 = x.data_ptr(), xs.data_ptr()
        c.packed_i32, c.sz_f16x2 = m.weight_packed.data_ptr(), m._scale_zero.data_ptr()
        c.bias_f16 = None if m.bias is None else m.bias.data_ptr()
        c.y_stage_f16, c.y_host_f16 = ys.data_ptr(), y.data_ptr()
        c.M, c.N, c.K, c.group = x.shape[0], m.out_features, m.in_features, m.group_size
        c.workspace = None if ws is None else ws.data_ptr()
        c.workspace_bytes = 0 if ws is None else ws.numel()
    if len(_HOST_MANY_PLANS) >= 256:
        _HOST_MANY_PLANS.clear()
    _HOST_MANY_PLANS[key] = (calls, [(m._scale_zero, m.weight_packed.data_ptr(), None if m.bias is None else m.bias.data_ptr())
                                     for m in linears], (list(linears), list(x_hosts), list(y_hosts)))
    return y_hosts


class SmoothQuantLinear(nn.Module):
    """Real-int twin of the reference's ``SmoothQuantLinear``
    (algorithm/quantization/ptq/smoothquant/source/smoothquant/fake_quant.py:38-121).

    Same constructor, ``from_float`` and ``forward(x)``; where the reference
    keeps a fake-quantised fp16 ``weight`` and multiplies in fp16, this module
    keeps the int8 codes and per-channel scales (buffer names of the W8A8
    exporter, scripts/repro/export_fp16_to_ascend_w8a8_dynamic_probe.py:175-195:
    ``weight``, ``weight_scale``, ``weight_offset``) and runs per-token int8
    activation quantisation followed by the int8 tensor-core GEMM with an
    int32-accumulate, scale epilogue.  The codes and scales are exactly those
    of the reference's fp16 arithmetic (fake_quant.py:10-31).
    """

    def __init__(self, in_features, out_features, bias=True, weight_bits=8, activation_bits=8,
                 act_quant="per_token", quantize_output=False, dtype=torch.float16):
        super().__init__()
        if act_quant != "per_token":
            raise ValueError(f"Invalid act_quant: {act_quant}")
        if int(weight_bits) != 8 or int(activation_bits) != 8:
            raise ValueError("the integer kernels implement weight_bits=8, activation_bits=8")
        if dtype != torch.float16:
            raise ValueError("the integer kernels take fp16 activations")
        self.in_features = in_features
        self.out_features = out_features
        self.weight_bits = int(weight_bits)
        self.activation_bits = int(activation_bits)
        self.register_buffer("weight", torch.zeros((out_features, in_features), dtype=torch.int8))
        self.register_buffer("weight_scale", torch.zeros((out_features, 1), dtype=dtype))
        self.register_buffer("weight_offset", torch.zeros((out_features, 1), dtype=dtype))
        if bias:
            self.register_buffer("bias", torch.zeros((out_features,), dtype=dtype))
        else:
            self.register_buffer("bias", None)
        self.weight_quant_name = "per_channel"
        self.act_quant_name = act_quant
        self.quantize_output = bool(quantize_output)
        self.output_quant_name = act_quant if quantize_output else "none"
        self._weight_scale_fp32 = None

    @staticmethod
    @torch.no_grad()
    def from_float(module, weight_bits=8, activation_bits=8, act_quant="per_token", quantize_output=False):
        assert isinstance(module, nn.Linear)
        new = SmoothQuantLinear(module.in_features, module.out_features, module.bias is not None,
                                weight_bits=weight_bits, activation_bits=activation_bits, act_quant=act_quant,
                                quantize_output=quantize_output, dtype=module.weight.dtype)
        new = new.to(device=module.weight.device)
        q, s, _ = ops.act_quant_per_token(module.weight.detach().contiguous())   # per output channel
        new.weight = q
        new.weight_scale = s.to(module.weight.dtype).reshape(-1, 1)
        new.weight_offset = torch.zeros_like(new.weight_scale)
        if module.bias is not None:
            new.bias = module.bias.detach().clone()
        return new

    def process_weights_after_loading(self) -> None:
        """fp32 copy of the per-channel scales, as the runtime method keeps
        (acceleration/runtime_patches/vllm_ascend.patch:4029-4031)."""
        self._weight_scale_fp32 = self.weight_scale.detach().flatten().to(torch.float32).contiguous()
        self._derived_from = (self.weight_scale.data_ptr(), self.weight_scale._version)

    def _apply(self, fn, *args, **kwargs):
        self._weight_scale_fp32 = None
        return super()._apply(fn, *args, **kwargs)

    def _ensure_prepared(self) -> None:
        """Rebuild the fp32 scales when missing or when ``weight_scale`` was replaced, loaded
        (``load_state_dict`` copies in place) or edited in place since they were derived."""
        if self._weight_scale_fp32 is None or \
                getattr(self, "_derived_from", None) != (self.weight_scale.data_ptr(), self.weight_scale._version):
            self.process_weights_after_loading()

    def dequantize(self) -> torch.Tensor:
        """The reference's fake-quantised fp16 weight: ``f16(code * scale)``."""
        return (self.weight.to(torch.float16) * self.weight_scale).to(torch.float16)

    @torch.no_grad()
    def forward(self, x):
        """``x`` is an fp16 tensor, or a ``(int8 codes, per-token scale)`` pair produced upstream
        (the tuple input of AscendW8A8DynamicLinearMethod.apply, vllm_ascend.patch:3945-3962)."""
        self._ensure_prepared()
        if isinstance(x, tuple):
            q, s = x
            lead = q.shape[:-1]
            q2 = q.reshape(-1, q.shape[-1])
            s2 = s.reshape(-1).to(torch.float32)
        else:
            lead = x.shape[:-1]
            x2 = x.reshape(-1, x.shape[-1])
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            q2, s2, _ = ops.act_quant_per_token(x2)
        y = ops.w8a8_gemm(q2.contiguous(), s2.contiguous(), self.weight, self._weight_scale_fp32, self.bias)
        if self.quantize_output:
            _, _, y = ops.act_quant_per_token(y, want_codes=False, want_fake=True)
        return y.reshape(*lead, self.out_features)

    def __repr__(self):
        return (f"SmoothQuantLinear({self.in_features}, {self.out_features}, bias={self.bias is not None}, "
                f"weight_bits={self.weight_bits}, activation_bits={self.activation_bits}, "
                f"weight_quant={self.weight_quant_name}, act_quant={self.act_quant_name}, "
                f"output_quant={self.output_quant_name}, int8=True)")


class QuantLinear(nn.Module):
    """Real-int twin of OmniQuant's ``QuantLinear``
    (algorithm/quantization/ptq/omniquant/source/omniquant/int_linear.py:10-59) for the W8A8 recipe:
    per-output-channel asymmetric 8-bit weights and per-token dynamic asymmetric 8-bit activations
    (``UniformAffineQuantizer`` with ``symmetric=False``, quantizer.py:124-150).  Same constructor
    shape (``org_module, weight_quant_params, act_quant_params, disable_input_quant``) and
    ``set_quant_state``; the forward runs on unsigned 8-bit codes with the zero-point correction
    folded into the tensor-core GEMM's epilogue.
    """

    def __init__(self, org_module: nn.Linear, weight_quant_params: dict | None = None,
                 act_quant_params: dict | None = None, disable_input_quant: bool = False):
        super().__init__()
        wq, aq = dict(weight_quant_params or {}), dict(act_quant_params or {})
        for name, prm in (("weight", wq), ("activation", aq)):
            if int(prm.get("n_bits", 8)) != 8 or prm.get("symmetric", False) or prm.get("group_size") or \
                    prm.get("lwc", False) or prm.get("disable_zero_point", False):
                raise ValueError(f"{name} quantiser: the integer kernels implement 8-bit, asymmetric, "
                                 "ungrouped quantisation without learned clipping")
        if disable_input_quant:
            raise ValueError("disable_input_quant=True (fp16 activations) is not an integer path")
        w = org_module.weight.detach()
        if w.dtype != torch.float16:
            raise TypeError(f"expected an fp16 weight, got {w.dtype}")
        self.in_features = org_module.in_features
        self.out_features = org_module.out_features
        q, s, z, rs, _ = ops.affine_quant_per_row(w.contiguous())
        self.register_buffer("weight", q)                      # uint8 codes [N, K]
        self.register_buffer("scales", s)                      # names of register_scales_and_zeros (quantizer.py:152-155)
        self.register_buffer("zeros", z)
        self.register_buffer("weight_rowsum", rs)
        if org_module.bias is not None:
            self.register_buffer("bias", org_module.bias.detach().clone())
        else:
            self.bias = None
        self.use_weight_quant = True
        self.use_act_quant = True

    def set_quant_state(self, weight_quant: bool = False, act_quant: bool = False) -> None:
        if not (weight_quant and act_quant):
            raise ValueError("this module only holds the quantised weight; both quantisers stay on")
        self.use_weight_quant, self.use_act_quant = True, True

    def dequantize(self) -> torch.Tensor:
        """The reference's fake-quantised weight ``f16(f16(u - zp) * s)``."""
        return ((self.weight.to(torch.float16) - self.zeros.to(torch.float16)[:, None])
                * self.scales.to(torch.float16)[:, None]).to(torch.float16)

    @torch.no_grad()
    def forward(self, input: torch.Tensor) -> torch.Tensor:
        lead = input.shape[:-1]
        x2 = input.reshape(-1, input.shape[-1]).contiguous()
        q, s, z, rs, _ = ops.affine_quant_per_row(x2)
        y = ops.w8a8_affine_gemm(q, s, z, rs, self.weight, self.scales, self.zeros, self.weight_rowsum, self.bias)
        return y.reshape(*lead, self.out_features)


class W8A8DynamicLinearMethod:
    """Linear-method style entry, mirroring ``AscendW8A8DynamicLinearMethod``
    (acceleration/runtime_patches/vllm_ascend.patch:3933-4033): ``apply(layer, x, bias, tp_rank)``
    where ``layer`` carries ``weight`` int8 ``[N,K]``, ``weight_scale`` and an optional
    ``_ascend_quant_config`` dict with ``output_dtype``, ``pertoken_scale`` and ``return_scale``."""

    def process_weights_after_loading(self, layer) -> None:
        layer.weight_scale.data = layer.weight_scale.data.flatten()
        layer.weight_scale_fp32 = layer.weight_scale.data.to(torch.float32).contiguous()
        if hasattr(layer, "weight_offset"):
            layer.weight_offset.data = layer.weight_offset.data.flatten()

    @torch.no_grad()
    def apply(self, layer, x, bias=None, tp_rank=0):
        config = getattr(layer, "_ascend_quant_config", {})
        output_shape = None
        if not isinstance(x, tuple):
            output_dtype = config.get("output_dtype", x.dtype)
            if x.dim() > 2:
                output_shape = x.shape[:-1]
                x = x.reshape(-1, x.shape[-1])
            quantized_x, dynamic_scale, _ = ops.act_quant_per_token(x.contiguous())
        else:
            output_dtype = config.get("output_dtype", getattr(layer, "params_dtype", torch.float16))
            quantized_x, dynamic_scale = x
        if not config.get("pertoken_scale", True):
            raise NotImplementedError("pertoken_scale=False (static activation scale) is not part of this path")
        if not hasattr(layer, "weight_scale_fp32"):
            self.process_weights_after_loading(layer)
        scale = dynamic_scale.flatten().to(torch.float32).contiguous()
        if output_dtype == torch.int32:
            output = ops.w8a8_gemm_i32(quantized_x.contiguous(), layer.weight)
        elif output_dtype == torch.float16:
            output = ops.w8a8_gemm(quantized_x.contiguous(), scale, layer.weight, layer.weight_scale_fp32, bias)
        else:
            raise NotImplementedError(f"output_dtype {output_dtype} (fp16 and int32 are implemented)")
        if output_shape is not None:
            output = output.reshape(*output_shape, output.shape[-1])
            dynamic_scale = dynamic_scale.reshape(*output_shape)
        return (output, dynamic_scale) if config.get("return_scale", False) else output


class SmoothQuantPackedMoeExperts(nn.Module):
    """Real-int twin of the reference's ``SmoothQuantPackedMoeExperts``
    (fake_quant.py:124-198): same constructor (``gate_up_proj[E,2I,H]``, ``down_proj[E,H,I]``,
    ``act_fn``), ``from_float`` and ``forward(hidden_states, top_k_index, top_k_weights)``.

    The expert weights are stored as int8 codes with per-(expert, output row) scales; the
    forward is routing + gather + per-token quant, grouped int8 GEMM1 with SwiGLU, re-quant,
    grouped int8 GEMM2 and the weighted scatter-add.  ``expert_range`` restricts the module
    to the experts one GPU owns (expert parallelism): rows routed elsewhere contribute zero.
    """

    def __init__(self, gate_up_proj, down_proj, act_fn=None, *, weight_bits=8, activation_bits=8,
                 expert_range: tuple[int, int] | None = None, num_experts: int | None = None):
        super().__init__()
        if int(weight_bits) != 8 or int(activation_bits) != 8:
            raise ValueError("the integer kernels implement weight_bits=8, activation_bits=8")
        if act_fn is not None and not isinstance(act_fn, nn.SiLU) and getattr(act_fn, "__name__", "") != "silu":
            raise ValueError("the fused epilogue implements SiLU (SwiGLU) experts")
        local = int(gate_up_proj.shape[0])
        self.expert_range = (0, local) if expert_range is None else (int(expert_range[0]), int(expert_range[1]))
        if self.expert_range[1] - self.expert_range[0] != local:
            raise ValueError("expert_range does not match the number of expert weight slabs")
        self.num_experts = int(num_experts) if num_experts is not None else self.expert_range[1]
        self.hidden_dim = int(gate_up_proj.shape[2])
        self.intermediate_dim = int(down_proj.shape[2])
        self.weight_bits = int(weight_bits)
        self.activation_bits = int(activation_bits)
        self.act_fn = act_fn
        gq, gs = self._quantize(gate_up_proj)
        dq, ds = self._quantize(down_proj)
        self.register_buffer("gate_up_proj", gq)
        self.register_buffer("gate_up_proj_scale", gs)
        self.register_buffer("down_proj", dq)
        self.register_buffer("down_proj_scale", ds)

    @staticmethod
    @torch.no_grad()
    def _quantize(w):
        if w.dtype == torch.int8:
            raise TypeError("pass float expert weights; they are quantised here")
        q, s, _ = ops.act_quant_per_token(w.detach().to(torch.float16).contiguous())   # per (expert, out row)
        return q, s

    @staticmethod
    def from_float(module, weight_bits=8, activation_bits=8, expert_range=None, num_experts=None):
        return SmoothQuantPackedMoeExperts(module.gate_up_proj.detach(), module.down_proj.detach(), module.act_fn,
                                           weight_bits=weight_bits, activation_bits=activation_bits,
                                           expert_range=expert_range, num_experts=num_experts)

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor):
        shape = hidden_states.shape
        hs = hidden_states.reshape(-1, shape[-1]).contiguous()
        ids = top_k_index.reshape(hs.shape[0], -1).to(torch.int32).contiguous()
        w = top_k_weights.reshape(hs.shape[0], -1).to(torch.float16).contiguous()
        lo, hi = self.expert_range
        routing = ops.moe_route_gather_quant(hs, ids, lo, hi)
        d = ops.moe_expert_stage(routing.routed_q, routing.routed_scale, routing.plan, hi - lo,
                                 self.gate_up_proj, self.gate_up_proj_scale, self.down_proj, self.down_proj_scale)
        out = ops.moe_combine(d, routing.dest_row, ids, w, hs.shape[0])
        return out.reshape(shape)

    def __repr__(self):
        return (f"SmoothQuantPackedMoeExperts(num_experts={self.num_experts}, hidden_dim={self.hidden_dim}, "
                f"intermediate_dim={self.intermediate_dim}, weight_bits={self.weight_bits}, "
                f"activation_bits={self.activation_bits}, local_experts={self.expert_range})")
