"""Model-level installers: put the real-quant twins where the reference puts its pseudo-quant modules.

Two entry points with the reference's names, arguments and error behaviour:

* :func:`quantize_model` -- SmoothQuant's installer
  (``ptq/smoothquant/source/smoothquant/fake_quant.py:441-458`` -> ``quantize_llama_like`` ``:227-437``):
  walks the decoder layers of a llama-like model, replaces the attention and MLP projections by
  :class:`~mindpipe_b200.modules.SmoothQuantLinear` and packed MoE experts by
  :class:`~mindpipe_b200.modules.SmoothQuantPackedMoeExperts`, and returns the qualified names it replaced.
* :func:`real_quantize_model_weight` -- the real-int counterpart of AWQ's ``pseudo_quantize_model_weight``
  (``ptq/awq/source/awq/quantize/quantizer.py:109-130``): instead of writing fake-quant fp16 weights back into
  every ``nn.Linear`` of every block it replaces the linear by a
  :class:`~mindpipe_b200.modules.VllmPackedInt4Linear` holding the same codes, scales and zero points packed.

:func:`load_exported_state_dict` fills installed twins from a checkpoint in the reference's export formats
(``exporters/vllm.py:224-327``: ``*.weight_packed / weight_scale / weight_shape``; the W8A8 exporter
``scripts/repro/export_fp16_to_ascend_w8a8_dynamic_probe.py:175-195``: ``*.weight / weight_scale / weight_offset``).

The twins quantise on the GPU, so the model's linears must already live on a CUDA device.
"""
from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

from .modules import SmoothQuantLinear, SmoothQuantPackedMoeExperts, VllmPackedInt4Linear

_ATTN_PROJ = ("q_proj", "k_proj", "v_proj")
_MLP_PROJ = ("gate_proj", "up_proj", "down_proj")


def get_blocks(model: nn.Module):
    """The decoder layers, found the way ``awq/quantize/pre_quant.py:47-76`` finds them (text backbones only)."""
    if hasattr(model, "model") and hasattr(model.model, "language_model"):
        return model.model.language_model.layers
    if hasattr(model, "language_model") and hasattr(model.language_model, "layers"):
        return model.language_model.layers
    if hasattr(model, "model") and hasattr(model.model, "layers"):
        return model.model.layers
    if hasattr(model, "layers") and isinstance(model.layers, (nn.ModuleList, list)):
        return model.layers
    raise NotImplementedError(type(model))


def _blocks_prefix(model: nn.Module) -> str:
    layers = get_blocks(model)
    for name, mod in model.named_modules():
        if mod is layers:
            return name
    return "layers"


def get_named_linears(module: nn.Module) -> dict[str, nn.Linear]:
    """``awq/quantize/pre_quant.py:34-35``: every ``nn.Linear`` below ``module`` by its relative name."""
    return {name: m for name, m in module.named_modules() if isinstance(m, nn.Linear)}


def _set_submodule(root: nn.Module, name: str, new: nn.Module) -> None:
    parent = root
    parts = name.split(".")
    for part in parts[:-1]:
        parent = getattr(parent, part)
    setattr(parent, parts[-1], new)


def _require_cuda(linear: nn.Linear, name: str) -> None:
    if linear.weight.device.type != "cuda":
        raise ValueError(f"{name}: the real-quant modules quantise on the GPU; move the model to a CUDA device first")


@torch.no_grad()
def real_quantize_model_weight(model: nn.Module, w_bit: int, q_config: dict, skip: Iterable[str] = ()) -> list[str]:
    """Replace every ``nn.Linear`` of every block by a packed int4 linear.

    ``q_config`` is AWQ's dictionary (``{"zero_point": bool, "q_group_size": int}``).  Only ``w_bit == 4`` and
    positive group sizes exist as kernels; anything else raises ``ValueError`` (the reference would fake-quantise
    it, a real-int format for it does not exist here).  Returns the qualified names that were replaced.
    """
    if w_bit != 4:
        raise ValueError(f"only w_bit=4 has a packed format and kernels, got {w_bit}")
    group = int(q_config.get("q_group_size", 128))
    if group <= 0:
        raise ValueError("per-channel (q_group_size <= 0) int4 has no packed kernel format; use a positive group size")
    zero_point = bool(q_config.get("zero_point", True))
    skip = tuple(skip)
    prefix = _blocks_prefix(model)
    replaced = []
    for i, block in enumerate(get_blocks(model)):
        for name, linear in get_named_linears(block).items():
            if any(s in name for s in skip):
                continue
            qualified = f"{prefix}.{i}.{name}"
            _require_cuda(linear, qualified)
            _set_submodule(block, name, VllmPackedInt4Linear.from_float(linear, w_bit=4, group_size=group,
                                                                         zero_point=zero_point))
            replaced.append(qualified)
    return replaced


def _replace_linear_with_smoothquant(module, proj_name, names, qualified, *, weight_bits, activation_bits, act_quant,
                                     quantize_output=False):
    linear = getattr(module, proj_name)
    _require_cuda(linear, qualified)
    setattr(module, proj_name, SmoothQuantLinear.from_float(linear, weight_bits=weight_bits,
                                                            activation_bits=activation_bits, act_quant=act_quant,
                                                            quantize_output=quantize_output))
    names.append(qualified)


@torch.no_grad()
def quantize_llama_like(model, weight_bits=8, activation_bits=8, act_quant="per_token", quantize_bmm_input=True):
    """``fake_quant.py:227-437`` for the standard attention + (dense | MoE) MLP layer layout: q/k/v (output
    re-quantised when ``quantize_bmm_input``), o, gate/up/down, shared expert, expert lists and packed experts.
    Models without ``config.model_type`` are accepted (the reference needs the type to pick a layout; this
    walker reads the layout off the modules), unsupported layouts raise ``ValueError``."""
    layers = get_blocks(model)
    prefix = _blocks_prefix(model)
    names: list[str] = []
    kw = dict(weight_bits=weight_bits, activation_bits=activation_bits, act_quant=act_quant)
    for i, layer in enumerate(layers):
        lp = f"{prefix}.{i}"
        attn = getattr(layer, "self_attn", None)
        mlp = getattr(layer, "mlp", None)
        if attn is None or mlp is None:
            raise ValueError(f"Unsupported layer layout at {lp}: expected .self_attn and .mlp")
        for proj in _ATTN_PROJ:
            _replace_linear_with_smoothquant(attn, proj, names, f"{lp}.self_attn.{proj}",
                                             quantize_output=quantize_bmm_input, **kw)
        _replace_linear_with_smoothquant(attn, "o_proj", names, f"{lp}.self_attn.o_proj", **kw)
        experts = getattr(mlp, "experts", None)
        if experts is None:
            for proj in _MLP_PROJ:
                _replace_linear_with_smoothquant(mlp, proj, names, f"{lp}.mlp.{proj}", **kw)
            continue
        shared = getattr(mlp, "shared_expert", None)
        if shared is not None:
            for proj in _MLP_PROJ:
                _replace_linear_with_smoothquant(shared, proj, names, f"{lp}.mlp.shared_expert.{proj}", **kw)
        if isinstance(experts, nn.ModuleList):
            for e, expert in enumerate(experts):
                for proj in _MLP_PROJ:
                    _replace_linear_with_smoothquant(expert, proj, names, f"{lp}.mlp.experts.{e}.{proj}", **kw)
        else:
            mlp.experts = SmoothQuantPackedMoeExperts.from_float(experts, weight_bits=weight_bits,
                                                                 activation_bits=activation_bits)
            names.append(f"{lp}.mlp.experts.gate_up_proj")
            names.append(f"{lp}.mlp.experts.down_proj")
    return names


def quantize_model(model, weight_bits=8, activation_bits=8, weight_quant="per_channel", act_quant="per_token",
                   quantize_bmm_input=True):
    """``fake_quant.py:441-458``: same arguments, same ``ValueError`` for anything but per-channel weights."""
    if weight_quant != "per_channel":
        raise ValueError(f"Invalid weight_quant: {weight_quant}")
    return quantize_llama_like(model, weight_bits=weight_bits, activation_bits=activation_bits, act_quant=act_quant,
                               quantize_bmm_input=quantize_bmm_input)


_W4_KEYS = ("weight_packed", "weight_scale", "weight_zero_point", "weight_shape", "bias")
_W8_KEYS = ("weight", "weight_scale", "weight_offset", "bias")


@torch.no_grad()
def load_exported_state_dict(model: nn.Module, state_dict: dict) -> list[str]:
    """Copy an exported real-quant checkpoint into the installed twins; returns the module names it filled.

    W4 modules take ``weight_packed`` / ``weight_scale`` / ``weight_shape`` (+ ``weight_zero_point`` when the
    export is asymmetric); W8A8 modules take ``weight`` (int8) / ``weight_scale`` and check that
    ``weight_offset`` is zero (the kernels are symmetric, as the exporter's dynamic-W8A8 format is).  A module
    whose tensors are missing or mis-shaped raises ``KeyError`` / ``ValueError`` naming it.
    """
    filled = []
    for name, mod in model.named_modules():
        pre = f"{name}." if name else ""
        if isinstance(mod, VllmPackedInt4Linear):
            for key in ("weight_packed", "weight_scale"):
                if pre + key not in state_dict:
                    raise KeyError(f"{pre}{key} is missing from the checkpoint")
            shape = state_dict.get(pre + "weight_shape")
            if shape is not None and [int(v) for v in shape] != [mod.out_features, mod.in_features]:
                raise ValueError(f"{name}: checkpoint weight_shape {list(map(int, shape))} != "
                                 f"[{mod.out_features}, {mod.in_features}]")
            for key in ("weight_packed", "weight_scale", "weight_zero_point", "bias"):
                src = state_dict.get(pre + key)
                dst = getattr(mod, key, None)
                if src is None:
                    if key == "weight_zero_point" and dst is not None:
                        raise KeyError(f"{pre}{key} is missing: the module was built for an asymmetric export")
                    continue
                if dst is None:
                    raise ValueError(f"{name}: the checkpoint has {key} but the module was built without it")
                if tuple(dst.shape) != tuple(src.shape):
                    raise ValueError(f"{name}.{key}: checkpoint shape {tuple(src.shape)} != {tuple(dst.shape)}")
                dst.copy_(src.to(dst.dtype))
            mod._scale_zero = None
            mod.process_weights_after_loading()
            filled.append(name)
        elif isinstance(mod, SmoothQuantLinear):
            for key in ("weight", "weight_scale"):
                if pre + key not in state_dict:
                    raise KeyError(f"{pre}{key} is missing from the checkpoint")
            off = state_dict.get(pre + "weight_offset")
            if off is not None and bool(torch.any(off != 0)):
                raise ValueError(f"{name}: non-zero weight_offset; the W8A8 kernels are symmetric")
            w = state_dict[pre + "weight"]
            if w.dtype != torch.int8 or tuple(w.shape) != tuple(mod.weight.shape):
                raise ValueError(f"{name}.weight: expected int8 {tuple(mod.weight.shape)}, got {w.dtype} {tuple(w.shape)}")
            mod.weight.copy_(w)
            mod.weight_scale.copy_(state_dict[pre + "weight_scale"].reshape(mod.weight_scale.shape).to(mod.weight_scale.dtype))
            b = state_dict.get(pre + "bias")
            if b is not None and getattr(mod, "bias", None) is not None:
                mod.bias.copy_(b.to(mod.bias.dtype))
            mod.process_weights_after_loading()
            filled.append(name)
    return filled
