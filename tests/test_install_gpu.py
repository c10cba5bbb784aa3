"""Model-level installers on a tiny llama-shaped model: the installed real-quant twins against the oracle's
restatement of what the reference's installers leave in the model (AWQ pseudo_quantize_model_weight,
quantizer.py:109-130; SmoothQuant quantize_model, fake_quant.py:441-458)."""
import numpy as np
import pytest
import torch

from mindpipe_b200 import install
from mindpipe_b200.modules import SmoothQuantLinear, VllmPackedInt4Linear
from oracle import pseudo_quant as O
from tests._tiny_llama import PROJ_ORDER, TinyLlama

pytestmark = pytest.mark.gpu
TOL = 1e-2   # relative Frobenius error of fp16 outputs


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def _linears(model):
    return {f"model.layers.{i}.{n}": m for i, layer in enumerate(model.model.layers)
            for n, m in install.get_named_linears(layer).items()}


def test_real_quantize_model_weight_matches_awq_pseudo_quant_bit_for_bit():
    ref = TinyLlama(seed=1)
    originals = {k: v.weight.detach().numpy().copy() for k, v in _linears(ref).items()}
    model = TinyLlama(seed=1).cuda()
    names = install.real_quantize_model_weight(model, 4, {"zero_point": True, "q_group_size": 128})
    assert names == [f"model.layers.{i}.{p}" for i in range(2) for p in PROJ_ORDER]
    assert isinstance(model.lm_head, torch.nn.Linear)                     # outside the blocks: untouched
    x = torch.randn((5, 256), generator=torch.Generator().manual_seed(0)).half()
    for name in names:
        mod = model.get_submodule(name)
        assert isinstance(mod, VllmPackedInt4Linear)
        wdq, _, _, _ = O.w4_group_asym_quantize(originals[name], 128)
        assert np.array_equal(bits(mod.dequantize().cpu().numpy()), bits(wdq)), name
        if mod.in_features == 256:
            b = None if mod.bias is None else mod.bias.cpu().numpy()
            y = mod(x.cuda()).cpu().numpy()
            assert O.rel_frobenius(y, O.linear_f16(x.numpy(), wdq, b)) <= TOL, name


def test_quantize_model_installs_smoothquant_twins_in_reference_order():
    ref = TinyLlama(seed=2)
    originals = {k: (v.weight.detach().numpy().copy(), None if v.bias is None else v.bias.detach().numpy().copy())
                 for k, v in _linears(ref).items()}
    model = TinyLlama(seed=2).cuda()
    names = install.quantize_model(model)
    assert names == [f"model.layers.{i}.{p}" for i in range(2) for p in PROJ_ORDER]
    x = (torch.randn((7, 256), generator=torch.Generator().manual_seed(3)) * 2).half()
    for name in names:
        mod = model.get_submodule(name)
        assert isinstance(mod, SmoothQuantLinear)
        assert mod.quantize_output == name.endswith(("q_proj", "k_proj", "v_proj"))   # fake_quant.py quantize_bmm_input
        w, b = originals[name]
        w_fake, codes, _ = O.absmax_quant_last_dim(w)
        assert np.array_equal(mod.weight.cpu().numpy(), codes.astype(np.int8)), name
        if mod.in_features == 256:
            y = mod(x.cuda()).cpu().numpy()
            ref_y = O.smoothquant_linear_forward(x.numpy(), w_fake, b, quantize_output=mod.quantize_output)
            assert O.rel_frobenius(y, ref_y) <= TOL, name


def test_exported_checkpoint_round_trip_is_identical():
    src = TinyLlama(seed=4).cuda()
    install.real_quantize_model_weight(src, 4, {"zero_point": True, "q_group_size": 64})
    sd = {k: v.detach().cpu() for k, v in src.state_dict().items()}
    assert "model.layers.0.mlp.down_proj.weight_packed" in sd and "model.layers.1.self_attn.v_proj.bias" in sd
    dst = TinyLlama(seed=5).cuda()                                         # different weights, same layout
    install.real_quantize_model_weight(dst, 4, {"zero_point": True, "q_group_size": 64})
    filled = install.load_exported_state_dict(dst, sd)
    assert len(filled) == 14
    x = torch.randn((3, 256), generator=torch.Generator().manual_seed(6)).half().cuda()
    for name in filled:
        a, b = src.get_submodule(name), dst.get_submodule(name)
        assert torch.equal(a.weight_packed, b.weight_packed) and torch.equal(a.weight_zero_point, b.weight_zero_point)
        if a.in_features == 256:
            assert torch.equal(a(x), b(x)), name

    s8 = TinyLlama(seed=7).cuda()
    install.quantize_model(s8)
    sd8 = {k: v.detach().cpu() for k, v in s8.state_dict().items()}
    d8 = TinyLlama(seed=8).cuda()
    install.quantize_model(d8)
    assert len(install.load_exported_state_dict(d8, sd8)) == 14
    for name in ("model.layers.0.self_attn.q_proj", "model.layers.1.mlp.gate_proj"):
        assert torch.equal(s8.get_submodule(name)(x), d8.get_submodule(name)(x))
    sd8["model.layers.0.mlp.up_proj.weight_offset"] = torch.ones_like(sd8["model.layers.0.mlp.up_proj.weight_offset"])
    with pytest.raises(ValueError, match="weight_offset"):
        install.load_exported_state_dict(d8, sd8)
