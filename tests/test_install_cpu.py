"""Host logic of the model-level installers (argument checks and error behaviour; no kernel runs)."""
import pytest
import torch
from torch import nn

from mindpipe_b200 import install
from mindpipe_b200.modules import VllmPackedInt4Linear
from tests._tiny_llama import TinyLlama


def test_quantize_model_rejects_other_weight_quant_like_the_reference():
    with pytest.raises(ValueError, match="Invalid weight_quant"):          # fake_quant.py:449-450
        install.quantize_model(TinyLlama(), weight_quant="per_tensor")


def test_installers_refuse_cpu_models():
    with pytest.raises(ValueError, match="CUDA"):
        install.quantize_model(TinyLlama())
    with pytest.raises(ValueError, match="CUDA"):
        install.real_quantize_model_weight(TinyLlama(), 4, {"zero_point": True, "q_group_size": 128})


def test_real_quantize_argument_checks():
    m = TinyLlama()
    with pytest.raises(ValueError, match="w_bit=4"):
        install.real_quantize_model_weight(m, 8, {"zero_point": True, "q_group_size": 128})
    with pytest.raises(ValueError, match="group size"):
        install.real_quantize_model_weight(m, 4, {"zero_point": True, "q_group_size": -1})


def test_get_blocks_layouts():
    m = TinyLlama()
    assert install.get_blocks(m) is m.model.layers
    assert install._blocks_prefix(m) == "model.layers"
    with pytest.raises(NotImplementedError):
        install.get_blocks(nn.Linear(4, 4))
    names = install.get_named_linears(m.model.layers[0])
    assert sorted(names) == sorted(["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                                    "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"])


def test_load_exported_state_dict_errors_name_the_module():
    holder = nn.Module()
    holder.proj = VllmPackedInt4Linear(packed_weight=torch.zeros((8, 16), dtype=torch.int32),
                                       scale=torch.ones((8, 1), dtype=torch.float16), bias=None,
                                       in_features=128, out_features=8,
                                       zero_point=torch.zeros((8, 1), dtype=torch.int32))
    with pytest.raises(KeyError, match="proj.weight_packed"):
        install.load_exported_state_dict(holder, {})
    sd = {"proj.weight_packed": torch.zeros((8, 16), dtype=torch.int32),
          "proj.weight_scale": torch.ones((8, 1), dtype=torch.float16),
          "proj.weight_shape": torch.tensor([16, 128])}
    with pytest.raises(ValueError, match="weight_shape"):
        install.load_exported_state_dict(holder, sd)
    sd["proj.weight_shape"] = torch.tensor([8, 128])
    with pytest.raises(KeyError, match="weight_zero_point"):              # asymmetric module, symmetric checkpoint
        install.load_exported_state_dict(holder, sd)
    sd["proj.weight_zero_point"] = torch.zeros((8, 2), dtype=torch.int32)
    with pytest.raises(ValueError, match="checkpoint shape"):
        install.load_exported_state_dict(holder, sd)
