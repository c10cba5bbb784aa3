"""A two-layer llama-shaped module tree (attention and MLP projections only) for the installer tests."""
import torch
from torch import nn


class _Attn(nn.Module):
    def __init__(self, h, kv):
        super().__init__()
        self.q_proj = nn.Linear(h, h, bias=False)
        self.k_proj = nn.Linear(h, kv, bias=False)
        self.v_proj = nn.Linear(h, kv, bias=True)
        self.o_proj = nn.Linear(h, h, bias=False)


class _Mlp(nn.Module):
    def __init__(self, h, f):
        super().__init__()
        self.gate_proj = nn.Linear(h, f, bias=False)
        self.up_proj = nn.Linear(h, f, bias=False)
        self.down_proj = nn.Linear(f, h, bias=False)


class _Layer(nn.Module):
    def __init__(self, h, kv, f):
        super().__init__()
        self.self_attn = _Attn(h, kv)
        self.mlp = _Mlp(h, f)


class _Backbone(nn.Module):
    def __init__(self, n, h, kv, f):
        super().__init__()
        self.layers = nn.ModuleList([_Layer(h, kv, f) for _ in range(n)])


class TinyLlama(nn.Module):
    def __init__(self, n_layers=2, hidden=256, kv=128, ffn=512, seed=0):
        super().__init__()
        self.model = _Backbone(n_layers, hidden, kv, ffn)
        self.lm_head = nn.Linear(hidden, 64, bias=False)
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
        self.half()


PROJ_ORDER = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
              "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]
