"""Seeded synthetic tensors for the quantized-linear workloads.

Real checkpoints and calibration sets are not available offline, so every
workload is built from random tensors with the layer shapes of the named
model families (Llama-2-7B / 70B, Llama-3-8B, Mixtral-8x7B).  Each tensor
draws from its own ``torch.Generator`` seeded ``seed + index`` on the CPU,
so the same call gives the same bits on any machine (device RNGs differ).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

# Layer shapes (out_features, in_features) of one decoder layer's linears.
LLAMA2_7B_LINEARS = {
    "q_proj": (4096, 4096),
    "k_proj": (4096, 4096),
    "v_proj": (4096, 4096),
    "o_proj": (4096, 4096),
    "gate_proj": (11008, 4096),
    "up_proj": (11008, 4096),
    "down_proj": (4096, 11008),
}
LLAMA3_8B_LINEARS = {
    "q_proj": (4096, 4096),
    "kv_proj": (1024, 4096),
    "gate_up_proj": (14336, 4096),
    "down_proj": (4096, 14336),
}
LLAMA2_70B_LINEARS = {
    "attn_proj": (8192, 8192),
    "kv_proj": (1024, 8192),
    "gate_up_proj": (28672, 8192),
    "down_proj": (8192, 28672),
}


@dataclass(frozen=True)
class MoeShape:
    num_experts: int = 8
    hidden: int = 4096
    ffn: int = 14336
    top_k: int = 2
    tokens: int = 8192


MIXTRAL_8X7B = MoeShape()


def _gen(seed: int, index: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed) * 1000003 + int(index))
    return g


def normal_weight(out_features: int, in_features: int, *, seed: int = 0, index: int = 0,
                  std: float = 0.02, dtype=torch.float16) -> torch.Tensor:
    """``N(0, std)`` weight ``[out, in]`` rounded to ``dtype``."""
    w = torch.randn((out_features, in_features), generator=_gen(seed, index), dtype=torch.float32)
    return (w * std).to(dtype)


def normal_activation(rows: int, features: int, *, seed: int = 0, index: int = 100,
                      dtype=torch.float16) -> torch.Tensor:
    """``N(0, 1)`` activations ``[rows, features]``."""
    x = torch.randn((rows, features), generator=_gen(seed, index), dtype=torch.float32)
    return x.to(dtype)


def outlier_activation(rows: int, features: int, *, seed: int = 0, index: int = 100,
                       outlier_fraction: float = 0.01, outlier_gain: float = 20.0,
                       dtype=torch.float16) -> torch.Tensor:
    """``N(0, 1)`` activations where a seeded random 1 % of channels is scaled x20.

    This mimics the channel outliers that SmoothQuant-style W8A8 has to cope
    with; the channel set is drawn from generator ``index + 1``.
    """
    x = torch.randn((rows, features), generator=_gen(seed, index), dtype=torch.float32)
    n_out = max(1, int(round(features * outlier_fraction)))
    perm = torch.randperm(features, generator=_gen(seed, index + 1))
    x[:, perm[:n_out]] *= outlier_gain
    return x.to(dtype)


def router_logits(tokens: int, num_experts: int, *, seed: int = 0, index: int = 200) -> torch.Tensor:
    """fp32 ``N(0, 1)`` router logits ``[tokens, experts]``."""
    return torch.randn((tokens, num_experts), generator=_gen(seed, index), dtype=torch.float32)


def moe_weights(shape: MoeShape, *, seed: int = 0, index: int = 300, std: float = 0.02,
                dtype=torch.float16, experts: range | None = None):
    """Packed expert weights ``gate_up[E, 2I, H]`` and ``down[E, H, I]``.

    ``experts`` restricts generation to a sub-range (each expert has its own
    generator, so a shard sees exactly the slices of the full tensor).
    """
    experts = range(shape.num_experts) if experts is None else experts
    gu, dn = [], []
    for e in experts:
        gu.append(normal_weight(2 * shape.ffn, shape.hidden, seed=seed, index=index + 2 * e, std=std, dtype=dtype))
        dn.append(normal_weight(shape.hidden, shape.ffn, seed=seed, index=index + 2 * e + 1, std=std, dtype=dtype))
    return torch.stack(gu), torch.stack(dn)
