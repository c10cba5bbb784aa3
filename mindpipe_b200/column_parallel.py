"""Column-parallel W4A16 linear for the 70B-shaped layers: split the output rows of the
packed weight over the ranks, replicate the activations, all-gather the outputs.

Rank ``r`` of ``P`` holds rows ``[r*N/P, (r+1)*N/P)`` of ``weight_packed``, ``weight_scale`` and
``weight_zero_point``; each rank computes ``y[:, slice]`` with the single-GPU kernels and one
``all_gather_into_tensor`` assembles ``y[M, N]`` on every rank (tensor parallelism of the
column-parallel kind, as the third-party runtime does around ``AscendLinearMethod``;
acceleration/runtime_patches/vllm_ascend.patch:3260-3305 shows its all-gather call sites).
Per GPU the weight stream shrinks by ``P``; the collective moves ``2*M*N`` bytes in total.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(n_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Row range of ``rank``; ``n_rows`` must divide evenly (it does for the 70B shapes and P <= 8)."""
    if n_rows % world_size != 0:
        raise ValueError(f"{n_rows} output rows do not divide over {world_size} ranks")
    per = n_rows // world_size
    return rank * per, (rank + 1) * per


def shard_packed_linear(packed, scale, zero_point, bias, world_size: int, rank: int):
    """Slices of the four weight-side tensors for ``rank`` (views; call ``.contiguous()`` after ``.to(device)``)."""
    lo, hi = shard_rows(packed.shape[0], world_size, rank)
    return (packed[lo:hi], scale[lo:hi], None if zero_point is None else zero_point[lo:hi],
            None if bias is None else bias[lo:hi])


def assemble_gathered(gathered: torch.Tensor) -> torch.Tensor:
    """``[P, M, N/P]`` (what all-gather returns, rank-major) -> ``[M, N]``."""
    p, m, n_loc = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, p * n_loc)


class ColumnParallelW4A16Linear(torch.nn.Module):
    """``VllmPackedInt4Linear`` sharded by output rows over a process group."""

    def __init__(self, local_linear, out_features: int, group=None, gather_output: bool = True):
        super().__init__()
        self.local = local_linear
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.out_features = int(out_features)
        self.gather_output = gather_output
        lo, hi = shard_rows(self.out_features, self.world, self.rank)
        if local_linear.out_features != hi - lo:
            raise ValueError(f"rank {self.rank} must hold {hi - lo} rows, got {local_linear.out_features}")

    @staticmethod
    def from_full(packed, scale, zero_point, bias, in_features: int, group=None, device=None):
        from .modules import VllmPackedInt4Linear
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        p, s, z, b = shard_packed_linear(packed, scale, zero_point, bias, world, rank)
        to = (lambda t: None if t is None else t.to(device).contiguous())
        local = VllmPackedInt4Linear(packed_weight=to(p), scale=to(s), bias=to(b), in_features=in_features,
                                     out_features=p.shape[0], zero_point=to(z))
        return ColumnParallelW4A16Linear(local, packed.shape[0], group)

    @torch.no_grad()
    def forward(self, x):
        y_loc = self.local(x)
        if not self.gather_output or self.world == 1:
            return y_loc
        lead = y_loc.shape[:-1]
        y2 = y_loc.reshape(-1, y_loc.shape[-1]).contiguous()
        m, n_loc = y2.shape
        gathered = torch.empty((self.world * m, n_loc), dtype=y2.dtype, device=y2.device)   # rank-major rows
        dist.all_gather_into_tensor(gathered, y2, group=self.group)
        return assemble_gathered(gathered.view(self.world, m, n_loc)).reshape(*lead, self.out_features)
