"""Column-parallel split of a mixed-precision linear over the GPUs of one node.

The reference has no multi-GPU path; this is the sharding the operator's layout suggests.
Output channels are independent, so each format group (NVFP4 | FP8 | FP16, rows in permuted
order) is cut at 128-channel boundaries into ``world`` contiguous row ranges -- a pure row
slice of the packed checkpoint tensors, the on-disk layout is unchanged.  Every rank runs
the fused kernels on its rows (x replicated, no collective on that path).  Where the full
output vector is needed on every rank (whole-model decode) one NCCL ``all_gather`` per layer
collects the ``[M, N_r]`` slices; the kernel writes its slice in local permuted order and a
precomposed index restores original channel order after the gather.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

FORMAT_ORDER = ("NVFP4", "FP8", "FP16")
_KEYS = {
    "NVFP4": ("weight_nvfp4", "weight_nvfp4_scale"),
    "FP8": ("weight_fp8", "weight_fp8_scale"),
    "FP16": ("weight_fp16",),
}


def split_points(n_rows: int, world: int, align: int = 128) -> list[int]:
    """``world + 1`` row offsets cutting ``n_rows`` into contiguous ranges on ``align``-row tiles
    (the last tile may be short); tile counts differ by at most one between ranks."""
    if n_rows == 0:
        return [0] * (world + 1)
    tiles = (n_rows + align - 1) // align
    return [min((r * tiles // world) * align, n_rows) for r in range(world)] + [n_rows]


@dataclass
class ColumnParallelPlan:
    """Row ranges of every rank and the index that undoes permutation + sharding."""

    world: int
    splits: dict            # full layer
    ranges: dict            # fmt -> list of world + 1 offsets inside the group
    n_local: list           # rows owned by each rank
    n_max: int              # widest rank (gather buffers are padded to this)
    gather_index: torch.Tensor  # int64 [N]: position of original channel j in the [world, n_max] gather buffer

    @classmethod
    def build(cls, splits: dict, inv_perm: torch.Tensor, world: int, align: int = 128) -> "ColumnParallelPlan":
        sizes = {f: int(splits.get(f, 0)) for f in FORMAT_ORDER}
        ranges = {f: split_points(sizes[f], world, align) for f in FORMAT_ORDER}
        n_local = [sum(ranges[f][r + 1] - ranges[f][r] for f in FORMAT_ORDER) for r in range(world)]
        n_max = max(n_local) if n_local else 0
        n = sum(sizes.values())
        # position of every permuted row p in the gathered [world, n_max] buffer
        pos_of_perm_row = torch.empty(n, dtype=torch.int64)
        for r in range(world):
            local = 0
            for f in FORMAT_ORDER:
                start = sum(sizes[g] for g in FORMAT_ORDER[: FORMAT_ORDER.index(f)])
                lo, hi = ranges[f][r], ranges[f][r + 1]
                if hi > lo:
                    pos_of_perm_row[start + lo:start + hi] = r * n_max + local + torch.arange(hi - lo)
                local += hi - lo
        inv = inv_perm.to(torch.int64).cpu()
        return cls(world, sizes, ranges, n_local, n_max, pos_of_perm_row[inv])

    def local_splits(self, rank: int) -> dict:
        return {f: self.ranges[f][rank + 1] - self.ranges[f][rank] for f in FORMAT_ORDER}

    def shard_layer_data(self, layer_data: dict, rank: int) -> dict:
        """Row slices of the packed tensors owned by ``rank`` (identity local permutation)."""
        out = {}
        for f in FORMAT_ORDER:
            lo, hi = self.ranges[f][rank], self.ranges[f][rank + 1]
            if hi == lo:
                continue
            for key in _KEYS[f]:
                out[key] = layer_data[key][lo:hi].contiguous()
            if f == "NVFP4" and "nvfp4_global_scale" in layer_data:
                out["nvfp4_global_scale"] = layer_data["nvfp4_global_scale"]
        out["inv_permutation"] = torch.arange(self.n_local[rank], dtype=torch.int32)
        return out

    def packed_bytes(self, rank: int, k: int) -> int:
        s = self.local_splits(rank)
        return s["NVFP4"] * (k // 2 + k // 16) + s["FP8"] * (k + 4) + s["FP16"] * 2 * k


def gather_outputs(y_local: torch.Tensor, plan: ColumnParallelPlan, group=None,
                   buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather the ``[M, n_local]`` slices and return ``[M, N]`` in original channel order."""
    import torch.distributed as dist

    m = y_local.shape[0]
    world = plan.world
    send = y_local
    if y_local.shape[1] != plan.n_max:
        send = y_local.new_zeros(m, plan.n_max)
        send[:, : y_local.shape[1]] = y_local
    if buffer is None:
        buffer = y_local.new_empty(world, m, plan.n_max)
    dist.all_gather_into_tensor(buffer.view(world * m, plan.n_max), send.contiguous(), group=group)
    flat = buffer.permute(1, 0, 2).reshape(m, world * plan.n_max)
    return flat.index_select(1, plan.gather_index.to(flat.device))


class ColumnParallelMixedLinear(nn.Module):
    """One rank's share of a mixed-precision linear plus the all-gather of the outputs."""

    def __init__(self, layer_data: dict, splits: dict, k: int, device, rank: int, world: int, group=None,
                 gather: bool = True) -> None:
        super().__init__()
        from rdquant_b200.inference import FusedMixedLinear

        self.plan = ColumnParallelPlan.build(splits, layer_data["inv_permutation"], world)
        self.rank, self.world, self.group, self.gather = rank, world, group, gather
        self.K = int(k)
        self.N = sum(self.plan.splits.values())
        shard = self.plan.shard_layer_data(layer_data, rank)
        self.local = FusedMixedLinear.from_layer_data(shard, self.plan.local_splits(rank), k, device)
        bias = layer_data.get("bias")
        self.bias = nn.Parameter(bias.to(device)) if bias is not None else None
        self.register_buffer("_gather_index", self.plan.gather_index.to(device), persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y_local = self.local(x.reshape(-1, self.K))
        if not self.gather:
            return y_local
        y = gather_outputs(y_local, self.plan, self.group)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, self.N)
