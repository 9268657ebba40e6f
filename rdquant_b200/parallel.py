"""Column-parallel split of a mixed-precision linear over the GPUs of one node.

The reference has no multi-GPU path; this is the sharding the operator's layout suggests.
Output channels are independent, so each format group (NVFP4 | FP8 | FP16, rows in permuted
order) is cut at 128-channel boundaries into ``world`` contiguous row ranges -- a pure row
slice of the packed checkpoint tensors, the on-disk layout is unchanged.  Every rank runs
the fused kernels on its rows (x replicated, no collective on that path).  Where the full
output vector is needed on every rank (whole-model decode) one NCCL ``all_gather`` per layer
collects the ``[M, n_max]`` slices; the kernel writes its slice in local permuted order and a
precomposed index restores original channel order after the gather.

Ranks whose share is narrower than the widest one get zero-weight rows appended at pack time
(NVFP4 codes 0 with block scale 0: 0.56 bytes per element), so every rank's kernel writes a
full ``[M, n_max]`` slice straight into the send buffer: no pad copy, no allocation, and the
whole forward -- kernel, all-gather, one ``take`` -- can sit inside a CUDA graph.
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
    n_max: int              # widest rank (every rank's slice is padded to this)
    pad_format: str         # format group that receives a rank's zero rows
    gather_index: torch.Tensor  # int64 [N]: position of original channel j in the [world, n_max] gather buffer

    @classmethod
    def build(cls, splits: dict, inv_perm: torch.Tensor, world: int, align: int = 128) -> "ColumnParallelPlan":
        sizes = {f: int(splits.get(f, 0)) for f in FORMAT_ORDER}
        ranges = {f: split_points(sizes[f], world, align) for f in FORMAT_ORDER}
        n_local = [sum(ranges[f][r + 1] - ranges[f][r] for f in FORMAT_ORDER) for r in range(world)]
        n_max = max(n_local) if n_local else 0
        n = sum(sizes.values())
        pad_format = next((f for f in FORMAT_ORDER if sizes[f] > 0), "NVFP4")
        # position of every permuted row p in the gathered [world, n_max] buffer; a rank's zero
        # rows sit at the end of its pad_format group
        pos_of_perm_row = torch.empty(n, dtype=torch.int64)
        for r in range(world):
            local = 0
            for f in FORMAT_ORDER:
                start = sum(sizes[g] for g in FORMAT_ORDER[: FORMAT_ORDER.index(f)])
                lo, hi = ranges[f][r], ranges[f][r + 1]
                if hi > lo:
                    pos_of_perm_row[start + lo:start + hi] = r * n_max + local + torch.arange(hi - lo)
                local += hi - lo
                if f == pad_format:
                    local += n_max - n_local[r]
        inv = inv_perm.to(torch.int64).cpu()
        return cls(world, sizes, ranges, n_local, n_max, pad_format, pos_of_perm_row[inv])

    def local_splits(self, rank: int, padded: bool = True) -> dict:
        out = {f: self.ranges[f][rank + 1] - self.ranges[f][rank] for f in FORMAT_ORDER}
        if padded:
            out[self.pad_format] += self.n_max - self.n_local[rank]
        return out

    def shard_layer_data(self, layer_data: dict, rank: int, padded: bool = True) -> dict:
        """Row slices of the packed tensors owned by ``rank`` (identity local permutation), with
        the rank's zero rows appended to the ``pad_format`` group when ``padded``."""
        out = {}
        pad = self.n_max - self.n_local[rank] if padded else 0
        for f in FORMAT_ORDER:
            lo, hi = self.ranges[f][rank], self.ranges[f][rank + 1]
            extra = pad if f == self.pad_format else 0
            if hi == lo and extra == 0:
                continue
            for key in _KEYS[f]:
                part = layer_data[key][lo:hi]
                if extra:
                    fill = 1.0 if key == "weight_fp8_scale" else 0
                    zeros = torch.full((extra,) + tuple(part.shape[1:]), fill, dtype=part.dtype, device=part.device)
                    part = torch.cat([part, zeros], dim=0)
                out[key] = part.contiguous()
            if f == "NVFP4" and "nvfp4_global_scale" in layer_data:
                out["nvfp4_global_scale"] = layer_data["nvfp4_global_scale"]
        out["inv_permutation"] = torch.arange(self.n_local[rank] + pad, dtype=torch.int32)
        return out

    def local_bias(self, bias: torch.Tensor, rank: int) -> torch.Tensor:
        """``bias`` (original channel order) rearranged to ``rank``'s padded slice order."""
        flat = torch.zeros(self.world * self.n_max, dtype=bias.dtype)
        flat[self.gather_index] = bias.detach().cpu()
        return flat[rank * self.n_max:(rank + 1) * self.n_max].contiguous()

    def take_index(self, m: int) -> torch.Tensor:
        """int64 ``[m, N]``: flat positions inside a ``[world, m, n_max]`` gather buffer of
        ``y[row, original channel]``."""
        r = self.gather_index // self.n_max
        c = self.gather_index - r * self.n_max
        rows = torch.arange(m, dtype=torch.int64).unsqueeze(1)
        return (r.unsqueeze(0) * m + rows) * self.n_max + c.unsqueeze(0)

    def packed_bytes(self, rank: int, k: int) -> int:
        s = self.local_splits(rank, padded=False)
        return s["NVFP4"] * (k // 2 + k // 16) + s["FP8"] * (k + 4) + s["FP16"] * 2 * k


def gather_outputs(y_local: torch.Tensor, plan: ColumnParallelPlan, group=None,
                   buffer: Optional[torch.Tensor] = None, index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather the per-rank slices and return ``[M, N]`` in original channel order.

    ``y_local`` is ``[M, n_max]`` (padded slice) or ``[M, n_local]`` (then it is padded here,
    which costs a copy); ``buffer`` ``[world, M, n_max]`` and ``index`` (``plan.take_index(M)`` on
    the device) may be passed in to make the call allocation-free."""
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
    if index is None:
        index = plan.take_index(m).to(buffer.device)
    return torch.take(buffer, index)


class ColumnParallelMixedLinear(nn.Module):
    """One rank's share of a mixed-precision linear plus the all-gather of the outputs.

    Buffers (send slice, gather buffer, un-permute index) are allocated once per activation row
    count, so a forward pass is: one fused kernel launch, one ``all_gather_into_tensor``, one
    ``take`` -- all capturable in a CUDA graph.  The bias is added by the kernel's epilogue."""

    def __init__(self, layer_data: dict, splits: dict, k: int, device, rank: int, world: int, group=None,
                 gather: bool = True) -> None:
        super().__init__()
        from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv

        self.plan = ColumnParallelPlan.build(splits, layer_data["inv_permutation"], world)
        self.rank, self.world, self.group, self.gather = rank, world, group, gather
        self.K = int(k)
        self.N = sum(self.plan.splits.values())
        self.device = torch.device(device)
        shard = self.plan.shard_layer_data(layer_data, rank)
        self.local_splits = self.plan.local_splits(rank)
        self.fd = pack_for_fused_gemv(shard, self.local_splits, k, device)
        if self.fd is None:
            raise RuntimeError("rdquant_b200 kernels unavailable: build librdq_b200.so and run on a CUDA device")
        bias = layer_data.get("bias")
        self.bias_local = None
        if bias is not None:
            self.bias_local = self.plan.local_bias(bias, rank).to(device=self.device, dtype=torch.float16)
        self.use_pdl = False
        self._state: dict = {}

    def _io_buffers(self, m: int):
        st = self._state.get(m)
        if st is None:
            send = torch.zeros(m, self.plan.n_max, dtype=torch.float16, device=self.device)
            buf = torch.zeros(self.world, m, self.plan.n_max, dtype=torch.float16, device=self.device)
            idx = self.plan.take_index(m).to(self.device)
            st = (send, buf, idx)
            self._state[m] = st
        return st

    def packed_bytes(self) -> int:
        return self.plan.packed_bytes(self.rank, self.K)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from rdquant_b200 import _lib, rdquant_cuda

        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.K)
        xh = (x2 if x2.dtype == torch.float16 else x2.half()).contiguous()
        m = xh.shape[0]
        send, buf, idx = self._io_buffers(m)
        flags = _lib.RDQ_GEMV_PDL if self.use_pdl else 0
        rdquant_cuda.mixed_linear(xh, self.fd, self.bias_local, flags, out=send)
        if not self.gather:
            return send
        y = gather_outputs(send, self.plan, self.group, buffer=buf, index=idx)
        return y.to(x.dtype).reshape(*lead, self.N)


# ---------------------------------------------------------------------------------------------
# All-gather fused into the GEMV epilogue: every rank stores its output slice straight into the
# gather buffer of every GPU of the node (plain stores to peer memory over NVLink), then raises a
# flag there; the receiving side is one small kernel that waits for the flags (bounded) and
# un-permutes.  No NCCL call on the decode path: 4 small collectives per block cost more than the
# GEMVs they follow.
# ---------------------------------------------------------------------------------------------

class PeerArena:
    """One symmetric-memory allocation shared by the layers of a model: every rank allocates the
    same bytes, the ranks exchange handles once, and layers take equal sub-ranges of it."""

    def __init__(self, nbytes: int, device, group=None) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.local.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.rank, self.world = int(self.handle.rank), int(self.handle.world_size)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._used = 0
        dist.barrier(group=self.group)  # every rank's arena is zeroed before anyone writes into one

    def alloc(self, nbytes: int) -> int:
        """Byte offset of a fresh, 256-byte aligned range of the arena (the same on every rank)."""
        off = self._used
        self._used = off + (int(nbytes) + 255) // 256 * 256
        if self._used > self.nbytes:
            raise RuntimeError(f"peer arena of {self.nbytes} bytes is full")
        return off

    def view(self, off: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        return self.local[off:off + nbytes].view(dtype)


class PeerGatherMixedLinear(nn.Module):
    """Column-parallel mixed-precision linear whose decode path (M <= 16) needs no collective call:
    ``rdq_gemv_tiled_peer`` writes this rank's slice into every GPU's gather buffer and
    ``rdq_peer_gather`` waits for all slices and restores original channel order.  Larger M
    (prefill) goes through the tcgen05 GEMM and an NCCL all-gather like
    :class:`ColumnParallelMixedLinear`."""

    MAX_M = 16

    def __init__(self, layer_data: dict, splits: dict, k: int, arena: PeerArena, wait_ms: int = 500) -> None:
        super().__init__()
        from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv

        self.arena = arena
        rank, world = arena.rank, arena.world
        self.rank, self.world, self.group = rank, world, arena.group
        self.device = arena.device
        self.plan = ColumnParallelPlan.build(splits, layer_data["inv_permutation"], world)
        self.K, self.N = int(k), sum(self.plan.splits.values())
        shard = self.plan.shard_layer_data(layer_data, rank)
        self.fd = pack_for_fused_gemv(shard, self.plan.local_splits(rank), k, self.device)
        if self.fd is None or self.fd.get("w_tiled") is None:
            raise RuntimeError("PeerGatherMixedLinear needs the built kernels and a shape with a tiled layout")
        bias = layer_data.get("bias")
        self.bias_local = None
        if bias is not None:
            self.bias_local = self.plan.local_bias(bias, rank).to(device=self.device, dtype=torch.float16)
        n_max = self.plan.n_max
        self._buf_off = arena.alloc(world * self.MAX_M * n_max * 2)
        self._flag_off = arena.alloc(4 * 32)
        self._buf_local = arena.view(self._buf_off, world * self.MAX_M * n_max * 2, torch.float16)
        self._flags_local = arena.view(self._flag_off, 4 * 32, torch.int32)
        # local state words: [0] warps done, [1] launches sent, [2] unused, [3] status
        self._state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.wait_ms = int(wait_ms)
        self.use_pdl = False
        self._per_m: dict = {}
        self._nccl_state: dict = {}

    def packed_bytes(self) -> int:
        return self.plan.packed_bytes(self.rank, self.K)

    def _tables(self, m: int):
        st = self._per_m.get(m)
        if st is None:
            import ctypes

            n_max = self.plan.n_max
            # this rank's slice inside GPU d's gather buffer [world, m, n_max]; its flag word there
            dst = [p + self._buf_off + self.rank * m * n_max * 2 for p in self.arena.peer_ptrs]
            flg = [p + self._flag_off + 4 * self.rank for p in self.arena.peer_ptrs]
            dst_arr = (ctypes.c_void_p * self.world)(*dst)
            flg_arr = (ctypes.c_void_p * self.world)(*flg)
            idx = self.plan.take_index(m).reshape(-1).to(self.device)
            st = (dst_arr, flg_arr, idx)
            self._per_m[m] = st
        return st

    def prepare(self, m: int) -> None:
        """Build the per-M tables now (they involve a host-to-device copy, which a CUDA-graph
        capture does not allow)."""
        if m <= self.MAX_M:
            self._tables(m)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import ctypes

        from rdquant_b200 import _lib, rdquant_cuda

        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.K)
        xh = (x2 if x2.dtype == torch.float16 else x2.half()).contiguous()
        m = xh.shape[0]
        if m > self.MAX_M:
            send, buf, idx = self._nccl_buffers(m)
            rdquant_cuda.mixed_linear(xh, self.fd, self.bias_local, 0, out=send)
            y = gather_outputs(send, self.plan, self.group, buffer=buf, index=idx)
            return y.to(x.dtype).reshape(*lead, self.N)
        dst_arr, flg_arr, idx = self._tables(m)
        fd = self.fd
        y = torch.empty(m, self.N, dtype=torch.float16, device=self.device)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())  # noqa: E731
        lib = _lib.lib()
        rc = lib.rdq_gemv_tiled_peer(p(xh), m, p(fd["w_tiled"]), p(fd.get("w_fp8_scales")),
                                     float(fd.get("w_fp4_global_scale", 1.0)), p(fd.get("perm")), p(self.bias_local),
                                     ctypes.cast(dst_arr, ctypes.c_void_p), ctypes.cast(flg_arr, ctypes.c_void_p), self.world,
                                     ctypes.c_void_p(self._state.data_ptr()), fd["n_fp4"], fd["n_fp8"], fd["n_fp16"],
                                     self.K, p(fd["workspace"]), p(fd["tile_counters"]),
                                     _lib.RDQ_GEMV_PDL if self.use_pdl else 0, stream)
        _lib.check(rc, "rdq_gemv_tiled_peer")
        rc = lib.rdq_peer_gather(p(self._buf_local), p(idx), p(y), m * self.N, p(self._flags_local), self.world,
                                 ctypes.c_void_p(self._state.data_ptr()), ctypes.c_void_p(self._state.data_ptr() + 12),
                                 self.wait_ms, _lib.RDQ_GEMV_PDL if self.use_pdl else 0, stream)
        _lib.check(rc, "rdq_peer_gather")
        return y.to(x.dtype).reshape(*lead, self.N)

    def _nccl_buffers(self, m: int):
        st = self._nccl_state.get(m)
        if st is None:
            send = torch.zeros(m, self.plan.n_max, dtype=torch.float16, device=self.device)
            buf = torch.zeros(self.world, m, self.plan.n_max, dtype=torch.float16, device=self.device)
            st = (send, buf, self.plan.take_index(m).to(self.device))
            self._nccl_state[m] = st
        return st

    def reset_peer_state(self) -> None:
        """Collective: after a step in which a rank did not deliver, bring the launch counters and
        flag words of all ranks back to zero (all queued work is waited for first)."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._flags_local.zero_()
        self._state.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def check_status(self) -> None:
        """Wait for the queued work and raise if a rank's slice never arrived (status 10 + rank) or
        the GEMV gave up a wait; the local status word is cleared."""
        from rdquant_b200 import rdquant_cuda

        code = int(self._state[3].item())
        if code:
            self._state[3] = 0
            raise RuntimeError(f"peer gather: rank {code - 10} did not deliver its slice within {self.wait_ms} ms "
                               "(bounded device-side wait ran out); the output of that step is invalid")
        rdquant_cuda.check_status(self.fd)
