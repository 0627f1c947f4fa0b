"""Column-parallel (output-split) quantized linear over the GPUs of one node.

The path shards naturally over output rows: every row of the packed tensor carries its
own indices, scale and bias, and the codebook (64 KB) is replicated.  Rank ``r`` of ``g``
owns rows ``[r*N/g, (r+1)*N/g)`` -- a contiguous byte range of the packed stream whenever
a row's bits end on a byte boundary -- computes ``y[:, rows]`` with the single-GPU kernels
and the ranks exchange their column blocks with ONE all-gather over NVLink (NCCL through
``torch.distributed``).  Activations and their per-token scales are replicated, so each
output element is produced by exactly one GPU with the single-GPU summation order: the
gathered result is bit-identical to the one-GPU result.

The reference has no multi-GPU inference path (its only collective is the calibration
trainer's gradient all-reduce); this module is new work on top of the same payload format.

Nothing here waits on the device: the gather of chunk ``i`` runs on a side stream while
the GEMM of chunk ``i+1`` runs on the compute stream.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .packing import pack_indices, unpack_indices


def shard_rows(out_features: int, rank: int, world: int) -> tuple[int, int]:
    """Row range ``[begin, end)`` of ``rank``; requires ``out_features % world == 0``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if out_features % world != 0:
        raise ValueError(f"out_features={out_features} is not divisible by {world} ranks")
    per = out_features // world
    return rank * per, (rank + 1) * per


def shard_payload(payload: dict, rank: int, world: int) -> dict:
    """The ``packed_vector_codebook_v1`` payload of one rank's output rows (CPU, load time).

    Accepts ``indices`` or ``packed_indices`` payloads and returns the same flavour.  The
    packed stream is sliced byte-wise when the shard starts and ends on byte boundaries and
    re-packed from unpacked indices otherwise."""
    n = int(payload["out_features"])
    begin, end = shard_rows(n, rank, world)
    out = {k: v for k, v in payload.items() if k not in ("indices", "packed_indices", "index_shape", "scales",
                                                         "out_features")}
    out["out_features"] = end - begin
    out["scales"] = torch.as_tensor(payload["scales"])[begin:end].contiguous()
    if "packed_indices" in payload:
        bits = int(payload["index_bits"])
        shape = tuple(int(x) for x in payload["index_shape"])
        per_row = shape[1] * shape[2]
        packed = torch.as_tensor(payload["packed_indices"]).reshape(-1)
        lo_bit, hi_bit = begin * per_row * bits, end * per_row * bits
        if lo_bit % 8 == 0 and hi_bit % 8 == 0:
            shard = packed[lo_bit // 8: hi_bit // 8].clone()
        else:
            idx = unpack_indices(packed, bits, shape[0] * per_row).reshape(shape)[begin:end]
            shard = pack_indices(idx, bits)
        out["packed_indices"] = shard
        out["index_shape"] = (end - begin, shape[1], shape[2])
    else:
        out["indices"] = torch.as_tensor(payload["indices"])[begin:end].contiguous()
    return out


def gather_columns(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather ``[M, N/g]`` column blocks into ``[M, N]`` (rank order = column order)."""
    world = dist.get_world_size(group)
    m, n_local = y_local.shape
    stacked = torch.empty((world, m, n_local), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(stacked.view(world * m, n_local), y_local.contiguous(), group=group)
    full = stacked.permute(1, 0, 2).reshape(m, world * n_local)
    if out is not None:
        out.copy_(full)
        return out
    return full


class ColumnParallelCodebookLinear(torch.nn.Module):
    """One rank's slice of a quantized linear plus the all-gather of the result.

    ``forward(x)`` takes the replicated ``[..., K]`` activations and returns the full
    ``[..., N]`` output on every rank.  ``chunks > 1`` splits the token dimension so the
    gather of one chunk overlaps the GEMM of the next."""

    def __init__(self, payload: dict, bias: torch.Tensor | None, device: str, group=None, chunks: int = 1):
        super().__init__()
        from .linear import PrecomputedPackedVectorCodebookLinear
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.out_features = int(payload["out_features"])
        self.in_features = int(payload["in_features"])
        begin, end = shard_rows(self.out_features, self.rank, self.world)
        local_bias = None if bias is None else bias[begin:end]
        self.local = PrecomputedPackedVectorCodebookLinear(shard_payload(payload, self.rank, self.world), local_bias,
                                                           device)
        self.chunks = max(1, int(chunks))
        self._comm_stream = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a = x.reshape(-1, self.in_features)
        m = a.shape[0]
        if self.world == 1:
            return self.local(x)
        n_local = self.out_features // self.world
        if self.chunks == 1 or m < self.chunks:
            full = gather_columns(self.local(a), self.group)
            return full.reshape(*x.shape[:-1], self.out_features)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=a.device)
        compute = torch.cuda.current_stream()
        stacked = torch.empty((self.world, m, n_local), dtype=torch.bfloat16, device=a.device)
        bounds = [m * i // self.chunks for i in range(self.chunks + 1)]
        pieces = []
        for i in range(self.chunks):
            lo, hi = bounds[i], bounds[i + 1]
            y_local = self.local(a[lo:hi]).to(torch.bfloat16)
            ready = torch.cuda.Event()
            ready.record(compute)
            part = torch.empty((self.world, hi - lo, n_local), dtype=torch.bfloat16, device=a.device)
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                dist.all_gather_into_tensor(part.view(self.world * (hi - lo), n_local), y_local, group=self.group)
                stacked[:, lo:hi].copy_(part)
            y_local.record_stream(self._comm_stream)
            part.record_stream(self._comm_stream)
            pieces.append(part)
        compute.wait_stream(self._comm_stream)
        full = stacked.permute(1, 0, 2).reshape(m, self.out_features)
        full = full if x.dtype == torch.bfloat16 else full.to(x.dtype)
        return full.reshape(*x.shape[:-1], self.out_features)
