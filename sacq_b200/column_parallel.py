"""Column-parallel (output-split) quantized linear over the GPUs of one node.

The path shards naturally over output rows: every row of the packed tensor carries its
own indices, scale and bias, and the codebook (64 KB) is replicated.  Rank ``r`` of ``g``
owns rows ``[r*N/g, (r+1)*N/g)`` -- a contiguous byte range of the packed stream whenever
a row's bits end on a byte boundary -- computes ``y[:, rows]`` with the single-GPU kernels
and the ranks exchange their column blocks with ONE all-gather over NVLink (NCCL through
``torch.distributed``).  Activations and their per-token scales are replicated, so each
output element is produced by exactly one GPU.  The gathered result is bit-identical to the
one-GPU result whenever the shard and the whole layer sum an output in the same order (always
on the tensor-core kernel, whose order does not depend on the tile shape; on the small-M
kernel when both pick the same tile class), and otherwise equal up to the last bf16 bit.

The reference has no multi-GPU inference path (its only collective is the calibration
trainer's gradient all-reduce); this module is new work on top of the same payload format.

Nothing here waits on the device: the gather of chunk ``i`` runs on a side stream while
the GEMM of chunk ``i+1`` runs on the compute stream.

``fused_exchange=True`` replaces the all-gather by the GEMM itself: the result buffers of all
ranks are mapped into every process (CUDA IPC), and the GEMM epilogue stores each output
element into the local buffer and into every peer's buffer (``sacq_linear_a8_bcast``, plain
peer stores over NVLink), so the exchange overlaps the computation tile by tile.  What is left
after the kernel is a one-element all-reduce that orders the ranks; two buffers alternate so
a rank may start the next call while a slower peer still reads the previous result.
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


class _RawCuda:
    """A raw device pointer presented through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerBuffers:
    """``copies`` result buffers per rank, each mapped into every rank of the group.

    ``local[c]`` is this rank's buffer ``c`` (a uint8 tensor), ``peers[c]`` the device addresses
    of the other ranks' buffer ``c`` in this process, in rank order without this rank."""

    def __init__(self, nbytes: int, device: torch.device, group=None, copies: int = 2):
        import ctypes
        from . import _lib
        self._lib = _lib.load()
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        self.group = group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self._own, self._opened, self.local, self.peers = [], [], [], []
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._dev_index = dev_index
        for _ in range(copies):
            ptr = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            _lib.check(self._lib.sacq_peer_buffer_create(dev_index, self.nbytes, ctypes.byref(ptr), handle))
            self._own.append(ptr.value)
            everyone = [None] * world
            dist.all_gather_object(everyone, handle.raw, group=group)
            addrs = []
            for r in range(world):
                if r == rank:
                    continue
                p = ctypes.c_void_p()
                _lib.check(self._lib.sacq_peer_buffer_open(dev_index, everyone[r], ctypes.byref(p)))
                self._opened.append(p.value)
                addrs.append(p.value)
            self.peers.append(addrs)
            self.local.append(torch.as_tensor(_RawCuda(ptr.value, self.nbytes), device=self.device))

    def close(self):
        """Unmap the peers' buffers and free this rank's (collective: every rank calls it)."""
        if self._lib is None:
            return
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            self._lib.sacq_peer_buffer_close(self._dev_index, p)
        dist.barrier(group=self.group)                 # nobody still maps a buffer that is about to go
        for p in self._own:
            self._lib.sacq_peer_buffer_destroy(self._dev_index, p)
        self._own, self._opened, self.local, self.peers, self._lib = [], [], [], [], None


class ColumnParallelCodebookLinear(torch.nn.Module):
    """One rank's slice of a quantized linear plus the all-gather of the result.

    ``forward(x)`` takes the replicated ``[..., K]`` activations and returns the full
    ``[..., N]`` output on every rank.  ``chunks > 1`` splits the token dimension so the
    gather of one chunk overlaps the GEMM of the next."""

    def __init__(self, payload: dict, bias: torch.Tensor | None, device: str, group=None, chunks: int = 1,
                 fused_exchange: bool = False, max_tokens: int = 8192):
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
        self.fused_exchange = bool(fused_exchange) and self.world > 1
        self.max_tokens = int(max_tokens)
        self._peer = None
        self._turn = 0
        if self.fused_exchange:
            self._peer = PeerBuffers(self.max_tokens * self.out_features * 2, torch.device(device), group)
            self._order = torch.zeros(1, dtype=torch.float32, device=device)

    def close(self):
        if self._peer is not None:
            self._peer.close()
            self._peer = None

    def _forward_fused(self, a: torch.Tensor) -> torch.Tensor:
        """GEMM with the exchange in its epilogue.  Returns a view of one of the two mapped
        result buffers: it stays valid until the call after the next one."""
        import ctypes
        from . import _lib
        from .activation import quantize_rows
        from .linear import _Workspace, _stream_ptr
        m, n = a.shape[0], self.out_features
        if m > self.max_tokens:
            raise ValueError(f"{m} tokens exceed max_tokens={self.max_tokens} of the mapped result buffers")
        if a.dtype != torch.bfloat16:
            a = a.to(torch.bfloat16)
        q, s = quantize_rows(a.contiguous() if a.stride(-1) != 1 else a)
        c = self._turn
        self._turn ^= 1
        col0 = self.rank * (n // self.world)
        full = self._peer.local[c][: m * n * 2].view(torch.bfloat16).view(m, n)
        lib, layer = self.local._lib, self.local
        peers = (ctypes.c_void_p * (self.world - 1))(*[p + col0 * 2 for p in self._peer.peers[c]])
        buf = _Workspace.get(a.device).scratch(int(lib.sacq_workspace_bytes(layer._handle, m)))
        with torch.cuda.device(a.device):
            _lib.check(lib.sacq_linear_a8_bcast(layer._handle, q.data_ptr(), s.data_ptr(), m,
                                                full.data_ptr() + col0 * 2, peers, self.world - 1, n,
                                                buf.data_ptr(), buf.numel(), _stream_ptr()))
        # orders the ranks: when it completes here, every rank's kernel (and its peer stores) has
        dist.all_reduce(self._order, group=self.group)
        return full

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        a = x.reshape(-1, self.in_features)
        m = a.shape[0]
        if self.world == 1:
            return self.local(x)
        if self.fused_exchange:
            full = self._forward_fused(a)
            full = full if x.dtype == torch.bfloat16 else full.to(x.dtype)
            return full.reshape(*x.shape[:-1], self.out_features)
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
