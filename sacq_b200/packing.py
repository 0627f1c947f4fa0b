"""Host-side serialisation of codebook indices (load-time, CPU).

Same bit layout as the reference's ``pack_indices``
(sacq/calibration_layers.py:44-74) and ``pack_payload``
(gr00t_libero/acceleration/bootstrap_sources/gr00t_final_seed17_20260922/
pack_sacq_reference.py:9-30): index ``i`` occupies bits ``[i*b, i*b+b)`` of one
little-endian stream over the flattened ``[N, K/G, G/d]`` index tensor.
"""
from __future__ import annotations

import math

import torch


def index_bits_for(codebook_size: int) -> int:
    """Field width used when serialising a codebook of this size."""
    return max(1, (int(codebook_size) - 1).bit_length())


def index_window_bytes(index_bits: int) -> int:
    """Bytes a field can touch when it starts at the least favourable bit offset."""
    return (index_bits + (8 - math.gcd(index_bits, 8)) + 7) // 8


def check_index_range(indices: torch.Tensor, codebook_size: int) -> None:
    """Raise IndexError if an index does not address a codeword (the reference's CPU gather
    ``codebook[indices]`` raises the same; a GPU gather would read out of bounds)."""
    flat = torch.as_tensor(indices).detach().reshape(-1)
    if flat.numel() == 0:
        return
    lo, hi = int(flat.min()), int(flat.max())
    if lo < 0 or hi >= int(codebook_size):
        raise IndexError(f"index {lo if lo < 0 else hi} is out of bounds for a codebook of {int(codebook_size)} entries")


def pack_indices(indices: torch.Tensor, index_bits: int) -> torch.Tensor:
    """Flat uint8 tensor of ``ceil(count * index_bits / 8)`` bytes."""
    if index_bits < 1 or index_bits > 56:
        raise ValueError(f"index_bits must be in [1, 56], got {index_bits}")
    flat = torch.as_tensor(indices).detach().cpu().reshape(-1).to(torch.int64)
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= (1 << index_bits)):
        raise ValueError(f"indices do not fit in {index_bits} bits")
    count = flat.numel()
    n_bytes = (count * index_bits + 7) // 8
    # bit-plane scatter: bit j of index i lands at stream bit i*b + j
    stream_bits = torch.zeros(n_bytes * 8, dtype=torch.uint8)
    base = torch.arange(count, dtype=torch.int64) * index_bits
    for j in range(index_bits):
        stream_bits[base + j] = ((flat >> j) & 1).to(torch.uint8)
    weights = (1 << torch.arange(8, dtype=torch.int64)).to(torch.uint8)
    return (stream_bits.reshape(n_bytes, 8) * weights).sum(dim=1, dtype=torch.int64).to(torch.uint8)


def unpack_indices(packed: torch.Tensor, index_bits: int, count: int) -> torch.Tensor:
    """Inverse of :func:`pack_indices` (int64, CPU)."""
    p = torch.as_tensor(packed).detach().cpu().reshape(-1).to(torch.uint8)
    bits = ((p.to(torch.int64).unsqueeze(1) >> torch.arange(8, dtype=torch.int64)) & 1).reshape(-1)
    need = count * index_bits
    if bits.numel() < need:
        raise ValueError(f"packed stream has {p.numel()} bytes, need {(need + 7) // 8}")
    fields = bits[:need].reshape(count, index_bits)
    return (fields << torch.arange(index_bits, dtype=torch.int64)).sum(dim=1)


def pack_payload(payload: dict) -> dict:
    """Return a copy of an ``indices`` payload with ``packed_indices``, ``index_bits`` and
    ``index_shape`` in place of ``indices``."""
    if "indices" not in payload or "packed_indices" in payload:
        raise ValueError("pack_payload expects a payload with 'indices' and without 'packed_indices'")
    source = torch.as_tensor(payload["indices"]).detach().cpu()
    bits = index_bits_for(int(torch.as_tensor(payload["codebook"]).shape[0]))
    out = {k: v for k, v in payload.items() if k != "indices"}
    out.update(packed_indices=pack_indices(source, bits), index_bits=bits, index_shape=tuple(source.shape))
    return out
