"""The reference's CPU execution of the path, restated with the same PyTorch ops.

TEST/BENCHMARK INFRASTRUCTURE, NOT PRODUCT CODE.  This is what the reference itself
runs on a CPU: unpack with torch index arithmetic (cosmos_quant_shim.py:425-444),
bf16 gather / ``mul_`` / ``add_`` (sacq/index_correction.py:98-108), per-row FP8
quantizer (perrow_a8_candidate_r3.py:17-25) and a dense matmul.  It is the timed CPU
baseline of bench.py (all host threads through torch's intra-op pool) and is checked
against the reference-generated fixtures in tests/test_oracle_torch_port.py.
"""
from __future__ import annotations

import math

import torch


def unpack(packed: torch.Tensor, index_bits: int, index_shape) -> torch.Tensor:
    count = math.prod(index_shape)
    window = (index_bits + (8 - math.gcd(index_bits, 8)) + 7) // 8
    src = torch.cat([packed.reshape(-1), packed.new_zeros(window)])
    pos = torch.arange(count, dtype=torch.int64) * index_bits
    byte_ids = pos // 8
    words = src[byte_ids].to(torch.int64)
    for k in range(1, window):
        words |= src[byte_ids + k].to(torch.int64) << (8 * k)
    words >>= pos % 8
    words &= (1 << index_bits) - 1
    return words.reshape(index_shape)


def reconstruct(payload: dict) -> torch.Tensor:
    """bf16 [N, K]: gather, bf16 multiply by the group scale, bf16 add of the shift."""
    book = payload["codebook"].to(torch.bfloat16)
    if "packed_indices" in payload:
        ix = unpack(payload["packed_indices"], int(payload["index_bits"]), tuple(payload["index_shape"]))
    else:
        ix = payload["indices"].to(torch.long)
    scales = payload["scales"].to(torch.bfloat16)
    n, k, g = int(payload["out_features"]), int(payload["in_features"]), int(payload["group_size"])
    w = book[ix].reshape(n, -1, g)
    w.mul_(scales.unsqueeze(-1))
    w = w.reshape(n, k)
    w.add_(torch.as_tensor(payload.get("shift", 0.0), dtype=torch.bfloat16))
    return w


def quantize_rows(x: torch.Tensor):
    z = x.float()
    maximum = z.abs().amax(dim=1, keepdim=True)
    scale = torch.where(maximum > 0, maximum / 448.0, torch.ones_like(maximum))
    return (z / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn), scale


def forward(payload: dict, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """One A8 forward on CPU: quantize activations, reconstruct the weight (no cache, as the
    reference's recipe requires), fp32 matmul, scale, bias."""
    q, s = quantize_rows(x)
    w = reconstruct(payload)
    y = (q.float() @ w.float().t()) * s
    if bias is not None:
        y = y + bias.float()
    return y
