"""Seeded synthetic layers and activations with the shapes and value distributions of
the W1.5A8 benchmark configurations (no checkpoint or dataset is needed).

``make_payload`` produces a ``packed_vector_codebook_v1`` dict with the keys, dtypes
and shapes the reference's fitter returns (sacq/vector_quantization.py:369-382):
group abs-max scales, weights normalised to [-1, 1], a vector codebook from a few
Lloyd iterations on a seeded sample, nearest-codeword indices.  It is a generator of
test inputs, not a re-implementation of the reference's fitting pipeline: the codebook
it finds is not bit-identical to the reference's, and nothing downstream needs it to be.
"""
from __future__ import annotations

import torch

from .packing import index_bits_for, pack_indices


def _assign(vectors: torch.Tensor, centers: torch.Tensor, budget: int = 32 * 1024 * 1024) -> torch.Tensor:
    """Nearest centre per vector, in chunks that bound the distance matrix."""
    chunk = max(1, budget // max(1, centers.shape[0]))
    c2 = (centers * centers).sum(1)
    out = torch.empty(vectors.shape[0], dtype=torch.int64, device=vectors.device)
    for s in range(0, vectors.shape[0], chunk):
        v = vectors[s:s + chunk]
        dist = c2[None, :] - 2.0 * (v @ centers.t())          # |v|^2 is constant per row
        out[s:s + chunk] = dist.argmin(dim=1)
    return out


@torch.no_grad()
def make_payload(out_features: int, in_features: int, *, vector_dim: int = 8, codebook_size: int = 4096,
                 group_size: int | None = None, seed: int = 0, iters: int = 2, sample_size: int = 65536,
                 weight_std: float = 0.02, device: str | torch.device = "cpu", fit: bool = True,
                 packed: bool = True) -> dict:
    """A synthetic quantized layer.  ``fit=False`` draws indices at random (fast, for very
    large codebooks or throw-away layers)."""
    group_size = in_features if group_size is None else group_size
    if in_features % group_size or group_size % vector_dim:
        raise ValueError("in_features % group_size and group_size % vector_dim must be 0")
    dev = torch.device(device)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    W = (torch.randn(out_features, in_features, generator=gen) * weight_std).to(dev)
    groups = in_features // group_size
    Wg = W.reshape(out_features, groups, group_size)
    scales = Wg.abs().amax(dim=2, keepdim=True).clamp_min(1e-8)
    vectors = (Wg / scales).clamp(-1.0, 1.0).reshape(-1, vector_dim).contiguous()
    n = vectors.shape[0]
    perm = torch.randperm(n, generator=gen)
    sample = vectors[perm[:min(n, max(sample_size, codebook_size))].to(dev)]
    if sample.shape[0] >= codebook_size:
        centers = sample[:codebook_size].clone()
    else:
        reps = (codebook_size + sample.shape[0] - 1) // sample.shape[0]
        centers = sample.repeat(reps, 1)[:codebook_size].clone()
    if fit:
        for _ in range(iters):
            a = _assign(sample, centers)
            sums = torch.zeros_like(centers).index_add_(0, a, sample)
            cnt = torch.bincount(a, minlength=codebook_size).to(sums.dtype)
            centers = torch.where(cnt[:, None] > 0, sums / cnt[:, None].clamp_min(1.0), centers).clamp(-1.0, 1.0)
        indices = _assign(vectors, centers)
    else:
        indices = torch.randint(0, codebook_size, (n,), generator=gen).to(dev)
    idx_dtype = torch.uint8 if codebook_size <= 256 else torch.int32
    payload = {
        "format": "packed_vector_codebook_v1",
        "codebook": centers.to("cpu", torch.bfloat16),
        "scales": scales.squeeze(-1).to("cpu", torch.bfloat16),
        "shift": torch.zeros((), dtype=torch.bfloat16),
        "in_features": in_features,
        "out_features": out_features,
        "group_size": group_size,
        "vector_dim": vector_dim,
        "codebook_fit_scale_squared": False,
    }
    idx = indices.reshape(out_features, groups, group_size // vector_dim).to("cpu", idx_dtype)
    if packed:
        bits = index_bits_for(codebook_size)
        payload.update(packed_indices=pack_indices(idx, bits), index_bits=bits, index_shape=tuple(idx.shape))
    else:
        payload["indices"] = idx
    return payload


def make_activations(m: int, k: int, *, seed: int = 1, outlier_seed: int = 2, outlier_fraction: float = 0.01,
                     outlier_gain: float = 20.0) -> torch.Tensor:
    """bf16 ``[m, k]`` activations: N(0, 1) with ``floor(k * fraction)`` channels scaled up."""
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(seed))
    n_out = int(k * outlier_fraction)
    if n_out > 0:
        cols = torch.randperm(k, generator=torch.Generator().manual_seed(outlier_seed))[:n_out]
        x[:, cols] *= outlier_gain
    return x.to(torch.bfloat16)


# (name, K, N) of the decoder linears in the decode-shape sweep
DECODE_SHAPES = (("q", 2048, 2048), ("kv", 2048, 1024), ("o", 2048, 2048), ("gate_up", 2048, 6144),
                 ("down", 6144, 2048))
DECODE_MS = (1, 2, 4, 8, 16, 32, 64)
# (name, vector_dim, codebook_size) of the mixed-bit set on a 2048 x 6144 layer
MIXED_BIT_SET = (("1bpw", 8, 256), ("1.5bpw", 8, 4096), ("2bpw", 8, 65536), ("3bpw", 4, 4096))


def algorithmic_bytes(n: int, k: int, m: int, *, vector_dim: int = 8, codebook_size: int = 4096,
                      group_size: int | None = None, bias: bool = False, fused_quant: bool = False) -> int:
    """Bytes one quantized-linear call must move: packed indices + codebook + scales +
    activations (e4m3 + fp32 scales, or bf16 when the quantizer is fused in) + bf16 output."""
    g = k if group_size is None else group_size
    b = index_bits_for(codebook_size)
    total = n * (k // vector_dim) * b // 8 + codebook_size * vector_dim * 2 + n * (k // g) * 2
    total += m * k * 2 if fused_quant else m * k + 4 * m
    total += 2 * m * n + (2 * n if bias else 0)
    return total
