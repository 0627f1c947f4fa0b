"""Loader for SACQ overlay files: ``{"weights": {module_name: payload}, "expected_applied": N,
"expected_packed_applied": N, "meta": ...}`` written by the reference's calibration export
(reference_sources/calibration/train_centroid_ft_2026_08_05.py:951-985) and read by its shim
(gr00t/eval/cosmos_quant_shim.py:589-733).

``apply_overlay`` walks the entries, replaces each named ``parent.attr`` linear with a
``PrecomputedPackedVectorCodebookLinear`` (packed entries), a ``SeparateQKVCodebookLinear`` (a
fused q/k/v projection whose three row blocks keep their own codebooks, the
``packed_separate_qkv_codebooks_v1`` wrapper of sacq/index_correction.py:99-100,210-217) or a
bf16 ``torch.nn.Linear`` (dense tensor entries), keeps the old layer's bias, and enforces the
reference's strictness:
a listed module that does not resolve is a ``KeyError`` and a final count that differs from
``expected_applied`` / ``expected_packed_applied`` is a ``RuntimeError``.
"""
from __future__ import annotations

import os
from typing import Callable, Iterable

import torch

PACKED_FORMAT = "packed_vector_codebook_v1"
SEPARATE_QKV_FORMAT = "packed_separate_qkv_codebooks_v1"
QKV_ROLES = ("q", "k", "v")                    # row order of the fused weight (sacq/index_correction.py:24)


def load_overlay(source, *, allow_pickle: bool = False) -> dict:
    """``source`` is a path to a ``torch.save`` file or an already loaded dict.  Files are read
    with ``weights_only=True`` (an overlay holds tensors, numbers and strings only);
    ``allow_pickle=True`` opts into the unrestricted unpickler for a file that is trusted."""
    if isinstance(source, (str, os.PathLike)):
        if not os.path.exists(source):
            raise FileNotFoundError(f"overlay file not found: {source}")
        source = torch.load(source, map_location="cpu", weights_only=not allow_pickle)
    if not isinstance(source, dict):
        raise ValueError("Invalid codebook overlay payload: expected a dict")
    weights = source.get("weights", source)
    if not isinstance(weights, dict) or not weights:
        raise ValueError("Invalid codebook overlay payload: no weights")
    return source


def is_packed(entry) -> bool:
    return isinstance(entry, dict) and entry.get("format") in (PACKED_FORMAT, SEPARATE_QKV_FORMAT)


def split_qkv_roles(entry: dict) -> list[dict]:
    """The three role payloads of a ``packed_separate_qkv_codebooks_v1`` entry in row order, after
    the reference's checks (exactly the roles q, k, v; one input width)."""
    roles = entry.get("roles")
    if not isinstance(roles, dict) or set(roles) != set(QKV_ROLES):
        raise ValueError("Fused Q/K/V must retain separate books")
    parts = [roles[r] for r in QKV_ROLES]
    if len({int(p["in_features"]) for p in parts}) != 1:
        raise ValueError("Fused Q/K/V roles must share in_features")
    return parts


class SeparateQKVCodebookLinear(torch.nn.Module):
    """A fused q/k/v projection whose row blocks keep their own codebooks: three packed layers on
    one shared per-token quantization of the input (one launch where their geometry allows),
    outputs concatenated in the order q, k, v -- the reconstruction order of the reference's
    ``decode_fixed`` for this format (sacq/index_correction.py:99-100)."""

    def __init__(self, entry: dict, bias, device: str, factory=None):
        super().__init__()
        factory = factory or _default_factory
        parts = split_qkv_roles(entry)
        sizes = [int(p["out_features"]) for p in parts]
        if bias is not None and bias.numel() != sum(sizes):
            raise ValueError("Fused weight row count mismatch")
        chunks = [None] * 3 if bias is None else list(torch.split(bias.detach(), sizes))
        self.roles = torch.nn.ModuleList(factory(p, b, device) for p, b in zip(parts, chunks))
        self.in_features = int(parts[0]["in_features"])
        self.out_features = sum(sizes)
        self.runtime_backend = "sacq_b200"
        self.runtime_scope = "unknown"

    def dequantize_weight(self) -> torch.Tensor:
        return torch.cat([m.dequantize_weight() for m in self.roles], dim=0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .linear import forward_shared
        return torch.cat(forward_shared(list(self.roles), x), dim=-1)


def _default_factory(payload, bias, device):
    from .linear import PrecomputedPackedVectorCodebookLinear
    return PrecomputedPackedVectorCodebookLinear(payload, bias=bias, device=device)


def apply_overlay(model: torch.nn.Module, source, device: str = "cuda:0", *, scope: str = "unknown",
                  allowed_suffixes: Iterable[str] | None = None, required_substring: str | None = None,
                  packed_only: bool = False, skip_packed: bool = False,
                  packed_factory: Callable | None = None, verbose: bool = False, allow_pickle: bool = False) -> int:
    """Install the overlay's layers into ``model``; returns how many were applied.

    ``allowed_suffixes`` silently skips other entries (the language-model overlay lists only
    ``.q_proj`` ... ``.down_proj``); ``required_substring`` makes an entry outside it an error
    (the action-head overlay requires ``"action_head."``)."""
    payload = load_overlay(source, allow_pickle=allow_pickle)
    weights = payload.get("weights", payload)
    factory = packed_factory or _default_factory
    named = dict(model.named_modules())
    suffixes = tuple(allowed_suffixes) if allowed_suffixes is not None else None
    applied = packed_applied = 0
    for full, entry in weights.items():
        if suffixes is not None and not full.endswith(suffixes):
            continue
        if required_substring is not None and required_substring not in full:
            raise KeyError(f"overlay entry outside {required_substring!r}: {full}")
        if "." in full:
            parent_name, attr = full.rsplit(".", 1)
        else:
            parent_name, attr = "", full
        parent = named.get(parent_name)
        if parent is None or not hasattr(parent, attr):
            raise KeyError(f"Codebook overlay target not found: {full}")
        packed = is_packed(entry)
        if (packed_only and not packed) or (skip_packed and packed):
            continue
        bias = getattr(getattr(parent, attr), "bias", None)
        if packed:
            if entry.get("format") == SEPARATE_QKV_FORMAT:
                replacement = SeparateQKVCodebookLinear(entry, bias, device, factory)
            else:
                replacement = factory(entry, bias, device)
            replacement.runtime_scope = scope
            replacement.runtime_name = full
            packed_applied += 1
        else:
            w = torch.as_tensor(entry).to(device=device, dtype=torch.bfloat16)
            replacement = torch.nn.Linear(w.shape[1], w.shape[0], bias=bias is not None, device=device,
                                          dtype=torch.bfloat16)
            replacement.weight.data.copy_(w)
            if bias is not None:
                replacement.bias.data.copy_(bias.detach().to(device=device, dtype=torch.bfloat16))
        setattr(parent, attr, replacement)
        applied += 1
        if verbose:
            print(f"[sacq_b200] applied overlay to {full}", flush=True)

    expected = payload.get("expected_applied")
    expected_packed = payload.get("expected_packed_applied")
    if expected_packed is None and expected is not None and all(is_packed(e) for e in weights.values()):
        expected_packed = expected
    if packed_only and expected_packed is not None and applied != int(expected_packed):
        raise RuntimeError(f"Packed overlay applied {applied}, expected {expected_packed}")
    if expected is not None and not (packed_only or skip_packed) and applied != int(expected):
        raise RuntimeError(f"Codebook overlay applied {applied} layers, expected {expected}")
    return applied


def apply_overlay_from_env(model: torch.nn.Module, env_var: str, device: str = "cuda:0", **kwargs) -> int:
    """Same, with the file path taken from an environment variable (``VLM_CODEBOOK_OVERLAY_PATH``,
    ``DIT_CODEBOOK_OVERLAY_PATH`` in the reference); an unset or empty variable applies nothing."""
    path = os.environ.get(env_var, "").strip()
    if not path:
        return 0
    return apply_overlay(model, path, device, **kwargs)
