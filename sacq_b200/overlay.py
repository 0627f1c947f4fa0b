"""Loader for SACQ overlay files: ``{"weights": {module_name: payload}, "expected_applied": N,
"expected_packed_applied": N, "meta": ...}`` written by the reference's calibration export
(reference_sources/calibration/train_centroid_ft_2026_08_05.py:951-985) and read by its shim
(gr00t/eval/cosmos_quant_shim.py:589-733).

``apply_overlay`` walks the entries, replaces each named ``parent.attr`` linear with a
``PrecomputedPackedVectorCodebookLinear`` (packed entries) or a bf16 ``torch.nn.Linear``
(dense tensor entries), keeps the old layer's bias, and enforces the reference's strictness:
a listed module that does not resolve is a ``KeyError`` and a final count that differs from
``expected_applied`` / ``expected_packed_applied`` is a ``RuntimeError``.
"""
from __future__ import annotations

import os
from typing import Callable, Iterable

import torch

PACKED_FORMAT = "packed_vector_codebook_v1"


def load_overlay(source) -> dict:
    """``source`` is a path to a ``torch.save`` file or an already loaded dict."""
    if isinstance(source, (str, os.PathLike)):
        if not os.path.exists(source):
            raise FileNotFoundError(f"overlay file not found: {source}")
        source = torch.load(source, map_location="cpu", weights_only=False)
    if not isinstance(source, dict):
        raise ValueError("Invalid codebook overlay payload: expected a dict")
    weights = source.get("weights", source)
    if not isinstance(weights, dict) or not weights:
        raise ValueError("Invalid codebook overlay payload: no weights")
    return source


def is_packed(entry) -> bool:
    return isinstance(entry, dict) and entry.get("format") == PACKED_FORMAT


def _default_factory(payload, bias, device):
    from .linear import PrecomputedPackedVectorCodebookLinear
    return PrecomputedPackedVectorCodebookLinear(payload, bias=bias, device=device)


def apply_overlay(model: torch.nn.Module, source, device: str = "cuda:0", *, scope: str = "unknown",
                  allowed_suffixes: Iterable[str] | None = None, required_substring: str | None = None,
                  packed_only: bool = False, skip_packed: bool = False,
                  packed_factory: Callable | None = None, verbose: bool = False) -> int:
    """Install the overlay's layers into ``model``; returns how many were applied.

    ``allowed_suffixes`` silently skips other entries (the language-model overlay lists only
    ``.q_proj`` ... ``.down_proj``); ``required_substring`` makes an entry outside it an error
    (the action-head overlay requires ``"action_head."``)."""
    payload = load_overlay(source)
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
