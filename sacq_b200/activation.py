"""Per-token FP8 activation quantizer (fused CUDA kernel).

Same contract as the reference's ``quantize_rows(x, mode)``
(gr00t_libero/acceleration/sources/libero_pro_eval/inference_acceleration_2026_10_11/
a8_accuracy_recovery_2026_10_20_r1/perrow_a8_candidate_r3.py:17-25) for
``mode == 'fp8_e4m3fn'``: returns ``(encoded [M, K] float8_e4m3fn, scale [M, 1] float32)``
with ``scale = absmax / 448`` per row (1 for an all-zero row), and for
``mode == 'int8_symmetric'`` (the deployed recipe): ``(encoded [M, K] int8, scale)`` with
``scale = absmax / 127`` and round-half-to-even.
"""
from __future__ import annotations

import torch

from . import _lib


def quantize_rows(x: torch.Tensor, mode: str = "fp8_e4m3fn", out: torch.Tensor | None = None,
                  scale_out: torch.Tensor | None = None):
    if x.ndim != 2 or x.dtype != torch.bfloat16:
        raise TypeError("quantize_rows expects a 2-D bfloat16 tensor")
    if mode not in ("fp8_e4m3fn", "int8_symmetric"):
        raise ValueError(f"unsupported mode {mode!r}; this implementation provides 'fp8_e4m3fn' and 'int8_symmetric'")
    if not x.is_cuda:
        raise ValueError("quantize_rows needs a CUDA tensor; there is no CPU path")
    lib = _lib.load()
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    q = out if out is not None else torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = scale_out if scale_out is not None else torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if m > 0 and k > 0:
        fn = lib.sacq_quant_act_fp8 if mode == "fp8_e4m3fn" else lib.sacq_quant_act_int8
        with torch.cuda.device(x.device):
            _lib.check(fn(x.data_ptr(), x.stride(0), m, k, q.data_ptr(), s.data_ptr(),
                          torch.cuda.current_stream().cuda_stream))
    if mode == "int8_symmetric":
        return (q.view(torch.int8) if q.dtype == torch.uint8 else q), s
    return (q.view(torch.float8_e4m3fn) if q.dtype == torch.uint8 else q), s


def act_quantize_rows(kind: str, a: torch.Tensor, b: torch.Tensor | None = None):
    """Activation function fused into the per-token quantizer (``sacq_act_quant_fp8``):

    * ``kind='silu_mul'``: the bytes of ``quantize_rows(F.silu(a) * b)`` (gated MLP);
    * ``kind='gelu'``:     the bytes of ``quantize_rows(F.gelu(a))`` (erf form);

    in one launch, without materialising the ``[M, K]`` intermediate."""
    kinds = {"silu_mul": 0, "gelu": 1}
    if kind not in kinds:
        raise ValueError(f"unknown activation kind {kind!r}")
    if a.ndim != 2 or a.dtype != torch.bfloat16 or not a.is_cuda:
        raise TypeError("act_quantize_rows expects 2-D bfloat16 CUDA tensors")
    if kind == "silu_mul":
        if b is None or b.shape != a.shape or b.dtype != torch.bfloat16 or b.device != a.device:
            raise TypeError("silu_mul needs a second bfloat16 tensor of the same shape and device")
        if b.stride(1) != 1:
            b = b.contiguous()
    if a.stride(1) != 1:
        a = a.contiguous()
    lib = _lib.load()
    m, k = a.shape
    q = torch.empty((m, k), dtype=torch.uint8, device=a.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=a.device)
    if m > 0 and k > 0:
        with torch.cuda.device(a.device):
            _lib.check(lib.sacq_act_quant_fp8(kinds[kind], a.data_ptr(), a.stride(0),
                                              b.data_ptr() if kind == "silu_mul" else None,
                                              b.stride(0) if kind == "silu_mul" else 0, m, k, q.data_ptr(),
                                              s.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return q.view(torch.float8_e4m3fn), s


def modulate_quantize_rows(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor):
    """AdaLN modulation fused into the quantizer (``sacq_modulate_quant_fp8``): the bytes of
    ``quantize_rows(x * (1 + scale) + shift)`` for bf16 ``x [M, K]`` and bf16 vectors
    ``scale, shift [K]``, in one launch."""
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda:
        raise TypeError("modulate_quantize_rows expects a 2-D bfloat16 CUDA tensor")
    k = x.shape[1]
    for v in (scale, shift):
        if v.dtype != torch.bfloat16 or v.numel() != k or v.device != x.device:
            raise TypeError("scale and shift must be bfloat16 vectors of K elements on x's device")
    scale, shift = scale.reshape(-1).contiguous(), shift.reshape(-1).contiguous()
    if x.stride(1) != 1:
        x = x.contiguous()
    lib = _lib.load()
    m = x.shape[0]
    q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if m > 0 and k > 0:
        with torch.cuda.device(x.device):
            _lib.check(lib.sacq_modulate_quant_fp8(x.data_ptr(), x.stride(0), scale.data_ptr(), shift.data_ptr(), m, k,
                                                   q.data_ptr(), s.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return q.view(torch.float8_e4m3fn), s


def layernorm_quantize_rows(x: torch.Tensor, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                            eps: float = 1e-5, mod_scale: torch.Tensor | None = None,
                            mod_shift: torch.Tensor | None = None, return_normalized: bool = False):
    """LayerNorm over the last dimension, optionally the AdaLN modulation ``y * (1 + s) + t``,
    and the per-token FP8 quantizer in one launch (``sacq_layernorm_quant_fp8``).  Returns
    ``(q, scale)`` or ``(q, scale, y)`` with the bf16 normalised tensor.  ``y`` agrees with
    ``torch.nn.functional.layer_norm`` to one bf16 ulp (different reduction order); ``q`` and
    ``scale`` are exactly ``quantize_rows(y)``."""
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda:
        raise TypeError("layernorm_quantize_rows expects a 2-D bfloat16 CUDA tensor")
    k = x.shape[1]
    vecs = []
    for v in (weight, bias, mod_scale, mod_shift):
        if v is not None:
            if v.dtype != torch.bfloat16 or v.numel() != k or v.device != x.device:
                raise TypeError("weight, bias and modulation vectors must be bfloat16 with K elements on x's device")
            v = v.reshape(-1).contiguous()
        vecs.append(v)
    if (vecs[2] is None) != (vecs[3] is None):
        raise ValueError("modulation needs both its scale and its shift vector")
    if x.stride(1) != 1:
        x = x.contiguous()
    lib = _lib.load()
    m = x.shape[0]
    q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    y = torch.empty((m, k), dtype=torch.bfloat16, device=x.device) if return_normalized else None
    if m > 0 and k > 0:
        ptr = [None if v is None else v.data_ptr() for v in vecs]
        with torch.cuda.device(x.device):
            _lib.check(lib.sacq_layernorm_quant_fp8(x.data_ptr(), x.stride(0), ptr[0], ptr[1], float(eps), ptr[2], ptr[3],
                                                    m, k, None if y is None else y.data_ptr(), k, q.data_ptr(),
                                                    s.data_ptr(), torch.cuda.current_stream().cuda_stream))
    q = q.view(torch.float8_e4m3fn)
    return (q, s, y) if return_normalized else (q, s)
