"""Per-token FP8 activation quantizer (fused CUDA kernel).

Same contract as the reference's ``quantize_rows(x, mode)``
(gr00t_libero/acceleration/sources/libero_pro_eval/inference_acceleration_2026_10_11/
a8_accuracy_recovery_2026_10_20_r1/perrow_a8_candidate_r3.py:17-25) for
``mode == 'fp8_e4m3fn'``: returns ``(encoded [M, K] float8_e4m3fn, scale [M, 1] float32)``
with ``scale = absmax / 448`` per row (1 for an all-zero row).
"""
from __future__ import annotations

import torch

from . import _lib


def quantize_rows(x: torch.Tensor, mode: str = "fp8_e4m3fn", out: torch.Tensor | None = None,
                  scale_out: torch.Tensor | None = None):
    if x.ndim != 2 or x.dtype != torch.bfloat16:
        raise TypeError("quantize_rows expects a 2-D bfloat16 tensor")
    if mode != "fp8_e4m3fn":
        raise ValueError(f"unsupported mode {mode!r}; this implementation provides 'fp8_e4m3fn'")
    if not x.is_cuda:
        raise ValueError("quantize_rows needs a CUDA tensor; there is no CPU path")
    lib = _lib.load()
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    q = out if out is not None else torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = scale_out if scale_out is not None else torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if m > 0 and k > 0:
        with torch.cuda.device(x.device):
            _lib.check(lib.sacq_quant_act_fp8(x.data_ptr(), x.stride(0), m, k, q.data_ptr(), s.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream))
    return (q.view(torch.float8_e4m3fn) if q.dtype == torch.uint8 else q), s
