"""Drop-in quantized linear module backed by the sm_100a kernels.

Mirrors ``PrecomputedPackedVectorCodebookLinear`` of the reference
(gr00t_libero/sources/libero_pro_eval/Isaac-GR00T-N1.7/gr00t/eval/cosmos_quant_shim.py:313-541):
same constructor ``(payload, bias, device)``, same registered buffers and attributes
(``codebook``, ``packed_indices``, ``scales``, ``shift``, ``bias``, ``in_features``,
``out_features``, ``group_size``, ``vector_dim``, ``index_bits``, ``index_shape``,
``index_window_bytes``, ``runtime_backend``, ``runtime_scope``,
``runtime_kernel_eligible``), same ``dequantize_weight()`` result bit for bit, and a
``forward(x)`` that takes any ``[..., K]`` tensor and returns ``[..., N]`` in ``x.dtype``.

What differs is how ``forward`` computes: instead of materialising the bf16 weight and
calling a dense GEMM, it quantizes the activations per token to FP8 e4m3 and runs the
packed-index GEMM kernels (W1.5A8).  There is one backend and no CPU path: constructing
the module on a non-CUDA device raises.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from .packing import check_index_range, index_bits_for, index_window_bytes, pack_indices

_REQUIRED = ("codebook", "scales", "in_features", "out_features", "group_size", "vector_dim")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(index: int | None = None) -> int:
    """The current CUDA stream of device ``index`` (default: the current device) as an integer handle.
    The raw getter skips building a ``torch.cuda.Stream`` object, which costs more than a microsecond per
    call -- a visible share of a decode-sized layer call, whose whole host side is a few microseconds."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device() if index is None else index)
    return (torch.cuda.current_stream() if index is None else torch.cuda.current_stream(index)).cuda_stream


class _Workspace:
    """Scratch shared by the layers of a process, one set per (device, stream): split-K partial
    sums and the zero-initialised arrival counters of the small-M kernel, plus the FP8
    activation staging buffers.  Calls on one stream are ordered and may share a set; calls on
    different streams may overlap on the GPU, so each stream gets its own.  Grown on demand."""

    _by_device: dict[tuple[int, int], "_Workspace"] = {}

    def __init__(self, device: torch.device):
        self.device = device
        self.ws = None
        self.q = None
        self.scale = None
        self.host_scratch = None

    @classmethod
    def get(cls, device: torch.device) -> "_Workspace":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        key = (idx, _stream_ptr(idx))
        w = cls._by_device.get(key)
        if w is None:
            w = cls(torch.device("cuda", idx))
            cls._by_device[key] = w
        return w

    def scratch(self, nbytes: int) -> torch.Tensor:
        if self.ws is None or self.ws.numel() < nbytes:
            self.ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return self.ws

    def act(self, m: int, k: int):
        if self.q is None or self.q.numel() < m * k:
            self.q = torch.empty(max(m * k, 1 << 16), dtype=torch.uint8, device=self.device)
        if self.scale is None or self.scale.numel() < m:
            self.scale = torch.empty(max(m, 1024), dtype=torch.float32, device=self.device)
        return self.q, self.scale


class PrecomputedPackedVectorCodebookLinear(torch.nn.Module):
    """``packed_vector_codebook_v1`` layer executed by libsacq_b200."""

    def __init__(self, payload: dict, bias: torch.Tensor | None, device: str):
        super().__init__()
        missing = set(_REQUIRED).difference(payload)
        if missing:
            raise ValueError(f"Packed codebook payload is missing: {sorted(missing)}")
        if "indices" not in payload and "packed_indices" not in payload:
            raise ValueError("Packed codebook payload requires indices or packed_indices")
        device_obj = torch.device(device)
        if device_obj.type != "cuda":
            raise ValueError("sacq_b200 runs on CUDA devices only; there is no CPU path")
        if device_obj.index is None:
            device_obj = torch.device("cuda", torch.cuda.current_device())
        self._lib = _lib.load()                       # raises if the CUDA library is missing
        self.in_features = int(payload["in_features"])
        self.out_features = int(payload["out_features"])
        self.group_size = int(payload["group_size"])
        self.vector_dim = int(payload["vector_dim"])
        codebook = torch.as_tensor(payload["codebook"]).to(device=device_obj, dtype=torch.bfloat16).contiguous()
        self.register_buffer("codebook", codebook)

        if "packed_indices" in payload:
            self.index_bits = int(payload["index_bits"])
            self.index_shape = tuple(int(x) for x in payload["index_shape"])
            packed_source = torch.as_tensor(payload["packed_indices"])
            if packed_source.dtype != torch.uint8:
                packed_source = packed_source.to(torch.uint8)
            if packed_source.ndim != 1:
                raise ValueError(f"packed_indices must be flat, got shape={tuple(packed_source.shape)}")
            if self.index_bits < 1 or self.index_bits > 56:
                raise ValueError(f"index_bits must be in [1, 56], got {self.index_bits}")
        else:
            # an unpacked payload (uint8 or int32 indices) is serialised once at load time;
            # the kernels only ever see the bit stream
            source = torch.as_tensor(payload["indices"])
            check_index_range(source, int(codebook.shape[0]))
            self.index_shape = tuple(int(x) for x in source.shape)
            self.index_bits = index_bits_for(codebook.shape[0])
            packed_source = pack_indices(source, self.index_bits)
        expected_bytes = (math.prod(self.index_shape) * self.index_bits + 7) // 8
        if packed_source.numel() != expected_bytes:
            raise ValueError(
                f"packed_indices has {packed_source.numel()} bytes, expected {expected_bytes} "
                f"for shape={self.index_shape}, index_bits={self.index_bits}")
        self.index_window_bytes = index_window_bytes(self.index_bits)
        guard_bytes = self.index_window_bytes - 1
        # the buffer the attribute exposes has the reference's length (stream + window guard);
        # its storage is longer so the kernels' 128-bit reads stay inside the allocation
        storage = torch.zeros(expected_bytes + guard_bytes + _lib.SACQ_PACKED_GUARD_BYTES + 16,
                              dtype=torch.uint8, device=device_obj)
        storage[:expected_bytes].copy_(packed_source.to(device_obj))
        self._packed_storage = storage
        self.register_buffer("packed_indices", storage[: expected_bytes + guard_bytes])
        self.indices = None
        self._packed_bytes = expected_bytes

        self.register_buffer("scales", torch.as_tensor(payload["scales"]).to(device=device_obj, dtype=torch.bfloat16)
                             .contiguous())
        self.register_buffer("shift", torch.as_tensor(payload.get("shift", 0.0)).to(device=device_obj,
                                                                                     dtype=torch.bfloat16))
        if bias is None:
            self.bias = None
        else:
            self.register_buffer("bias", bias.detach().to(device=device_obj, dtype=torch.bfloat16).contiguous())

        self.runtime_backend = "sacq_b200"
        self.runtime_scope = "unknown"
        expected_index_shape = None
        if (self.vector_dim > 0 and self.group_size % self.vector_dim == 0
                and self.in_features % self.group_size == 0):
            expected_index_shape = (self.out_features, self.in_features // self.group_size,
                                    self.group_size // self.vector_dim)
        if self.index_shape != expected_index_shape:
            raise ValueError(f"index_shape {self.index_shape} does not match geometry {expected_index_shape}")
        if self.shift.numel() != 1:
            raise ValueError("shift must be a scalar")
        if tuple(self.scales.shape) != (self.out_features, self.in_features // self.group_size):
            raise ValueError(f"scales shape {tuple(self.scales.shape)} does not match geometry")
        if self.codebook.ndim != 2 or self.codebook.shape[1] != self.vector_dim:
            raise ValueError(f"codebook shape {tuple(self.codebook.shape)} does not match vector_dim")
        self.runtime_kernel_eligible = True
        self._ws_bytes = {}
        self._host_bytes = {}
        self._dev = device_obj                        # plain attribute: a buffer lookup per call costs a microsecond
        self._handle = None
        self._create_handle()

    # ------------------------------------------------------------------ handle
    def _create_handle(self):
        dev = self.codebook.device
        torch.cuda.synchronize(dev)          # uploads above must have landed before the tables are built
        desc = _lib.LayerDesc()
        desc.struct_size = ctypes.sizeof(_lib.LayerDesc)
        desc.device = dev.index
        desc.out_features = self.out_features
        desc.in_features = self.in_features
        desc.group_size = self.group_size
        desc.vector_dim = self.vector_dim
        desc.codebook_size = int(self.codebook.shape[0])
        desc.index_bits = self.index_bits
        desc.packed = self._packed_storage.data_ptr()
        desc.packed_bytes = self._packed_bytes
        desc.codebook = self.codebook.data_ptr()
        desc.scales = self.scales.data_ptr()
        desc.bias = self.bias.data_ptr() if self.bias is not None else None
        desc.shift_bf16 = int(self.shift.reshape(1).view(torch.int16).item()) & 0xFFFF
        handle = ctypes.c_void_p()
        _lib.check(self._lib.sacq_layer_create(ctypes.byref(desc), ctypes.byref(handle)))
        self._handle = handle

    def __del__(self):
        # runs during interpreter shutdown too: touch nothing but plain attributes
        d = self.__dict__
        h, lib = d.get("_handle"), d.get("_lib")
        d["_handle"] = None
        if h is not None and lib is not None:
            try:
                lib.sacq_layer_destroy(h)
            except Exception:
                pass

    def _apply(self, fn, recurse=True):
        # .to()/.cuda() would move the borrowed buffers out from under the handle
        old = self.codebook.data_ptr()
        out = super()._apply(fn, recurse)
        if self.codebook.data_ptr() != old:
            raise RuntimeError("a sacq_b200 layer is bound to the device it was created on; "
                               "construct a new module instead of moving it")
        return out

    # ------------------------------------------------------------------ reference API
    def dequantize_weight(self) -> torch.Tensor:
        """[N, K] bf16 reconstruction, bit-identical to the reference's."""
        w = torch.empty((self.out_features, self.in_features), dtype=torch.bfloat16, device=self.codebook.device)
        with torch.cuda.device(w.device):
            _lib.check(self._lib.sacq_dequant_bf16(self._handle, w.data_ptr(), _stream_ptr()))
        return w

    def quantize_activations(self, x: torch.Tensor):
        """Per-token FP8 quantization of a ``[M, K]`` bf16 tensor -> (e4m3 [M,K], fp32 [M,1])."""
        from .activation import quantize_rows
        return quantize_rows(x, "fp8_e4m3fn")

    def weight_row_scale(self, mode: str = "fp8_e4m3fn") -> torch.Tensor:
        """fp32 [N, 1]: max|W[n,:]| / 448 for ``'fp8_e4m3fn'`` or / 127 for ``'int8_symmetric'`` (the
        A8 recipe's per-output-row weight scale, ``quantize_rows(W, mode)[1]`` of the reference)."""
        if mode not in ("fp8_e4m3fn", "int8_symmetric"):
            raise ValueError(f"unknown weight format {mode!r}")
        sw = torch.empty((self.out_features, 1), dtype=torch.float32, device=self.codebook.device)
        fn = self._lib.sacq_weight_row_scale if mode == "fp8_e4m3fn" else self._lib.sacq_weight_row_scale_int8
        with torch.cuda.device(sw.device):
            _lib.check(fn(self._handle, sw.data_ptr(), _stream_ptr()))
        return sw

    def decode_weight_int8(self, weight_row_scale: torch.Tensor) -> torch.Tensor:
        """int8 [N, K] = round_half_even(clamp(W / row_scale, -127, 127)) decoded straight from the
        packed stream: the weight bytes of the reference's INT8 recipe."""
        sw = weight_row_scale.to(device=self.codebook.device, dtype=torch.float32).contiguous()
        if sw.numel() != self.out_features:
            raise ValueError("weight_row_scale must have out_features entries")
        wq = torch.empty((self.out_features, self.in_features), dtype=torch.int8, device=self.codebook.device)
        with torch.cuda.device(wq.device):
            _lib.check(self._lib.sacq_decode_weight_int8(self._handle, sw.data_ptr(), wq.data_ptr(), _stream_ptr()))
        return wq

    def linear_w8a8_int8(self, q: torch.Tensor, scale: torch.Tensor, weight_row_scale: torch.Tensor,
                         out: torch.Tensor | None = None) -> torch.Tensor:
        """The reference's deployed INT8 recipe: per-token int8 activations (``quantize_rows(x,
        'int8_symmetric')``) x per-output-row int8 weights (decoded per call), exact int32
        accumulation, ``bf16(fma(sa, float(acc) * sw, bias))``.  q int8 ``[M, K]``, scale fp32 ``[M]``,
        weight_row_scale = ``self.weight_row_scale('int8_symmetric')`` -> bf16 ``[M, N]``."""
        if q.dim() != 2 or q.shape[1] != self.in_features:
            raise ValueError("q must be [M, in_features]")
        if not q.is_cuda or q.device != self.codebook.device:
            raise ValueError("Matching CUDA operands required")
        if q.dtype != torch.int8:
            raise TypeError("q must be int8")
        q = q.contiguous()
        scale = scale.reshape(-1).to(torch.float32).contiguous()
        sw = weight_row_scale.reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        m = q.shape[0]
        if scale.numel() != m or sw.numel() != self.out_features:
            raise ValueError("scale needs one entry per row of q, weight_row_scale one per output feature")
        if out is None:
            out = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=q.device)
        buf = _Workspace.get(q.device).scratch(int(self._lib.sacq_workspace_bytes_w8a8(self._handle, m)))
        with torch.cuda.device(q.device):
            _lib.check(self._lib.sacq_linear_w8a8_int8(self._handle, q.data_ptr(), scale.data_ptr(), sw.data_ptr(), m,
                                                       out.data_ptr(), out.stride(0), buf.data_ptr(), buf.numel(),
                                                       _stream_ptr()))
        return out

    def linear_w8a8_fp8(self, q: torch.Tensor, scale: torch.Tensor, weight_row_scale: torch.Tensor,
                        out: torch.Tensor | None = None) -> torch.Tensor:
        """The reference's FP8 recipe: per-token e4m3 activations (``quantize_rows(x)``) x per-output-row
        e4m3 weights (re-quantized from the codebook weights, decoded per call), fp32 accumulation,
        ``bf16(fma(sa, acc * sw, bias))`` -- ``torch._scaled_mm(aq, wq.t(), sa, sw, bias)``.  q e4m3 (or its
        bytes) ``[M, K]``, scale fp32 ``[M]``, weight_row_scale = ``self.weight_row_scale('fp8_e4m3fn')``."""
        if q.dim() != 2 or q.shape[1] != self.in_features:
            raise ValueError("q must be [M, in_features]")
        if not q.is_cuda or q.device != self.codebook.device:
            raise ValueError("Matching CUDA operands required")
        if q.dtype not in (torch.float8_e4m3fn, torch.uint8):
            raise TypeError("q must be float8_e4m3fn (or its bytes as uint8)")
        q = q.contiguous()
        scale = scale.reshape(-1).to(torch.float32).contiguous()
        sw = weight_row_scale.reshape(-1).to(device=q.device, dtype=torch.float32).contiguous()
        m = q.shape[0]
        if scale.numel() != m or sw.numel() != self.out_features:
            raise ValueError("scale needs one entry per row of q, weight_row_scale one per output feature")
        if out is None:
            out = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=q.device)
        buf = _Workspace.get(q.device).scratch(int(self._lib.sacq_workspace_bytes_w8a8(self._handle, m)))
        with torch.cuda.device(q.device):
            _lib.check(self._lib.sacq_linear_w8a8_fp8(self._handle, q.data_ptr(), scale.data_ptr(), sw.data_ptr(), m,
                                                      out.data_ptr(), out.stride(0), buf.data_ptr(), buf.numel(),
                                                      _stream_ptr()))
        return out

    def decode_weight_fp8(self, weight_row_scale: torch.Tensor) -> torch.Tensor:
        """e4m3 [N, K] = e4m3(clamp(W / row_scale)) decoded straight from the packed stream."""
        sw = weight_row_scale.to(device=self.codebook.device, dtype=torch.float32).contiguous()
        if sw.numel() != self.out_features:
            raise ValueError("weight_row_scale must have out_features entries")
        wq = torch.empty((self.out_features, self.in_features), dtype=torch.uint8, device=self.codebook.device)
        with torch.cuda.device(wq.device):
            _lib.check(self._lib.sacq_decode_weight_fp8(self._handle, sw.data_ptr(), wq.data_ptr(), _stream_ptr()))
        return wq.view(torch.float8_e4m3fn)

    def linear_a8(self, q: torch.Tensor, scale: torch.Tensor, out: torch.Tensor | None = None,
                  residual: torch.Tensor | None = None) -> torch.Tensor:
        """GEMM on already-quantized activations: q e4m3 ``[M, K]``, scale fp32 ``[M]`` -> bf16 ``[M, N]``.
        ``residual`` (bf16 ``[M, N]``) is added in the GEMM epilogue: the bytes of
        ``linear_a8(q, scale) + residual``."""
        if q.dim() != 2 or q.shape[1] != self.in_features:
            raise ValueError("q must be [M, in_features]")
        if not q.is_cuda or q.device != self.codebook.device:
            raise ValueError("Matching CUDA operands required")
        if q.element_size() != 1:
            raise TypeError("q must hold e4m3 bytes")
        q = q.contiguous()
        scale = scale.reshape(-1).to(torch.float32).contiguous()
        m = q.shape[0]
        if scale.numel() != m:
            raise ValueError("scale must have one entry per row of q")
        if out is None:
            out = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=q.device)
        ws = _Workspace.get(q.device)
        need = int(self._lib.sacq_workspace_bytes(self._handle, m))
        buf = ws.scratch(need)
        if residual is not None:
            if residual.dtype != torch.bfloat16 or tuple(residual.shape) != (m, self.out_features) or \
                    residual.device != q.device or residual.stride(-1) != 1:
                raise ValueError("residual must be a bf16 [M, out_features] tensor on the layer's device")
        with torch.cuda.device(q.device):
            if residual is None:
                _lib.check(self._lib.sacq_linear_a8(self._handle, q.data_ptr(), scale.data_ptr(), m, out.data_ptr(),
                                                    out.stride(0), buf.data_ptr(), buf.numel(), _stream_ptr()))
            elif m > 0 and self.out_features > 0:
                _lib.check(self._lib.sacq_linear_a8_residual(self._handle, q.data_ptr(), scale.data_ptr(), m,
                                                             residual.data_ptr(), residual.stride(0), out.data_ptr(),
                                                             out.stride(0), buf.data_ptr(), buf.numel(), _stream_ptr()))
        return out

    def linear_a8i(self, q: torch.Tensor, scale: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """GEMM on INT8 per-token activations (``quantize_rows(x, 'int8_symmetric')``): q int8
        ``[M, K]``, scale fp32 ``[M]`` -> bf16 ``[M, N]``, with the exact (not re-quantized) weights."""
        if q.dim() != 2 or q.shape[1] != self.in_features:
            raise ValueError("q must be [M, in_features]")
        if not q.is_cuda or q.device != self.codebook.device:
            raise ValueError("Matching CUDA operands required")
        if q.dtype != torch.int8:
            raise TypeError("q must be int8")
        q = q.contiguous()
        scale = scale.reshape(-1).to(torch.float32).contiguous()
        m = q.shape[0]
        if scale.numel() != m:
            raise ValueError("scale must have one entry per row of q")
        if out is None:
            out = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=q.device)
        buf = _Workspace.get(q.device).scratch(int(self._lib.sacq_workspace_bytes_int8(self._handle, m)))
        with torch.cuda.device(q.device):
            _lib.check(self._lib.sacq_linear_a8i(self._handle, q.data_ptr(), scale.data_ptr(), m, out.data_ptr(),
                                                 out.stride(0), buf.data_ptr(), buf.numel(), _stream_ptr()))
        return out

    def forward_int8(self, x: torch.Tensor) -> torch.Tensor:
        """``forward`` with INT8 instead of FP8 per-token activations."""
        from .activation import quantize_rows
        if x.shape[-1] != self.in_features:
            raise ValueError("Linear shape mismatch")
        a = x.reshape(-1, self.in_features)
        if a.dtype != torch.bfloat16:
            a = a.to(torch.bfloat16)
        q, s = quantize_rows(a.contiguous() if a.stride(-1) != 1 else a, "int8_symmetric")
        y = self.linear_a8i(q, s).reshape(*x.shape[:-1], self.out_features)
        return y if x.dtype == torch.bfloat16 else y.to(x.dtype)

    def forward_residual(self, x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """``self(x) + residual`` with the addition done in the GEMM epilogue (bf16 operands)."""
        from .activation import quantize_rows
        if x.shape[-1] != self.in_features:
            raise ValueError("Linear shape mismatch")
        a = x.reshape(-1, self.in_features)
        if a.dtype != torch.bfloat16:
            a = a.to(torch.bfloat16)
        q, s = quantize_rows(a.contiguous() if a.stride(-1) != 1 else a)
        r = residual.reshape(-1, self.out_features)
        y = self.linear_a8(q, s, residual=r if r.dtype == torch.bfloat16 else r.to(torch.bfloat16))
        y = y.reshape(*x.shape[:-1], self.out_features)
        return y if x.dtype == torch.bfloat16 else y.to(x.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise ValueError("Linear shape mismatch")
        dev = self._dev
        if not x.is_cuda or x.device != dev:
            raise ValueError("Matching CUDA operands required")
        a = x if x.dim() == 2 else x.reshape(-1, self.in_features)
        if a.dtype != torch.bfloat16:
            a = a.to(torch.bfloat16)
        if a.stride(-1) != 1:
            a = a.contiguous()
        m = a.shape[0]
        y = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=dev)
        if m > 0 and self.out_features > 0:
            ws = _Workspace.get(dev)
            need = self._ws_bytes.get(m)
            if need is None:
                need = self._ws_bytes[m] = int(self._lib.sacq_workspace_bytes(self._handle, m))
            buf = ws.scratch(need)
            q, s = ws.act(m, self.in_features)
            if torch.cuda.current_device() == dev.index:
                rc = self._lib.sacq_linear_bf16(
                    self._handle, a.data_ptr(), a.stride(0), m, q.data_ptr(), s.data_ptr(), y.data_ptr(),
                    y.stride(0), buf.data_ptr(), buf.numel(), _stream_ptr(dev.index))
            else:
                with torch.cuda.device(dev):
                    rc = self._lib.sacq_linear_bf16(
                        self._handle, a.data_ptr(), a.stride(0), m, q.data_ptr(), s.data_ptr(), y.data_ptr(),
                        y.stride(0), buf.data_ptr(), buf.numel(), _stream_ptr(dev.index))
            if rc != 0:
                _lib.check(rc)
        if x.dim() != 2:
            y = y.reshape(*x.shape[:-1], self.out_features)
        return y if x.dtype == torch.bfloat16 else y.to(x.dtype)

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor | None = None) -> torch.Tensor:
        """Forward for host-resident activations: ``x_host`` is a CPU bf16 ``[M, K]`` tensor
        (pinned for asynchronous copies), the result is a CPU bf16 ``[M, N]`` tensor.  The
        copies and kernels are enqueued on the current stream of the layer's device; the
        caller synchronises that stream before reading ``out_host``."""
        if x_host.is_cuda or x_host.dtype != torch.bfloat16 or x_host.dim() != 2 or not x_host.is_contiguous():
            raise TypeError("forward_host expects a contiguous 2-D bfloat16 CPU tensor")
        if x_host.shape[1] != self.in_features:
            raise ValueError("Linear shape mismatch")
        m = x_host.shape[0]
        if out_host is None:
            out_host = torch.empty((m, self.out_features), dtype=torch.bfloat16, pin_memory=x_host.is_pinned())
        dev = self._dev
        need = self._host_bytes.get(m)
        if need is None:
            need = self._host_bytes[m] = int(self._lib.sacq_host_forward_scratch_bytes(self._handle, m))
        ws = _Workspace.get(dev)
        if ws.host_scratch is None or ws.host_scratch.numel() < need:
            ws.host_scratch = torch.zeros(max(need, 1 << 22), dtype=torch.uint8, device=dev)
        buf = ws.host_scratch
        if m > 0 and self.out_features > 0:
            # the library switches to the layer's device itself; the stream is that device's current one
            rc = self._lib.sacq_linear_bf16_host(self._handle, x_host.data_ptr(), m, out_host.data_ptr(),
                                                 buf.data_ptr(), buf.numel(), _stream_ptr(dev.index))
            if rc != 0:
                _lib.check(rc)
        return out_host

    # ------------------------------------------------------------------ extras
    def set_kernel(self, which: str | int) -> None:
        """Force a GEMM kernel: 'auto' (0), 'small' (1), 'large' (2), 'small_simt' (3), 'small_mma' (4),
        'small_mma_direct' (5), 'small_mma_unpacked' (6), 'large_grouped' (7), 'large_tmem' (8; 9-11 also
        fix its token sub-tiles per CTA to 1-3), 'large_tmem_grouped' (12; 13-15 likewise)."""
        code = {"auto": 0, "small": 1, "large": 2, "small_simt": 3, "small_mma": 4, "small_mma_direct": 5,
                "small_mma_unpacked": 6, "large_grouped": 7, "large_tmem": 8, "large_tmem1": 9,
                "large_tmem2": 10, "large_tmem3": 11, "large_tmem_grouped": 12, "large_tmem_grouped1": 13,
                "large_tmem_grouped2": 14, "large_tmem_grouped3": 15}.get(which, which)
        _lib.check(self._lib.sacq_layer_set_kernel(self._handle, int(code)))
        self._ws_bytes.clear()
        self._host_bytes.clear()

    def kernel_for(self, m: int) -> str:
        k = self._lib.sacq_layer_kernel_for(self._handle, m)
        if k < 0:
            _lib.check(k)
        return {1: "small", 2: "large", 3: "large_grouped", 4: "large_tmem", 5: "large_tmem_grouped"}[k]

    def device_status(self) -> int:
        st = ctypes.c_int(0)
        _lib.check(self._lib.sacq_layer_status(self._handle, ctypes.byref(st)))
        return st.value

    def resident_bytes(self) -> int:
        """Device bytes held for this layer: payload buffers plus derived tables."""
        own = sum(t.numel() * t.element_size() for t in (self._packed_storage, self.codebook, self.scales, self.shift))
        if self.bias is not None:
            own += self.bias.numel() * 2
        return own + int(self._lib.sacq_layer_resident_bytes(self._handle))

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, vector_dim={self.vector_dim}, "
                f"codebook={tuple(self.codebook.shape)}, index_bits={self.index_bits}, group_size={self.group_size}")


def forward_shared(layers, x: torch.Tensor):
    """Sibling projections that read the same input (q/k/v, gate/up): quantize ``x`` once and
    run every layer's GEMM on the shared FP8 activations, as the reference's overlay does
    (int8_shared_padded_activation_20261028_r1.py:44-63).  Returns one output per layer, each
    identical to ``layer(x)``."""
    from .activation import quantize_rows
    layers = list(layers)
    k = layers[0].in_features
    if any(l.in_features != k for l in layers):
        raise ValueError("layers that share an input must have the same in_features")
    a = x.reshape(-1, k)
    if a.dtype != torch.bfloat16:
        a = a.to(torch.bfloat16)
    q, s = quantize_rows(a.contiguous() if a.stride(-1) != 1 else a)
    ys = linear_a8_multi(layers, q, s)
    outs = []
    for layer, y in zip(layers, ys):
        y = y.reshape(*x.shape[:-1], layer.out_features)
        outs.append(y if x.dtype == torch.bfloat16 else y.to(x.dtype))
    return outs


def linear_a8_multi(layers, q: torch.Tensor, scale: torch.Tensor):
    """GEMMs of several layers on one set of quantized activations (``sacq_linear_a8_multi``):
    layers of one geometry run as a single launch at small M.  Returns one bf16 ``[M, N_l]``
    tensor per layer, byte-identical to ``layer.linear_a8(q, scale)``."""
    import ctypes
    layers = list(layers)
    first = layers[0]
    if q.dim() != 2 or any(l.in_features != q.shape[1] for l in layers):
        raise ValueError("q must be [M, in_features] of every layer")
    if not q.is_cuda or any(l.codebook.device != q.device for l in layers):
        raise ValueError("Matching CUDA operands required")
    if q.element_size() != 1:
        raise TypeError("q must hold e4m3 bytes")
    q = q.contiguous()
    scale = scale.reshape(-1).to(torch.float32).contiguous()
    m = q.shape[0]
    if scale.numel() != m:
        raise ValueError("scale must have one entry per row of q")
    outs = [torch.empty((m, l.out_features), dtype=torch.bfloat16, device=q.device) for l in layers]
    n = len(layers)
    lib = first._lib
    need = max(int(lib.sacq_workspace_bytes(l._handle, m)) for l in layers)
    buf = _Workspace.get(q.device).scratch(need)
    handles = (ctypes.c_void_p * n)(*[l._handle.value for l in layers])
    ys = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
    ldys = (ctypes.c_int64 * n)(*[o.stride(0) for o in outs])
    with torch.cuda.device(q.device):
        _lib.check(lib.sacq_linear_a8_multi(handles, n, q.data_ptr(), scale.data_ptr(), m, ys, ldys, buf.data_ptr(),
                                            buf.numel(), _stream_ptr()))
    return outs
