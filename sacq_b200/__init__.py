"""sacq_b200 -- B200 (sm_100a) implementation of SACQ's packed vector-codebook
quantized-linear forward (W1.5A8): hand-written CUDA kernels behind a C ABI, with a
PyTorch module that keeps the reference's payload format and module interface.

Importing the package does not need a GPU; constructing a layer or calling a kernel
does, and fails loudly when the CUDA library has not been built."""
from .packing import index_bits_for, index_window_bytes, pack_indices, pack_payload, unpack_indices  # noqa: F401

__all__ = [
    "PrecomputedPackedVectorCodebookLinear", "forward_shared", "linear_a8_multi", "quantize_rows", "act_quantize_rows", "modulate_quantize_rows", "layernorm_quantize_rows", "pack_indices", "unpack_indices",
    "pack_payload", "index_bits_for", "index_window_bytes",
]


def __getattr__(name):
    if name == "PrecomputedPackedVectorCodebookLinear":
        from .linear import PrecomputedPackedVectorCodebookLinear
        return PrecomputedPackedVectorCodebookLinear
    if name == "forward_shared":
        from .linear import forward_shared
        return forward_shared
    if name == "linear_a8_multi":
        from .linear import linear_a8_multi
        return linear_a8_multi
    if name == "layernorm_quantize_rows":
        from .activation import layernorm_quantize_rows
        return layernorm_quantize_rows
    if name == "modulate_quantize_rows":
        from .activation import modulate_quantize_rows
        return modulate_quantize_rows
    if name == "act_quantize_rows":
        from .activation import act_quantize_rows
        return act_quantize_rows
    if name == "quantize_rows":
        from .activation import quantize_rows
        return quantize_rows
    raise AttributeError(name)
