"""The allocation-free entry point, sacq_linear_a8_static_scratch.

It serves callers that must not allocate device memory once they are running (a control
loop with a fixed memory budget, a server whose arena owns the GPU).  Its scratch is an
array inside the library, shared by every call, so the test calls it twice in a row -- the
second call starts from the first call's leftovers -- and compares both results with the
ordinary entry point given a caller-allocated workspace.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from oracle import sacq_oracle as O

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, _lib, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload

    N, K = 2048, 2048
    payload = make_payload(N, K, seed=21, device="cuda", iters=1)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 0.05).to(torch.bfloat16)
    layer = PrecomputedPackedVectorCodebookLinear(payload, bias, "cuda")
    lib = layer._lib
    assert lib.sacq_static_scratch_bytes() == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream

    for call, (M, seed) in enumerate(((4, 1), (16, 2))):     # two calls in a row, different sizes
        q, s = quantize_rows(make_activations(M, K, seed=seed).cuda())
        s = s.reshape(-1).contiguous()
        layer.set_kernel("small_simt")                      # the kernel that uses split-K scratch
        want = layer.linear_a8(q, s)
        layer.set_kernel("auto")
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        free_before = torch.cuda.mem_get_info()[0]
        _lib.check(lib.sacq_linear_a8_static_scratch(layer._handle, q.data_ptr(), s.data_ptr(), M, got.data_ptr(),
                                                     N, stream))
        torch.cuda.synchronize()
        if call > 0:
            # the first call on a device makes the driver load the library image that holds the
            # built-in array; after that set-up a call changes nothing in device memory
            assert torch.cuda.mem_get_info()[0] == free_before, "the call must not allocate device memory"
        err = O.rel_frobenius(got.float().cpu().numpy(), want.float().cpu().numpy())
        assert err <= 1e-2, err
        assert torch.equal(got, want)                       # same kernel, same order of additions
        # and against the CPU oracle, with the tolerance of the other GEMM tests
        w_bits = layer.dequantize_weight().cpu().view(torch.int16).numpy().view(np.uint16)
        ref = O.linear_a8_reference(q.view(torch.uint8).cpu().numpy(), s.cpu().numpy(), w_bits,
                                    bias.view(torch.int16).numpy().view(np.uint16))
        assert O.rel_frobenius(got.float().cpu().numpy(), ref) <= 1e-2

    # a request beyond the built-in array is refused with a clear message, nothing is launched
    big = 8192
    q = torch.zeros(big, K, dtype=torch.uint8, device="cuda")
    s = torch.ones(big, device="cuda")
    out = torch.empty(big, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.sacq_linear_a8_static_scratch(layer._handle, q.data_ptr(), s.data_ptr(), big, out.data_ptr(), N, stream)
    assert rc == -4 and "built-in scratch" in _lib.last_error()
    assert layer.device_status() == 0

    # argument checks: an empty batch is a no-op that touches nothing, a negative one, a null
    # buffer, a short pitch and a null layer are refused before anything is launched
    sentinel = out[:4].clone()
    assert lib.sacq_linear_a8_static_scratch(layer._handle, None, None, 0, None, N, stream) == 0
    assert lib.sacq_linear_a8_static_scratch(layer._handle, q.data_ptr(), s.data_ptr(), -1, out.data_ptr(), N, stream) == -1
    assert lib.sacq_linear_a8_static_scratch(layer._handle, None, s.data_ptr(), 4, out.data_ptr(), N, stream) == -1
    assert lib.sacq_linear_a8_static_scratch(layer._handle, q.data_ptr(), None, 4, out.data_ptr(), N, stream) == -1
    assert lib.sacq_linear_a8_static_scratch(layer._handle, q.data_ptr(), s.data_ptr(), 4, None, N, stream) == -1
    assert lib.sacq_linear_a8_static_scratch(layer._handle, q.data_ptr(), s.data_ptr(), 4, out.data_ptr(), N - 1, stream) == -1
    assert lib.sacq_linear_a8_static_scratch(None, q.data_ptr(), s.data_ptr(), 4, out.data_ptr(), N, stream) == -1
    torch.cuda.synchronize()
    assert torch.equal(out[:4], sentinel) and layer.device_status() == 0
