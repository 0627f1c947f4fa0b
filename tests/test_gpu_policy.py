"""The synthetic policy forward: runs, is finite and deterministic, and its quantized
linears agree with dense reconstruct-then-matmul on the same quantized activations."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_policy_forward_runs_and_is_deterministic():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sacq_b200.policy import SyntheticGr00tPolicy
    policy = SyntheticGr00tPolicy("cuda", seed=1)
    image, noise = policy.example_inputs(42)
    a = policy(image, noise)
    b = policy(image, noise)
    torch.cuda.synchronize()
    assert tuple(a.shape) == (16, 32) and a.dtype == torch.bfloat16
    assert bool(torch.isfinite(a.float()).all())
    assert torch.equal(a, b)
    assert policy.num_quantized_linears == 24 * 6 + 1 + 12 * 7 + 16 * 11
    # sibling projections on one shared quantization give the same bytes as separate forwards
    from sacq_b200 import forward_shared
    blk = policy.llm[0]
    h = (torch.randn(300, 2048, generator=torch.Generator().manual_seed(3))).to("cuda", torch.bfloat16)
    for got, layer in zip(forward_shared((blk.q, blk.k, blk.v), h), (blk.q, blk.k, blk.v)):
        assert torch.equal(got, layer(h))
    # one layer of each tower against the dense product of its own reconstruction
    for layer, m in ((policy.vit[0].up, 256), (policy.llm[0].down, 300), (policy.dit[0].q, 16)):
        x = (torch.randn(m, layer.in_features, generator=torch.Generator().manual_seed(m)) * 2).to("cuda", torch.bfloat16)
        q, s = layer.quantize_activations(x)
        ref = (q.float() @ layer.dequantize_weight().float().t()) * s
        err = ((layer(x).float() - ref).norm() / ref.norm()).item()
        assert err <= 1e-2, err


def test_policy_batch_matches_single_requests():
    """A batch of independent requests gives every request the result of its own batch-1
    forward.  Not bit for bit: with more rows the linears move to other kernels (another
    summation order, FP8 high/low instead of fp16 codewords) and the attention kernel changes
    its tiling, and those last-bit differences pass through 52 blocks; the bar is 2e-2 relative
    Frobenius on the actions (the path's own GEMM tolerance is 1e-2 per layer)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sacq_b200.policy import SyntheticGr00tPolicy
    policy = SyntheticGr00tPolicy("cuda", seed=2)
    image, noise = policy.example_inputs(7, batch=3)
    batched = policy(image, noise)
    torch.cuda.synchronize()
    assert tuple(batched.shape) == (3, 16, 32) and bool(torch.isfinite(batched.float()).all())
    assert torch.equal(batched, policy(image, noise))
    for i in range(3):
        single = policy(image[i], noise[i])
        err = ((batched[i].float() - single.float()).norm() / single.float().norm()).item()
        assert err <= 2e-2, (i, err)
    # requests do not leak into each other: changing request 2 leaves requests 0 and 1 unchanged
    image2 = image.clone()
    image2[2] = 1.0 - image2[2]
    again = policy(image2, noise)
    assert torch.equal(again[:2], batched[:2]) and not torch.equal(again[2], batched[2])


def test_overlay_installs_real_layers():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, overlay
    from sacq_b200.synthetic import make_payload

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(256, 128, bias=True, device="cuda", dtype=torch.bfloat16)
            self.up_proj = torch.nn.Linear(256, 512, bias=False, device="cuda", dtype=torch.bfloat16)

    model = torch.nn.ModuleDict({"blk": Block()})
    ov = {"weights": {"blk.q_proj": make_payload(128, 256, seed=1, iters=1),
                      "blk.up_proj": make_payload(512, 256, seed=2, iters=1)}, "expected_applied": 2}
    bias = model["blk"].q_proj.bias.detach().clone()
    assert overlay.apply_overlay(model, ov, "cuda:0", scope="vlm",
                                 allowed_suffixes=(".q_proj", ".up_proj")) == 2
    q = model["blk"].q_proj
    assert isinstance(q, PrecomputedPackedVectorCodebookLinear) and q.runtime_scope == "vlm"
    assert torch.equal(q.bias, bias)
    x = torch.randn(4, 256, device="cuda", dtype=torch.bfloat16)
    aq, s = q.quantize_activations(x)
    ref = (aq.float() @ q.dequantize_weight().float().t()) * s + bias.float()
    assert ((q(x).float() - ref).norm() / ref.norm()).item() <= 1e-2
