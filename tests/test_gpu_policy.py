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
