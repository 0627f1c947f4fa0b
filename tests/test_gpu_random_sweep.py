"""Seeded random sweep over layer geometries, token counts and kernel variants: every variant
that accepts a case must stay within the GEMM tolerance of the dense product of the library's
own bit-exact reconstruction, be deterministic, add a residual with the bytes of a separate
addition, and a shared launch of two layers must equal two separate launches."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

KERNELS = ("auto", "small", "small_simt", "small_mma_unpacked", "large", "large_grouped", "large_tmem", "large_tmem_grouped")


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_geometries(seed):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, linear_a8_multi, quantize_rows
    from sacq_b200.synthetic import make_activations, make_payload
    rng = random.Random(seed)
    checked = 0
    for it in range(40):
        d = rng.choice([4, 8])
        C = rng.choice([3, 16, 32, 64, 81, 128, 251, 256, 512, 1000, 1024, 2048, 3000, 4096])
        K = rng.choice([256, 512, 768, 1024, 1536, 2048, 3072])
        G = rng.choice([None, None, 64, 128, 256])
        if G is not None and K % G:
            G = None
        N = rng.choice([1, 7, 8, 24, 40, 64, 100, 101, 128, 136, 256, 333, 520, 1000, 1024, 1536, 2048, 3072])
        M = rng.choice([1, 2, 3, 5, 8, 16, 17, 31, 33, 48, 49, 64, 65, 96, 127, 128, 129, 200, 256, 300, 513])
        p = make_payload(N, K, vector_dim=d, codebook_size=C, group_size=G, seed=100 * seed + it, device="cuda", iters=1,
                         fit=False)
        p["shift"] = torch.tensor(rng.choice([0.0, 0.0, 0.00390625]), dtype=torch.bfloat16)
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(it)) * 0.05).to(torch.bfloat16) \
            if rng.random() < 0.5 else None
        mod = PrecomputedPackedVectorCodebookLinear(p, bias, "cuda")
        q, s = quantize_rows(make_activations(M, K, seed=it).cuda())
        ref = (q.float() @ mod.dequantize_weight().float().t()) * s
        if bias is not None:
            ref = ref + bias.cuda().float()
        res = (torch.randn(M, N, generator=torch.Generator().manual_seed(it + 1)) * 0.3).to(torch.bfloat16).cuda()
        case = (seed, it, N, K, d, C, G, M)
        for kern in KERNELS:
            mod.set_kernel(kern)
            try:
                y = mod.linear_a8(q, s)
            except Exception as e:
                if getattr(e, "code", 0) == -2:
                    continue                        # this variant does not take the geometry
                raise
            err = float((y.float() - ref).norm() / ref.norm().clamp_min(1e-20))
            assert err <= 1e-2, (case, kern, err)
            assert torch.equal(y, mod.linear_a8(q, s)), (case, kern)
            assert torch.equal(mod.linear_a8(q, s, residual=res), y + res), (case, kern)
            checked += 1
        mod.set_kernel("auto")
        assert mod.device_status() == 0, case
        if it % 3 == 0:
            p2 = make_payload(max(8, N // 2 // 8 * 8), K, vector_dim=d, codebook_size=C, group_size=G,
                              seed=100 * seed + it + 50, device="cuda", iters=1, fit=False)
            p2["shift"] = p["shift"]
            mod2 = PrecomputedPackedVectorCodebookLinear(p2, None, "cuda")
            a, b = linear_a8_multi([mod, mod2], q, s)
            assert torch.equal(a, mod.linear_a8(q, s)) and torch.equal(b, mod2.linear_a8(q, s)), case
    assert checked > 100
