"""Runs one quantized-linear shape a few times on distinct layer instances -- a small,
self-terminating workload to put under a profiler (ncu) or to time one kernel:

    python profile_case.py --K 2048 --N 6144 --M 16 --kernel small_mma --instances 64
    python profile_case.py --K 2048 --N 6144 --M 1024 --kernel large --instances 8 --time
    python profile_case.py --K 2048 --N 6144 --M 300 --d 4 --C 1024 --G 64 --instances 24

Each instance owns its packed indices, so with enough instances (> 126 MB in total) every
launch reads its weights from HBM, not from L2.  ``--op`` selects the entry point:
``linear`` (GEMM on pre-quantized activations), ``forward`` (quantizer + GEMM),
``dequant`` or ``quant``.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from sacq_b200 import PrecomputedPackedVectorCodebookLinear  # noqa: E402
from sacq_b200.synthetic import algorithmic_bytes, make_activations, make_payload  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--N", type=int, default=2048)
    ap.add_argument("--M", type=int, default=16)
    ap.add_argument("--d", type=int, default=8)
    ap.add_argument("--C", type=int, default=4096)
    ap.add_argument("--G", type=int, default=0, help="scale group size (0 = one scale per output row)")
    ap.add_argument("--kernel", default="auto")
    ap.add_argument("--op", default="linear", choices=["linear", "forward", "dequant", "quant"])
    ap.add_argument("--instances", type=int, default=8)
    ap.add_argument("--passes", type=int, default=1)
    ap.add_argument("--time", action="store_true", help="print the mean time per call (CUDA events)")
    a = ap.parse_args()
    payload = make_payload(a.N, a.K, vector_dim=a.d, codebook_size=a.C, group_size=a.G or None, seed=1, device="cuda",
                           iters=1, fit=a.C <= 4096)
    layers = [PrecomputedPackedVectorCodebookLinear(payload, None, "cuda") for _ in range(a.instances)]
    for layer in layers:
        layer.set_kernel(a.kernel)
    x = make_activations(a.M, a.K).cuda()
    q, s = layers[0].quantize_activations(x)

    def call(layer):
        if a.op == "linear":
            return layer.linear_a8(q, s)
        if a.op == "forward":
            return layer(x)
        if a.op == "dequant":
            return layer.dequantize_weight()
        return layer.quantize_activations(x)[0]

    for layer in layers[:2]:
        call(layer)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.passes):
        for layer in layers:
            out = call(layer)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.passes * len(layers))
    msg = f"ok op={a.op} kernel={layers[0].kernel_for(a.M)} K={a.K} N={a.N} M={a.M} checksum={float(out.float().abs().mean()):.6f}"
    if a.time:
        ab = algorithmic_bytes(a.N, a.K, a.M, vector_dim=a.d, codebook_size=a.C, group_size=a.G or None)
        msg += f" us_per_call={us:.2f} (eager launches) algorithmic_GBps={ab / us / 1e3:.1f} TFLOPs={2.0 * a.M * a.N * a.K / us / 1e6:.1f}"
    print(msg)


if __name__ == "__main__":
    main()
