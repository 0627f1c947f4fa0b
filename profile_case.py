"""Runs one quantized-linear shape a few times on distinct layer instances -- a small,
self-terminating workload to put under a profiler (ncu) or to time one kernel:

    python profile_case.py --K 2048 --N 6144 --M 16 --kernel small_mma --instances 64
    python profile_case.py --K 2048 --N 6144 --M 1024 --kernel large --instances 8 --time
    python profile_case.py --K 2048 --N 6144 --M 300 --d 4 --C 1024 --G 64 --instances 24

    SACQ_NVCC_EXTRA=-DSACQ_TRACE python -m sacq_b200.build --force    # profiling build with in-kernel timestamps
    python profile_case.py --K 2048 --N 6144 --M 16 --kernel small_mma --instances 64 --trace

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
    ap.add_argument("--op", default="linear", choices=["linear", "forward", "dequant", "quant", "w8a8"])
    ap.add_argument("--instances", type=int, default=8)
    ap.add_argument("--passes", type=int, default=1)
    ap.add_argument("--time", action="store_true", help="print the mean time per call (CUDA events)")
    ap.add_argument("--graph", action="store_true", help="run the calls as one CUDA graph replay instead of eager launches")
    ap.add_argument("--timeline", action="store_true",
                    help="print entry / dependency / ready / exit times of the kernels of the last pass "
                         "(needs a library built with -DSACQ_TRACE)")
    ap.add_argument("--trace", action="store_true",
                    help="print the in-kernel phase timestamps of the last launch (needs a library built with -DSACQ_TRACE)")
    a = ap.parse_args()
    payload = make_payload(a.N, a.K, vector_dim=a.d, codebook_size=a.C, group_size=a.G or None, seed=1, device="cuda",
                           iters=1, fit=a.C <= 4096)
    layers = [PrecomputedPackedVectorCodebookLinear(payload, None, "cuda") for _ in range(a.instances)]
    for layer in layers:
        layer.set_kernel(a.kernel)
    x = make_activations(a.M, a.K).cuda()
    q, s = layers[0].quantize_activations(x)

    if a.op == "w8a8":                                 # the INT8 recipe: weight decode + integer GEMM per call
        from sacq_b200 import quantize_rows
        q8, s8 = quantize_rows(x, "int8_symmetric")
        sw8 = layers[0].weight_row_scale("int8_symmetric")

    def call(layer):
        if a.op == "w8a8":
            return layer.linear_w8a8_int8(q8, s8, sw8)
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
    if a.graph:
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for layer in layers:
                out = call(layer)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for layer in layers:
                out = call(layer)
        with torch.cuda.stream(stream):
            graph.replay()
            stream.synchronize()
            if a.timeline:
                read_timeline(reset_only=True)
            e0.record(stream)
            for _ in range(a.passes):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
    else:
        if a.timeline:
            read_timeline(reset_only=True)
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
    if a.trace:
        print_trace(layers[0], a)
    if a.timeline:
        print(f"per call: {us:.2f} us")
        for kind, t_entry, t_dep, t_ready, t_exit in read_timeline()[20:32]:
            print(f"  {kind:5s} entry {t_entry:8d}  predecessor seen finished {t_dep:8d}  operands landed {t_ready:8d}  exit {t_exit:8d}")


def read_timeline(reset_only=False):
    """Merged kernel timeline of a -DSACQ_TRACE build: (kind, entry, dependency, ready, exit) in ns
    from the first entry, ordered by entry time."""
    import ctypes
    lib = ctypes.CDLL(os.path.join(ROOT, "sacq_b200", "libsacq_b200.so"))
    rows = []
    for name, kind in (("sacq_debug_timeline_quant", "quant"), ("sacq_debug_timeline_gemm", "gemm")):
        if not hasattr(lib, name):
            continue
        buf = (ctypes.c_longlong * (512 * 8))()
        n = getattr(lib, name)(None if reset_only else buf, 1)
        if not reset_only:
            for i in range(min(n, 512)):
                rows.append((kind,) + tuple(buf[8 * i + 1: 8 * i + 5]))
    if not rows:
        return []
    rows.sort(key=lambda r: r[1])
    t0 = rows[0][1]
    return [(k, e - t0, d - t0, (r - t0) if r else 0, x - t0) for k, e, d, r, x in rows]


def print_trace(layer, a):
    """Phase breakdown of CTA 0 of the last launch, from %globaltimer stamps (ns) that only a
    -DSACQ_TRACE build of the library records."""
    import ctypes
    lib = ctypes.CDLL(os.path.join(ROOT, "sacq_b200", "libsacq_b200.so"))
    kern = layer.kernel_for(a.M)
    if kern == "small" and hasattr(lib, "sacq_debug_small_trace"):
        buf = (ctypes.c_longlong * 96)()
        lib.sacq_debug_small_trace(buf)
        t = list(buf)
        t0 = t[0]
        print(f"staged small-M kernel, CTA 0 (ns from kernel entry): barriers+copies issued {t[1]-t0}, "
              f"predecessor done {t[2]-t0}, codebook landed {t[3]-t0}, activations landed {t[4]-t0}, exit {t[5]-t0}")
        it = 0
        while 8 + 6 * it + 5 < 96 and t[8 + 6 * it] >= t0 and t[8 + 6 * it] <= t[5]:
            b = 8 + 6 * it
            print(f"  tile {it}: index rows landed {t[b]-t0}, CTA in step {t[b+1]-t0}, gathers+MMAs done {t[b+2]-t0}, "
                  f"partials exchanged {t[b+3]-t0}, reduced+stored {t[b+4]-t0}, tile closed {t[b+5]-t0}")
            it += 1
    elif kern == "large_tmem" and hasattr(lib, "sacq_debug_tmem_trace"):
        buf = (ctypes.c_longlong * (8 * 72))()
        lib.sacq_debug_tmem_trace(buf)
        t = [list(buf)[i * 72:(i + 1) * 72] for i in range(8)]
        t0, nk = t[0][0], a.K // 128
        print(f"TMEM-weight kernel, CTA (0,0) (ns from the end of the prologue): accumulator complete {t[0][3]-t0}, exit {t[0][4]-t0}")
        print("  expander: weight stage free   ", [v - t0 for v in t[2][8:8 + nk]])
        print("  expander: weight stage written", [v - t0 for v in t[5][8:8 + nk]])
        print("  issuer: operands ready        ", [v - t0 for v in t[1][8:8 + nk]])
    else:
        print("no trace: the library was not built with -DSACQ_TRACE, or this kernel records none")


if __name__ == "__main__":
    main()
