"""Benchmark of the W1.5A8 quantized-linear path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sections a,b,...]

HEADLINE workload (`config.workload = "decode_sweep"`): the decode-shape sweep of
Qwen3-1.7B-shaped decoder linears at W1.5A8 (dim-8 vectors, 4096-entry codebook, per-channel
scales): shapes K x N = 2048x2048 (q), 2048x1024 (kv), 2048x2048 (o), 2048x6144 (gate/up),
6144x2048 (down), each at M in {1,2,4,8,16,32,64}.  One STEP = one pass over all 35
(shape, M) layer calls, every call on its own layer instance; consecutive steps rotate through
enough replica sets that the touched weights exceed the 126 MB L2 before anything repeats.
Weights are N(0, 0.02) fitted with a seeded k-means, activations N(0,1) with 1 % outlier
channels x20.  The timed pass of K steps is repeated (at least 9 times, at least 0.6 s in
total) and the median pass is reported.

Reported on the one JSON line: metric = microseconds per layer call (whole job: elapsed /
(35 * ranks * steps)); `value` with inputs resident in HBM (CUDA-graph replay of quantizer +
GEMM kernels); `e2e` through the module's forward with host buffers (pinned H2D of the
activations and D2H of the result inside the timed region); `roofline` for the dominant kernel
(small-M GEMM; algorithmic bytes / its mean launch time measured with CUDA events on a graph
that holds only that kernel); `cpu_baseline` = the reference's CPU path (PyTorch ops, all host
threads) on the same sweep, with the C restatement of the same arithmetic (all threads and one
thread) beside it as `cpu_baseline.c_restatement`.  Further objects carry the rest of the metric, each timed with CUDA
events over graph replays that rotate through more than two L2 sizes of distinct operands:

  `large_m`      batched sweep: 2048x6144 and 6144x2048 at M in {256, 1024, 4096, 8192}; us,
                 algorithmic TFLOP/s, fraction of the measured dense-bf16 tensor peak, and beside
                 it `dense_baseline_us` = this library's reconstruction kernel followed by a
                 dense bf16 `torch.matmul` on the same inputs (a stated secondary baseline; it is
                 never on the product path);
  `config0`      the single 2048x2048 layer at M in {1, 4, 16};
  `mixed_bits`   2048x6144 at 1 / 1.5 / 2 / 3 bits per weight, M in {1, 16, 256};
  `policy`       the synthetic GR00T-shaped policy forward: one CUDA-graph launch per query,
                 5 warm-up + 20 measured queries, median (the protocol of the reference's timing
                 worker, gr00t_libero/acceleration/reference/final_worker.py:155-163), batch 1
                 latency and batched forwards/s;
  `column_split` (N > 1 only) the output-split layer over the N ranks: result equal to the
                 one-GPU result (checked on every rank), us for the NCCL all-gather and for the
                 exchange inside the GEMM epilogue, bytes per rank, NVLink GB/s per direction.

`--impl reference` times the CPU path alone, on every rank under torchrun with the host
threads divided between the ranks (the same weak-scaling semantics as the GPU arm).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from sacq_b200.synthetic import DECODE_MS, DECODE_SHAPES, algorithmic_bytes, make_activations, make_payload  # noqa: E402

METRIC = "w1p5a8_codebook_gemm_us_per_layer"
UNIT = "us/layer"
L2_BYTES = 126 * 1024 * 1024
DRAM_TRAFFIC_RATIO = 2.500096 / 2.666560      # ncu dram bytes / algorithmic bytes, small-M GEMM
ALL_SECTIONS = ("large_m", "config0", "mixed_bits", "policy", "column_split")
MIN_TIMED_SECONDS = 0.6
MIN_PASSES = 9


def sweep_calls():
    return [(name, K, N, M) for (name, K, N) in DECODE_SHAPES for M in DECODE_MS]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_mhz_min": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def workload_config(n_gpus):
    return {"workload": "decode_sweep", "shapes_KxN": [f"{K}x{N}" for _, K, N in DECODE_SHAPES],
            "M": list(DECODE_MS), "vector_dim": 8, "codebook_size": 4096, "index_bits": 12,
            "scales": "per-output-channel bf16", "activations": "fp8 e4m3 per-token",
            "calls_per_step": len(sweep_calls()), "parallelism": f"dp{n_gpus} (independent layer calls per rank)",
            "l2": "distinct layer instances rotate between steps, more than 2x the 126 MB L2 (GPU arm); not "
                  "applicable on the CPU arm"}


# --------------------------------------------------------------------------- CPU reference arm

def cpu_sweep_payloads():
    """One payload per shape on the CPU (random indices: the CPU path's cost does not depend
    on which codewords are hit, and fitting 6144-wide layers on the host would dominate)."""
    out = {}
    for i, (name, K, N) in enumerate(DECODE_SHAPES):
        out[name] = make_payload(N, K, seed=i, fit=False)
    return out


def run_cpu_reference(steps: int, warmup: int):
    from oracle import torch_port
    payloads = cpu_sweep_payloads()
    xs = {(name, M): make_activations(M, K, seed=M) for (name, K, N, M) in sweep_calls()}
    threads = torch.get_num_threads()

    def step():
        for name, K, N, M in sweep_calls():
            torch_port.forward(payloads[name], xs[(name, M)])

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return dt, threads


def run_c_restatement(passes: int):
    """The same sweep through the C restatement (oracle/sacq_oracle.c: unpack, two-rounding bf16
    reconstruction, per-row e4m3 quantizer, fp32 dot products; OpenMP over output rows): seconds
    per pass with all threads and with one, so that there is a CPU figure that does not depend
    on PyTorch's kernels."""
    import numpy as np
    from oracle import build_oracle as C

    def bits(t):
        return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)

    layers = {}
    for name, p in cpu_sweep_payloads().items():
        N, K = int(p["out_features"]), int(p["in_features"])
        layers[name] = (p["packed_indices"].numpy(), int(p["index_bits"]), bits(p["codebook"]),
                        bits(p["scales"]).reshape(N, -1), int(bits(p["shift"].reshape(1))[0]), None, N, K,
                        int(p["group_size"]))
    xs = {(name, M): bits(make_activations(M, K, seed=M)) for (name, K, N, M) in sweep_calls()}

    def one_pass():
        t0 = time.perf_counter()
        for name, K, N, M in sweep_calls():
            q, s = C.quant_rows(xs[(name, M)])
            C.linear(*layers[name], q, s)
        return time.perf_counter() - t0

    all_threads = C.threads()
    one_pass()
    t_all = min(one_pass() for _ in range(passes))
    C.set_threads(1)
    try:
        t_one = one_pass()
    finally:
        C.set_threads(all_threads)
    return t_all, all_threads, t_one


def reference_main(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
        dist.init_process_group("gloo")
    dt, threads = run_cpu_reference(args.steps, args.warmup)
    if dist is not None:
        t = torch.tensor([dt], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    if rank == 0:
        calls = len(sweep_calls())
        us_per_layer = dt / (args.steps * calls * world) * 1e6
        line = {
            "impl": "reference", "metric": METRIC, "value": us_per_layer, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {"value": us_per_layer, "unit": UNIT, "cores": threads * world, "kind": "port",
                             "sample": f"full 35-call sweep per step on each of {world} rank(s) with {threads} "
                                       f"thread(s) each, {args.steps} steps after {args.warmup} warm-up; PyTorch CPU "
                                       "ops as the reference runs them (unpack, bf16 gather/mul/add, fp32 matmul)"},
            "e2e": {"value": us_per_layer, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "tokens_per_s": sum(M for *_, M in sweep_calls()) * world / (dt / args.steps),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- GPU arm helpers

class Ctx:
    """What every section of the GPU arm shares."""

    def __init__(self, args):
        import torch.distributed as dist
        from sacq_b200 import _lib
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device (no CPU fallback); use --impl reference for the CPU arm")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.lib = _lib.load()
        self._lib_mod = _lib
        self.stream = torch.cuda.Stream(device=self.dev)
        self.peaks = load_peaks()

    def check(self, rc):
        self._lib_mod.check(rc)

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, values):
        if self.dist is None:
            return [float(v) for v in values]
        t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    def capture(self, fn):
        """One CUDA graph of fn(stream); returns (graph, kernels of this library launched inside)."""
        g = torch.cuda.CUDAGraph()
        before = self.lib.sacq_launch_count()
        with torch.cuda.graph(g, stream=self.stream):
            fn(torch.cuda.current_stream())
        return g, self.lib.sacq_launch_count() - before

    def time_graphs(self, graphs, replays_per_pass, warmup, min_seconds=MIN_TIMED_SECONDS, min_passes=MIN_PASSES,
                    max_passes=2000):
        """Median seconds of one pass (= `replays_per_pass` replays rotating through `graphs`),
        CUDA events on the launching stream, barrier + synchronize on both sides of every pass."""
        times, k = [], 0

        def one_pass():
            nonlocal k
            self.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(replays_per_pass):
                graphs[k % len(graphs)].replay()
                k += 1
            e1.record(self.stream)
            self.stream.synchronize()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 1e3)

        with torch.cuda.stream(self.stream):
            for i in range(warmup):
                graphs[i % len(graphs)].replay()
            self.stream.synchronize()
            for _ in range(min_passes):
                one_pass()
            # every rank runs the same number of further passes (each pass holds a barrier): the
            # largest any rank needs to reach min_seconds of timed work
            total = sum(times)
            more = 0
            if total < min_seconds:
                more = min(max_passes - min_passes, int((min_seconds - total) / max(total / len(times), 1e-7)) + 1)
            more = int(self.max_over_ranks([more])[0])
            for _ in range(more):
                one_pass()
        self.barrier()
        return statistics.median(times), len(times)


def rotating_sets(bytes_per_set, lo=2, hi=400):
    return max(lo, min(hi, -(-int(2.2 * L2_BYTES) // max(1, int(bytes_per_set)))))


def time_layer_calls(ctx, payload, M, n_sets, bias=None, kernel=None, reps_target=0.25):
    """us per `sacq_linear_a8` call (GEMM alone, quantized activations resident) on `n_sets`
    distinct (layer instance, activations, output) sets replayed as one CUDA graph."""
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    K, N = int(payload["in_features"]), int(payload["out_features"])
    mods = [PrecomputedPackedVectorCodebookLinear(payload, bias, str(ctx.dev)) for _ in range(n_sets)]
    if kernel is not None:
        for m in mods:
            m.set_kernel(kernel)
    n_act = max(1, min(n_sets, -(-int(2.2 * L2_BYTES) // max(1, M * K + 2 * M * N))))
    qs, ss, ys = [], [], []
    for i in range(n_act):
        q, s = quantize_rows(make_activations(M, K, seed=M + i).to(ctx.dev))
        qs.append(q)
        ss.append(s.reshape(-1).contiguous())
        ys.append(torch.empty(M, N, dtype=torch.bfloat16, device=ctx.dev))
    ws = torch.zeros(max(int(ctx.lib.sacq_workspace_bytes(mods[0]._handle, M)), 1 << 16), dtype=torch.uint8,
                     device=ctx.dev)

    def enqueue(s):
        for i, m in enumerate(mods):
            j = i % n_act
            ctx.check(ctx.lib.sacq_linear_a8(m._handle, qs[j].data_ptr(), ss[j].data_ptr(), M, ys[j].data_ptr(), N,
                                             ws.data_ptr(), ws.numel(), s.cuda_stream))

    with torch.cuda.stream(ctx.stream):
        enqueue(ctx.stream)
    ctx.stream.synchronize()
    graph, launches = ctx.capture(enqueue)
    sec, passes = ctx.time_graphs([graph], 1, 3, min_seconds=reps_target, min_passes=5)
    sec = ctx.max_over_ranks([sec])[0]
    kern = mods[0].kernel_for(M)
    del graph
    return sec / n_sets * 1e6, kern, launches / n_sets


# --------------------------------------------------------------------------- sections

def section_large_m(ctx):
    """BASELINE config 4, single GPU part: the batched sweep on the tensor-core kernels."""
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear, quantize_rows
    rows = []
    peak = ctx.peaks["bf16_tflops"]
    for K, N in ((2048, 6144), (6144, 2048)):
        payload = make_payload(N, K, seed=K // 7 + N, device=ctx.dev, iters=1)
        for M in (256, 1024, 4096, 8192):
            per_set = N * (K // 8) * 12 // 8 + M * K + 2 * M * N
            n_sets = rotating_sets(per_set, lo=2, hi=64)
            us, kern, _ = time_layer_calls(ctx, payload, M, n_sets)
            flops = 2.0 * M * N * K
            # secondary baseline: materialise the bf16 weight with this library's reconstruction
            # kernel, then a dense bf16 GEMM of the framework on bf16 activations
            mod = PrecomputedPackedVectorCodebookLinear(payload, None, str(ctx.dev))
            x = make_activations(M, K, seed=M).to(ctx.dev)
            q, s = quantize_rows(x)
            xq = (q.float() * s).to(torch.bfloat16)               # the same quantized activations, as bf16
            y = torch.empty(M, N, dtype=torch.bfloat16, device=ctx.dev)

            def dense(stream):
                w = mod.dequantize_weight()
                torch.matmul(xq, w.t(), out=y)

            with torch.cuda.stream(ctx.stream):
                dense(ctx.stream)
            ctx.stream.synchronize()
            g, _ = ctx.capture(dense)
            sec, _ = ctx.time_graphs([g], 4, 3, min_seconds=0.1, min_passes=5)
            dense_us = ctx.max_over_ranks([sec])[0] / 4 * 1e6
            del g
            # the reference's deployed INT8 recipe on the same layer: int8 weight rows decoded per
            # call + tcgen05 kind::i8 GEMM (another numerical recipe: weights re-quantized per row)
            q8, s8 = quantize_rows(x, "int8_symmetric")
            sw8 = mod.weight_row_scale("int8_symmetric")

            def int8_recipe(stream):
                mod.linear_w8a8_int8(q8, s8, sw8, out=y)

            with torch.cuda.stream(ctx.stream):
                int8_recipe(ctx.stream)
            ctx.stream.synchronize()
            g, _ = ctx.capture(int8_recipe)
            sec, _ = ctx.time_graphs([g], 4, 3, min_seconds=0.1, min_passes=5)
            int8_us = ctx.max_over_ranks([sec])[0] / 4 * 1e6
            del g
            # ... and its FP8 recipe (per-row e4m3 weights decoded per call + tcgen05 kind::f8f6f4 GEMM)
            qf, sf = quantize_rows(x)
            swf = mod.weight_row_scale("fp8_e4m3fn")

            def fp8_recipe(stream):
                mod.linear_w8a8_fp8(qf, sf, swf, out=y)

            with torch.cuda.stream(ctx.stream):
                fp8_recipe(ctx.stream)
            ctx.stream.synchronize()
            g, _ = ctx.capture(fp8_recipe)
            sec, _ = ctx.time_graphs([g], 4, 3, min_seconds=0.1, min_passes=5)
            fp8_us = ctx.max_over_ranks([sec])[0] / 4 * 1e6
            del g
            rows.append({"shape_KxN": f"{K}x{N}", "M": M, "us": us, "kernel": kern,
                         "algorithmic_tflops": flops / us / 1e6, "tokens_per_s": M / us * 1e6,
                         "frac_of_bf16_peak": flops / us / 1e6 / peak, "dense_baseline_us": dense_us,
                         "int8_recipe_us": int8_us, "int8_recipe_tops": flops / int8_us / 1e6,
                         "fp8_recipe_us": fp8_us,
                         "rotating_sets": n_sets})
    best = max(rows, key=lambda r: r["M"] * 10 + (r["shape_KxN"] == "2048x6144"))
    return {"rows": rows,
            "roofline": {"bound": "tensor", "kernel": "large_m_tmem_kernel / large_m_kernel (tcgen05 kind::f8f6f4)",
                         "achieved": best["algorithmic_tflops"], "peak": peak, "peak_kind": ctx.peaks["kind"],
                         "unit": "TFLOP/s", "frac": best["algorithmic_tflops"] / peak, "traffic": None,
                         "peak_sustained": ctx.peaks["bf16_tflops_sustained"],
                         "frac_of_sustained_peak": best["algorithmic_tflops"] / ctx.peaks["bf16_tflops_sustained"],
                         "timing_note": "rows are medians of back-to-back graph replays (sustained, under the power "
                                        "cap): `frac` divides by the burst peak all the same, "
                                        "`frac_of_sustained_peak` by the peak measured the way the rows are",
                         "at": {"shape_KxN": best["shape_KxN"], "M": best["M"]},
                         "peak_note": "algorithmic flops 2*M*N*K over the measured dense bf16 GEMM peak; the kernel "
                                      "executes twice the algorithmic flops in FP8 (high + low codeword halves), so "
                                      "the dense-bf16 rate is the equal-work ceiling"},
            "dense_baseline_note": "sacq_dequant_bf16 + torch.matmul (bf16) on the same quantized activations; a "
                                   "secondary baseline, never on the product path",
            "int8_recipe_note": "sacq_linear_w8a8_int8: the reference's deployed INT8 recipe (per-output-row int8 "
                                "weights decoded per call, int32 accumulation), one layer instance, GEMM side only"}


def section_config0(ctx):
    """BASELINE config 0 on the GPU: the single 2048x2048 layer at M in {1, 4, 16}."""
    payload = make_payload(2048, 2048, seed=0, device=ctx.dev)
    rows = []
    n_sets = rotating_sets(2048 * 256 * 12 // 8 + 4096 * 16, lo=2, hi=360)
    for M in (1, 4, 16):
        us, kern, _ = time_layer_calls(ctx, payload, M, n_sets)
        alg = algorithmic_bytes(2048, 2048, M)
        rows.append({"M": M, "us": us, "kernel": kern, "tokens_per_s": M / us * 1e6,
                     "algorithmic_gbs": alg / us / 1e3, "frac_of_hbm_peak": alg / us / 1e3 / ctx.peaks["hbm_gbs"],
                     "rotating_sets": n_sets})
    return {"shape_KxN": "2048x2048", "rows": rows}


def section_mixed_bits(ctx):
    """BASELINE config 2: one 2048x6144 layer per codebook geometry, M in {1, 16, 256}."""
    rows = []
    K, N = 2048, 6144
    for bpw, d, C in ((1.0, 8, 256), (1.5, 8, 4096), (2.0, 8, 65536), (3.0, 4, 4096)):
        bits = max(1, (C - 1).bit_length())
        payload = make_payload(N, K, vector_dim=d, codebook_size=C, seed=C + d, device=ctx.dev, iters=1,
                               sample_size=max(65536, 2 * C), fit=(C < 65536))
        n_sets = rotating_sets(N * (K // d) * bits // 8 + C * d * 4, lo=2, hi=200)
        for M in (1, 16, 256):
            us, kern, _ = time_layer_calls(ctx, payload, M, n_sets)
            alg = algorithmic_bytes(N, K, M, vector_dim=d, codebook_size=C)
            rows.append({"bits_per_weight": bpw, "vector_dim": d, "codebook_size": C, "M": M, "us": us,
                         "kernel": kern, "algorithmic_gbs": alg / us / 1e3,
                         "algorithmic_tflops": 2.0 * M * N * K / us / 1e6, "rotating_sets": n_sets})
    return {"shape_KxN": f"{K}x{N}", "rows": rows}


def section_policy(ctx):
    """BASELINE config 3 (+ the batched half of config 4): the synthetic policy forward."""
    from sacq_b200.policy import SyntheticGr00tPolicy
    policy = SyntheticGr00tPolicy(str(ctx.dev), seed=0)
    out = {"workload": "synthetic GR00T-N1.5-shaped policy, 4 denoising steps, all linears W1.5A8, one CUDA-graph "
                       "launch per query, 5 warm-up + 20 measured, median",
           "quantized_linears": policy.num_quantized_linears}
    for batch in (1, policy.BENCH_BATCH):
        image, noise = policy.example_inputs(42, batch=batch)
        with torch.cuda.stream(ctx.stream):
            for _ in range(2):
                ref = policy(image, noise)
        ctx.stream.synchronize()
        before = ctx.lib.sacq_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=ctx.stream):
            y = policy(image, noise)
        launches = ctx.lib.sacq_launch_count() - before
        times = []
        with torch.cuda.stream(ctx.stream):
            for i in range(5 + 20):
                if i == 5:
                    ctx.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(ctx.stream)
                graph.replay()
                e1.record(ctx.stream)
                ctx.stream.synchronize()
                if i >= 5:
                    times.append(e0.elapsed_time(e1))
        med = ctx.max_over_ranks([statistics.median(times)])[0]
        key = "batch1" if batch == 1 else f"batch{batch}"
        out[key] = {"ms_per_query" if batch == 1 else "ms_per_batch": med,
                    "forwards_per_s": ctx.world * batch * 1e3 / med,
                    "sacq_kernel_launches": int(launches), "deterministic": bool(torch.equal(y, ref))}
        del graph
    out["ms_per_query"] = out["batch1"]["ms_per_query"]
    out["forwards_per_s"] = max(v["forwards_per_s"] for k, v in out.items() if isinstance(v, dict))
    out["parallelism"] = f"dp{ctx.world}: independent queries per rank, no data-path collective"
    return out


def section_column_split(ctx):
    """BASELINE config 4, multi-GPU part: output rows split over the ranks, all-gather or the
    exchange inside the GEMM epilogue; every rank also computes the whole layer alone and
    checks that the split result has the same bytes."""
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    from sacq_b200.column_parallel import ColumnParallelCodebookLinear
    dist, world = ctx.dist, ctx.world
    rows, all_equal = [], True
    ms = (1024, 8192)
    for K, N in ((2048, 6144), (6144, 2048)):
        # ONE payload for all ranks: the k-means fit runs on the GPU with atomics, so two ranks fitting
        # "the same" layer can differ in an index or a scale; rank 0 fits, everyone receives its bytes
        box = [None]
        if ctx.rank == 0:
            made = make_payload(N, K, seed=1, iters=1, device=ctx.dev)
            box[0] = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in made.items()}
        dist.broadcast_object_list(box, src=0)
        payload = box[0]
        bias = (torch.randn(N, generator=torch.Generator().manual_seed(6)) * 0.05).to(torch.bfloat16)
        whole = PrecomputedPackedVectorCodebookLinear(payload, bias, str(ctx.dev))
        gathered = ColumnParallelCodebookLinear(payload, bias, str(ctx.dev))
        fused = ColumnParallelCodebookLinear(payload, bias, str(ctx.dev), fused_exchange=True, max_tokens=max(ms))
        for M in ms:
            x = make_activations(M, K, seed=M).to(ctx.dev)
            y_one = whole(x)
            eq_g = bool(torch.equal(gathered(x), y_one))
            eq_f = bool(torch.equal(fused(x), y_one))
            torch.cuda.synchronize()
            flags = ctx.max_over_ranks([0.0 if eq_g else 1.0, 0.0 if eq_f else 1.0])
            eq_g, eq_f = flags[0] == 0.0, flags[1] == 0.0
            all_equal = all_equal and eq_g and eq_f
            times = {}
            for name, layer in (("allgather", gathered), ("fused_exchange", fused)):
                with torch.cuda.stream(ctx.stream):
                    for _ in range(2):
                        layer(x)
                ctx.stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=ctx.stream):
                    layer(x)
                    layer(x)                            # two calls: the fused variant alternates its two buffers
                sec, _ = ctx.time_graphs([g], 2, 3, min_seconds=0.1, min_passes=5)
                times[name] = ctx.max_over_ranks([sec])[0] / 4 * 1e6
                del g
            with torch.cuda.stream(ctx.stream):
                for _ in range(2):
                    whole(x)
            ctx.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=ctx.stream):
                whole(x)
                whole(x)
            sec, _ = ctx.time_graphs([g], 2, 3, min_seconds=0.1, min_passes=5)
            one_gpu_us = ctx.max_over_ranks([sec])[0] / 4 * 1e6
            del g
            sent = (world - 1) * M * (N // world) * 2          # bytes each rank pushes to (and takes from) its peers
            rows.append({"shape_KxN": f"{K}x{N}", "M": M, "one_gpu_us": one_gpu_us,
                         "allgather_us": times["allgather"], "fused_exchange_us": times["fused_exchange"],
                         "equal_to_one_gpu": {"allgather": eq_g, "fused_exchange": eq_f},
                         "bytes_sent_per_rank": sent,
                         "nvlink_gbs_per_direction_fused": sent / times["fused_exchange"] / 1e3,
                         "speedup_vs_one_gpu_fused": one_gpu_us / times["fused_exchange"]})
        fused.close()
    return {"ranks": world, "rows": rows, "parity": all_equal,
            "note": "quantizer + GEMM + exchange per call, CUDA-graph replays, max over ranks; every rank receives "
                    "(ranks-1)/ranks of the M x N bf16 result over NVLink, which bounds the call from below"}


# --------------------------------------------------------------------------- GPU arm

def gpu_main(args):
    from sacq_b200 import PrecomputedPackedVectorCodebookLinear
    ctx = Ctx(args)
    dev, lib, world, rank = ctx.dev, ctx.lib, ctx.world, ctx.rank
    calls = sweep_calls()
    sections = [s for s in args.sections.split(",") if s]
    sampler = ClockSampler(ctx.local)
    if rank == 0:
        sampler.start()                      # samples through every timed region below

    # ---- layers: one fitted payload per shape, one device instance per (call, replica set)
    per_set_bytes = sum(N * (K // 8) * 12 // 8 + 4096 * 16 + N * 2 for _, K, N, _ in calls)
    n_sets = max(2, -(-int(2.2 * L2_BYTES) // per_set_bytes))
    payloads = {name: make_payload(N, K, seed=i, device=dev, iters=1) for i, (name, K, N) in enumerate(DECODE_SHAPES)}
    sets = []
    for _ in range(n_sets):
        sets.append([PrecomputedPackedVectorCodebookLinear(payloads[name], None, str(dev)) for name, K, N, M in calls])
    x_host = [make_activations(M, K, seed=M).pin_memory() for name, K, N, M in calls]
    x_dev = [x.to(dev) for x in x_host]
    y_dev = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for name, K, N, M in calls]
    y_host = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for name, K, N, M in calls]
    q_dev = [torch.empty(M, K, dtype=torch.uint8, device=dev) for name, K, N, M in calls]
    s_dev = [torch.empty(M, dtype=torch.float32, device=dev) for name, K, N, M in calls]
    ws_bytes = max(int(lib.sacq_workspace_bytes(m._handle, M)) for m, (_, _, _, M) in zip(sets[0], calls))
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)

    def enqueue_full(layer_set, s):
        for i, (mod, (name, K, N, M)) in enumerate(zip(layer_set, calls)):
            ctx.check(lib.sacq_linear_bf16(mod._handle, x_dev[i].data_ptr(), K, M, q_dev[i].data_ptr(),
                                           s_dev[i].data_ptr(), y_dev[i].data_ptr(), N, ws.data_ptr(), ws.numel(),
                                           s.cuda_stream))

    def enqueue_gemm_only(layer_set, s):
        for i, (mod, (name, K, N, M)) in enumerate(zip(layer_set, calls)):
            ctx.check(lib.sacq_linear_a8(mod._handle, q_dev[i].data_ptr(), s_dev[i].data_ptr(), M,
                                         y_dev[i].data_ptr(), N, ws.data_ptr(), ws.numel(), s.cuda_stream))

    with torch.cuda.stream(ctx.stream):
        enqueue_full(sets[0], ctx.stream)          # eager warm-up: module loading, attribute setting
    ctx.stream.synchronize()
    full_graphs, gemm_graphs, full_launches, gemm_launches = [], [], 0, 0
    for layer_set in sets:
        g, full_launches = ctx.capture(lambda s, ls=layer_set: enqueue_full(ls, s))
        full_graphs.append(g)
        g, gemm_launches = ctx.capture(lambda s, ls=layer_set: enqueue_gemm_only(ls, s))
        gemm_graphs.append(g)

    sec, passes = ctx.time_graphs(full_graphs, args.steps, args.warmup)
    sec_gemm, _ = ctx.time_graphs(gemm_graphs, args.steps, args.warmup)

    # ---- end to end through the module's forward with host buffers
    def e2e_step(layer_set):
        # host activations in, host results out: the module's host-buffer forward copies x to
        # the device, runs quantizer + GEMM and copies y back, all on the current stream
        for i, mod in enumerate(layer_set):
            mod.forward_host(x_host[i], y_host[i])
        torch.cuda.current_stream().synchronize()

    for i in range(max(3, args.warmup)):
        e2e_step(sets[i % n_sets])
    e2e_times, k = [], 0

    def e2e_pass():
        nonlocal k
        torch.cuda.synchronize()
        ctx.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step(sets[k % n_sets])
            k += 1
        torch.cuda.synchronize()
        e2e_times.append(time.perf_counter() - t0)

    for _ in range(MIN_PASSES):
        e2e_pass()
    total = sum(e2e_times)
    more = 0 if total >= MIN_TIMED_SECONDS else int((MIN_TIMED_SECONDS - total) / (total / len(e2e_times))) + 1
    for _ in range(int(ctx.max_over_ranks([min(more, 2000)])[0])):      # the same count on every rank: each pass holds a barrier
        e2e_pass()
    sec_e2e = statistics.median(e2e_times)
    sec, sec_gemm, sec_e2e = ctx.max_over_ranks([sec, sec_gemm, sec_e2e])

    extra = {}
    for name, fn in (("large_m", section_large_m), ("config0", section_config0), ("mixed_bits", section_mixed_bits),
                     ("policy", section_policy), ("column_split", section_column_split)):
        if name not in sections or (name == "column_split" and world == 1):
            continue
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        extra[name] = fn(ctx)
        extra[name]["section_seconds"] = round(time.perf_counter() - t0, 1)
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        n_calls = len(calls)
        us_layer = sec / args.steps / (n_calls * world) * 1e6
        us_layer_e2e = sec_e2e / args.steps / (n_calls * world) * 1e6
        gemm_launch_s = sec_gemm / (args.steps * gemm_launches)
        alg = sum(algorithmic_bytes(N, K, M) for _, K, N, M in calls) / n_calls
        peak, peak_kind = ctx.peaks["hbm_gbs"], ctx.peaks["kind"]
        achieved = alg / gemm_launch_s / 1e9
        tokens = sum(M for *_, M in calls)
        line = {
            "metric": METRIC, "value": us_layer, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8 hi+lo codewords, fp32 accumulate",
            "data": "synthetic",
            "config": workload_config(world),
            "timed_passes": passes, "pass_statistic": "median",
            "replica_sets": f"{n_sets} x {per_set_bytes / 1e6:.1f} MB",
            "tokens_per_s": tokens * world / (sec / args.steps),
            "e2e": {"value": us_layer_e2e, "unit": UNIT,
                    "h2d_bytes_per_step": sum(M * K * 2 for _, K, N, M in calls),
                    "d2h_bytes_per_step": sum(M * N * 2 for _, K, N, M in calls),
                    "ms_per_step": sec_e2e / args.steps * 1e3},
            "gpu_launches": int(full_launches * args.steps),
            "roofline": {"bound": "hbm", "kernel": "small_m_mma_staged_kernel (packed-index GEMM; the M=64 calls of layers with N>=2048 run on the tensor-core kernel)",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": alg * DRAM_TRAFFIC_RATIO,
                         "traffic_note": "dram bytes read+written per launch = algorithmic bytes x 0.94, the ratio "
                                         "ncu measured on the K=2048 N=6144 M=16 launch "
                                         "(profiles/small_m_mma_staged_2048x6144_m16.md)",
                         "algorithmic_bytes_per_launch": alg, "us_per_launch": gemm_launch_s * 1e6,
                         "launches_timed": int(gemm_launches * args.steps)},
            "clocks": clocks,
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            cpu_steps = 3
            dt, threads = run_cpu_reference(cpu_steps, 1)
            line["cpu_baseline"] = {
                "value": dt / (cpu_steps * n_calls) * 1e6, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"the same 35-call sweep, {cpu_steps} passes after 1 warm-up, PyTorch CPU ops as the "
                          "reference runs them (random-index layers of the same shapes)"}
            try:
                t_all, c_threads, t_one = run_c_restatement(2)
                line["cpu_baseline"]["c_restatement"] = {
                    "value": t_all / n_calls * 1e6, "unit": UNIT, "cores": c_threads,
                    "value_one_thread": t_one / n_calls * 1e6,
                    "sample": "the same sweep through oracle/sacq_oracle.c (gcc -O3, OpenMP over output rows): best "
                              "of 2 passes with all threads, one pass with a single thread"}
            except (OSError, RuntimeError) as e:       # no compiler and no prebuilt oracle library on this host
                line["cpu_baseline"]["c_restatement"] = {"unavailable": str(e).splitlines()[0][:200]}
        print(json.dumps(line), flush=True)
    if ctx.dist is not None:
        ctx.dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sections", default=",".join(ALL_SECTIONS),
                    help="comma-separated subset of: " + ", ".join(ALL_SECTIONS) + " (empty: headline only)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        reference_main(args)
    else:
        gpu_main(args)


if __name__ == "__main__":
    main()
