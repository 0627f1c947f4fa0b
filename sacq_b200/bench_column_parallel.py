"""Batched-throughput sweep of the column-split quantized linear (run under torchrun):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        --master-port 29511 -m sacq_b200.bench_column_parallel [--ms 256,1024,4096,8192]

Layers 2048x6144 and 6144x2048 (K x N) at W1.5A8, output rows split over the G ranks,
result all-gathered over NVLink.  Prints one JSON line per (shape, M): GEMM-only time,
GEMM + all-gather time (max over ranks, CUDA events), tokens/s and algorithmic TFLOP/s.
With G = 1 it measures the single-GPU kernels.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .column_parallel import ColumnParallelCodebookLinear
from .synthetic import make_activations, make_payload


def _time(fn, reps, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) * 1e3       # microseconds


def _time_graph(fn, reps, dev):
    """Device time of fn() from CUDA-graph replays; the graph holds TWO calls (the fused
    exchange alternates between its two mapped result buffers)."""
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for _ in range(2):
            fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        fn()
        fn()
    with torch.cuda.stream(stream):
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / (2 * reps)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del graph
    return float(t.item()) * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", default="256,1024,4096,8192")
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--graph", action="store_true",
                    help="also time CUDA-graph replays of both exchange variants (device time without host launch work)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    for k, n in ((2048, 6144), (6144, 2048)):
        payload = make_payload(n, k, seed=1, iters=1, device=dev)
        for chunks in sorted({1, args.chunks}):
            layer = ColumnParallelCodebookLinear(payload, None, str(dev), chunks=chunks)
            fused = None
            if chunks == 1 and world > 1:
                fused = ColumnParallelCodebookLinear(payload, None, str(dev), fused_exchange=True,
                                                     max_tokens=max(int(v) for v in args.ms.split(",")))
            for m in [int(v) for v in args.ms.split(",")]:
                x = make_activations(m, k, seed=m).to(dev)
                q, s = layer.local.quantize_activations(x)
                t_gemm = _time(lambda: layer.local.linear_a8(q, s), args.reps, dev)
                t_full = _time(lambda: layer(x), args.reps, dev)
                t_fused = None
                if chunks == 1 and world > 1 and fused is not None:
                    t_fused = _time(lambda: fused(x), args.reps, dev)
                t_full_g = t_fused_g = None
                if args.graph and chunks == 1 and world > 1:
                    t_full_g = _time_graph(lambda: layer(x), args.reps, dev)
                    t_fused_g = _time_graph(lambda: fused(x), args.reps, dev)
                if rank == 0:
                    print(json.dumps({
                        "shape_KxN": f"{k}x{n}", "M": m, "gpus": world, "chunks": chunks,
                        "gemm_only_us": round(t_gemm, 2), "forward_with_gather_us": round(t_full, 2),
                        "forward_fused_exchange_us": None if t_fused is None else round(t_fused, 2),
                        "graph_replay_with_gather_us": None if t_full_g is None else round(t_full_g, 2),
                        "graph_replay_fused_exchange_us": None if t_fused_g is None else round(t_fused_g, 2),
                        "tokens_per_s": m / (t_full * 1e-6),
                        "algorithmic_tflops_gemm_only": 2.0 * m * n * k / (t_gemm * 1e-6) / 1e12,
                        "gather_bytes_per_rank": 2 * m * n // world}), flush=True)
            if fused is not None:
                fused.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
