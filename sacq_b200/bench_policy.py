"""Policy-forward throughput of the synthetic GR00T-shaped model (all linears W1.5A8):

    python -m sacq_b200.bench_policy [--queries 20] [--no-graph]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        --master-port 29521 -m sacq_b200.bench_policy

Each rank serves independent batch-1 queries (data parallel, no communication).  Protocol
mirrors the reference's timing worker (5 warm-up + N measured queries, fixed observation
and noise, one CUDA-graph launch per query, CUDA events): prints one JSON line with the
median latency and the aggregate forwards/s over all ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from . import _lib
from .policy import SyntheticGr00tPolicy


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--queries", type=int, default=20)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    policy = SyntheticGr00tPolicy(str(dev), seed=0)
    image, noise = policy.example_inputs(42)
    lib = _lib.load()
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for _ in range(2):
            ref = policy(image, noise)
    stream.synchronize()
    launches0 = lib.sacq_launch_count()
    if args.no_graph:
        def run():
            return policy(image, noise)
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = policy(image, noise)

        def run():
            graph.replay()
            return out
    launches = lib.sacq_launch_count() - launches0
    times = []
    with torch.cuda.stream(stream):
        for i in range(5 + args.queries):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            y = run()
            e1.record(stream)
            stream.synchronize()
            if i >= 5:
                times.append(e0.elapsed_time(e1))
    same = bool(torch.equal(y, ref))
    med = statistics.median(times)
    t = torch.tensor([med], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "workload": "synthetic GR00T-N1.5-shaped policy, batch 1, 4 denoising steps, all linears W1.5A8",
            "gpus": world, "median_ms_per_query": float(t.item()), "forwards_per_s": world * 1e3 / float(t.item()),
            "quantized_linears": policy.num_quantized_linears,
            "quantized_linear_calls_per_query": policy.quantized_linear_calls_per_query(),
            "sacq_kernel_launches_per_query": int(launches) if not args.no_graph else None,
            "graph": not args.no_graph, "deterministic": same, "queries": args.queries}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
