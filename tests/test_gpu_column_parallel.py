"""Column split on real GPUs: 2 NCCL ranks (child processes) must reproduce the single-GPU
result bit for bit.  Skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sacq_b200 import PrecomputedPackedVectorCodebookLinear
        from sacq_b200.column_parallel import ColumnParallelCodebookLinear
        from sacq_b200.synthetic import make_activations, make_payload
        ok = True
        failed = []
        for (n, k, m, chunks) in ((2048, 2048, 16, 1), (6144, 2048, 512, 1), (2048, 6144, 300, 3)):
            payload = make_payload(n, k, seed=3, iters=1)
            bias = (torch.randn(n, generator=torch.Generator().manual_seed(1)) * 0.05).to(torch.bfloat16)
            x = make_activations(m, k, seed=m).cuda()
            full = PrecomputedPackedVectorCodebookLinear(payload, bias, f"cuda:{rank}")
            want = full(x)
            split = ColumnParallelCodebookLinear(payload, bias, f"cuda:{rank}", chunks=chunks)
            got = split(x)
            torch.cuda.synchronize()
            if not (tuple(got.shape) == (m, n) and torch.equal(got, want)):
                ok = False
                failed.append(("gather", n, k, m, float((got.float() - want.float()).abs().max())))
            # the exchange inside the GEMM epilogue (peer stores into IPC-mapped buffers): same bytes,
            # also on the second and third call (the two result buffers alternate)
            fused = ColumnParallelCodebookLinear(payload, bias, f"cuda:{rank}", fused_exchange=True, max_tokens=m)
            for rep in range(3):
                got2 = fused(x)
                torch.cuda.synchronize()
                if not (tuple(got2.shape) == (m, n) and torch.equal(got2, want)):
                    ok = False
                    failed.append(("fused", n, k, m, rep, float((got2.float() - want.float()).abs().max())))
            x2 = make_activations(max(1, m // 2), k, seed=m + 1).cuda()
            if not torch.equal(fused(x2), full(x2)):
                ok = False
                failed.append(("fused-half", n, k, m))
            torch.cuda.synchronize()
            fused.close()
        ret[rank] = bool(ok)
        ret[f"failed{rank}"] = failed
    finally:
        dist.destroy_process_group()


def test_two_rank_column_split_matches_single_gpu():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world)), {r: ret.get(f"failed{r}") for r in range(world)}
