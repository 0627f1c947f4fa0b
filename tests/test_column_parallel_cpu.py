"""Host-side logic of the column split, on CPU: payload sharding against the oracle, and
the all-gather layout with two gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sacq_oracle as O
from sacq_b200 import column_parallel as cp
from sacq_b200.synthetic import make_payload


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _weight(p):
    return O.dequantize_packed_bf16_bits(p["packed_indices"].numpy(), p["index_bits"], _bits(p["codebook"]),
                                         _bits(p["scales"]), 0, p["out_features"], p["in_features"], p["group_size"])


@pytest.mark.parametrize("N,K,d,C,world", [(64, 128, 8, 4096, 2), (64, 128, 8, 4096, 4), (24, 24, 4, 8, 8),
                                           (12, 24, 4, 8, 4), (32, 64, 8, 256, 8)])
def test_shards_reconstruct_to_the_full_weight(N, K, d, C, world):
    full = make_payload(N, K, vector_dim=d, codebook_size=C, seed=N + world, iters=1)
    w_full = _weight(full)
    parts = [_weight(cp.shard_payload(full, r, world)) for r in range(world)]
    assert np.array_equal(np.concatenate(parts, axis=0), w_full)
    unpacked = make_payload(N, K, vector_dim=d, codebook_size=C, seed=N + world, iters=1, packed=False)
    sh = cp.shard_payload(unpacked, 1, world)
    assert tuple(sh["indices"].shape)[0] == N // world and sh["out_features"] == N // world


def test_shard_argument_errors():
    p = make_payload(10, 16, vector_dim=4, codebook_size=16, seed=0)
    with pytest.raises(ValueError):
        cp.shard_payload(p, 0, 3)
    with pytest.raises(ValueError):
        cp.shard_rows(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n = 5, 12
        ref = torch.arange(m * n, dtype=torch.float32).reshape(m, n)
        begin, end = cp.shard_rows(n, rank, world)
        full = cp.gather_columns(ref[:, begin:end].contiguous())
        ok = torch.equal(full, ref)
        out = torch.empty(m, n)
        cp.gather_columns(ref[:, begin:end].contiguous(), out=out)
        ok = ok and torch.equal(out, ref)
        # a rank that disagrees about the shard width is caught by the collective's shape check
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_gather_columns_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world))
