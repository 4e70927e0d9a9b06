"""World-size-2 gloo ranks on CPU: the sharding and gathering logic of the multi-GPU schemes, with
the CPU oracle standing in for the single-GPU forward (the CUDA kernels are covered by the gpu tests)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from bitnet_mlx_rs_b200 import parallel


def test_shard_range_is_a_partition():
    for n in (0, 1, 7, 64, 1000):
        for world in (1, 2, 3, 8):
            ranges = [parallel.shard_range(n, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_range(4, 2, 2)


def _oracle_compute(wp, scale, x, n_local):
    return torch.from_numpy(oracle.bitlinear_forward(wp.numpy(), scale, x.numpy(), n_local)["y"])


def _worker(rank, world, port, M, K, N, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wp = torch.from_numpy(oracle.gen_ternary_packed(3, 1, N * K))
        x = torch.from_numpy(oracle.gen_activations(3, 2, (M, K)))
        scale = oracle.gen_weight_scale(3, 1, K)
        layer = parallel.NSplitBitLinear(wp, scale, N, K, compute=_oracle_compute)
        y = layer.forward(x)
        full = oracle.bitlinear_forward(wp.numpy(), scale, x.numpy(), N)["y"]
        ok_split = np.array_equal(y.numpy(), full)
        # independent rows: every rank handles its own rows, no communication
        rows = parallel.row_sharded_forward(lambda xs: _oracle_compute(wp, scale, xs, N), x)
        b, e = parallel.shard_range(M, world, rank)
        ok_rows = np.array_equal(rows.numpy(), full[b:e])
        out[rank] = int(ok_split) + 2 * int(ok_rows)
    finally:
        dist.destroy_process_group()


def test_nsplit_allgather_and_row_sharding_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world, (M, K, N) = 2, (5, 128, 96)
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, M, K, N, out), nprocs=world, join=True)
    assert dict(out) == {0: 3, 1: 3}
