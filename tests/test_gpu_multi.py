"""Two-GPU checks (skipped on a single-GPU box): the output-feature-split layer with an NCCL
all-gather, and row-sharded independent tokens, against the CPU oracle.  Ranks are child
processes, one per GPU; NVLS is switched off so that a rank that exits early cannot disturb peers."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, M, K, N, out):
    import torch.distributed as dist
    from bitnet_mlx_rs_b200 import ops, parallel
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        wp_h = oracle.gen_ternary_packed(3, 1, N * K)
        x_h = oracle.gen_activations(3, 2, (M, K))
        scale = oracle.gen_weight_scale(3, 1, K)
        wp, x = torch.from_numpy(wp_h).cuda(), torch.from_numpy(x_h).cuda()
        layer = parallel.NSplitBitLinear(wp, scale, N, K)
        y = layer.forward(x)
        full = oracle.bitlinear_forward(wp_h, scale, x_h, N)["y"]
        ok_split = np.array_equal(y.cpu().numpy(), full)
        if M <= 16:   # the same split with the slices stored straight into every rank's output
            fused = parallel.FusedNSplitBitLinear(wp, scale, N, K)
            for _ in range(2):
                yf = fused.forward(x)
            ok_split = ok_split and np.array_equal(yf.cpu().numpy(), full)
        rows = parallel.row_sharded_forward(lambda xs: ops.bitlinear_forward(wp, scale, xs, N), x)
        b, e = parallel.shard_range(M, world, rank)
        ok_rows = np.array_equal(rows.cpu().numpy(), full[b:e])
        torch.cuda.synchronize()
        out[rank] = int(ok_split) + 2 * int(ok_rows)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M,K,N", [(1, 2560, 1024), (16, 1024, 512), (300, 256, 768)])
def test_nsplit_and_row_sharding_on_two_gpus(M, K, N):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, M, K, N, out), nprocs=2, join=True)
    assert dict(out) == {0: 3, 1: 3}
