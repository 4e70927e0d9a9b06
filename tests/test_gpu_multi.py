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
        # the same split with the slices stored straight into every rank's output (decode kernel up to 16 tokens,
        # the persistent GEMM above; its slice must satisfy that kernel's shape rules)
        if M <= 16 or (K % 128 == 0 and (N // world) % 16 == 0):
            fused = parallel.FusedNSplitBitLinear(wp, scale, N, K, max_tokens=max(M, 16))
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


@pytest.mark.parametrize("M,K,N", [(1, 2560, 1024), (16, 1024, 512), (300, 256, 768), (70, 1024, 1280)])
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


def _c_worker(rank, world, port, M, K, N, out):
    """The exchange through the C symbols alone: slice forward, then (a) ncclAllGather found by dlopen with a
    communicator made from an id passed between the ranks, (b) peer stores into every rank's output."""
    import ctypes as C
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    from bitnet_mlx_rs_b200 import _lib as L
    from bitnet_mlx_rs_b200 import cuda, ops, parallel
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        lib = L.load()
        wp_h = oracle.gen_ternary_packed(4, 1, N * K)
        x_h = oracle.gen_activations(4, 2, (M, K))
        scale = oracle.gen_weight_scale(4, 1, K)
        full = oracle.bitlinear_forward(wp_h, scale, x_h, N)["y"]
        wp, x = torch.from_numpy(wp_h).cuda(), torch.from_numpy(x_h).cuda()
        sl, (r0, r1) = parallel.packed_row_slice(wp, N, K, world, rank)
        n_local = r1 - r0
        y_local = ops.bitlinear_forward(sl.contiguous(), scale, x, n_local)
        stream = torch.cuda.current_stream().cuda_stream
        # (a) NCCL
        uid = (C.c_uint8 * 128)()
        if rank == 0:
            cuda.check(lib.bitnet_nccl_unique_id(uid))
        box = [bytes(uid)]
        dist.broadcast_object_list(box, src=0)
        uid = (C.c_uint8 * 128).from_buffer_copy(box[0])
        comm = C.c_void_p()
        cuda.check(lib.bitnet_nccl_comm_create(uid, world, rank, C.byref(comm)))
        staging = torch.empty((world, M, n_local), device="cuda")
        y_full = torch.full((M, N), float("nan"), device="cuda")
        cuda.check(lib.bitnet_allgather_output_nccl(comm, y_local.data_ptr(), M, n_local, staging.data_ptr(), y_full.data_ptr(), world, N, stream))
        torch.cuda.synchronize()
        ok_nccl = np.array_equal(y_full.cpu().numpy(), full)
        cuda.check(lib.bitnet_nccl_comm_destroy(comm))
        # (b) peer stores into symmetric memory
        y_sym = symm_mem.empty((M, N), dtype=torch.float32, device="cuda")
        handle = symm_mem.rendezvous(y_sym, dist.group.WORLD)
        y_sym.fill_(float("nan"))
        handle.barrier(channel=0)
        peers = (C.c_void_p * world)(*[int(p) + 4 * r0 for p in handle.buffer_ptrs])
        cuda.check(lib.bitnet_allgather_output(y_local.data_ptr(), M, n_local, n_local, peers, world, N, stream))
        handle.barrier(channel=1)
        torch.cuda.synchronize()
        ok_peer = np.array_equal(y_sym.cpu().numpy(), full)
        out[rank] = int(ok_nccl) + 2 * int(ok_peer)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M,K,N", [(3, 2560, 1024), (40, 1024, 512)])
def test_exchange_through_the_c_symbols_on_two_gpus(M, K, N):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_c_worker, args=(2, port, M, K, N, out), nprocs=2, join=True)
    assert dict(out) == {0: 3, 1: 3}
