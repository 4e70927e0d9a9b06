"""Grouped FFN decode (bitnet_ffn_group_*): every member bit-identical to the oracle's FFN block
(FeedForwardNetwork::forward, bitnet-inference/src/engine/transformer_layers.rs:608-629) and to the
member-by-member launches, for ragged widths, every token count, members that straddle CTA shares, replays."""
import numpy as np
import pytest
import torch

import oracle
from bitnet_mlx_rs_b200 import cuda, ops

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_members(seed, H, F, token_counts):
    host, members = [], []
    for i, M in enumerate(token_counts):
        g, u, d = (oracle.gen_ternary_packed(seed, 10 * i + j, F * H) for j in (1, 2, 3))
        sg, su, sd = (oracle.gen_weight_scale(seed, 10 * i + j, k) for j, k in ((1, H), (2, H), (3, F)))
        x = oracle.gen_activations(seed, 100 + i, (M, H))
        host.append((g, sg, u, su, d, sd, x))
        members.append((dev(g), sg, dev(u), su, dev(d), sd, dev(x), torch.full((M, H), float("nan"), device="cuda")))
    return host, members


def check_members(host, members, F):
    for i, ((g, sg, u, su, d, sd, x), m) in enumerate(zip(host, members)):
        ry, _ = oracle.ffn_forward(g, sg, u, su, d, sd, x, F)
        got = m[7].cpu().numpy()
        assert np.array_equal(got, ry), f"member {i} (M={x.shape[0]}): {np.abs(got - ry).max()}"


@pytest.mark.parametrize("H,F,token_counts", [
    (2560, 6912, [1, 4, 8]),                       # the 2B shape: ten warps x one step, fourteen x two
    (2560, 6912, [16, 9, 1]),                      # the same with two token tiles: five warps x two steps, seven x four
    (256, 192, [1, 2, 3, 5, 8]),                   # every image height (1, 2, 4, 8 token rows)
    (128, 1088, [7, 1]),                           # seventeen chunks over five warps: uneven K slices
    (1024, 2048, [16, 9, 1, 12]),                  # two token tiles
    (4096, 1024, [3, 16]),                         # pair at two steps per warp
    (64, 64, [1] * 5),                             # fewer blocks than SMs
])
def test_group_matches_oracle(H, F, token_counts):
    host, members = make_members(31, H, F, token_counts)
    group = ops.FfnGroup(members, H, F)
    group.run()
    torch.cuda.synchronize()
    check_members(host, members, F)
    assert ops.device_error_flags() == 0
    group.close()


def test_group_with_many_members_equals_single_launches_and_replays():
    H, F = 512, 1408
    token_counts = [1 + (i * 5) % 8 for i in range(40)]      # 40 members: every CTA share crosses members
    host, members = make_members(32, H, F, token_counts)
    group = ops.FfnGroup(members, H, F)
    group.run()
    torch.cuda.synchronize()
    for i, m in enumerate(members):
        y, _ = ops.ffn_forward(m[0], m[1], m[2], m[3], m[4], m[5], m[6], F)
        assert torch.equal(y, m[7]), f"member {i}"
    check_members(host[:6], members[:6], F)
    # new activations in the bound buffers, replayed from a CUDA graph
    for i, m in enumerate(members):
        m[6].copy_(dev(oracle.gen_activations(33, i, tuple(m[6].shape))))
        m[7].fill_(float("nan"))
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        group.run(stream=s)                                    # attributes are set outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            group.run(stream=s)
        for m in members:
            m[7].fill_(float("nan"))
        graph.replay()
        graph.replay()
    torch.cuda.synchronize()
    for i, m in enumerate(members):
        y, _ = ops.ffn_forward(m[0], m[1], m[2], m[3], m[4], m[5], m[6], F)
        assert torch.equal(y, m[7]), f"member {i} after replay"
    assert ops.device_error_flags() == 0


def test_group_refuses_what_it_cannot_run():
    host, members = make_members(34, 128, 128, [1])
    with pytest.raises(cuda.UnsupportedOperation):
        ops.FfnGroup([(*m[:6], torch.zeros((17, 128), device="cuda"), torch.zeros((17, 128), device="cuda")) for m in members], 128, 128)
    with pytest.raises(cuda.IncompatibleShapes):
        ops.FfnGroup(members, 128, 192)                         # packed sizes disagree with the stated shape


@pytest.mark.parametrize("K,N,token_counts", [
    (2560, 2560, [1, 1, 4, 8, 1]),                 # the attention-projection shape
    (64, 100, [1, 16, 3]),                          # a ragged last block of rows, two token tiles
    (1088, 40, [2] * 9),                            # uneven K slices, fewer blocks than SMs
    (8192, 48, [8, 1]),                             # four steps per warp
])
def test_bitlinear_group_matches_oracle(K, N, token_counts):
    host, members = [], []
    for i, M in enumerate(token_counts):
        wp = oracle.gen_ternary_packed(41, i, N * K)
        ws = oracle.gen_weight_scale(41, i, K)
        x = oracle.gen_activations(41, 100 + i, (M, K))
        host.append((wp, ws, x))
        members.append((dev(wp), ws, dev(x), torch.full((M, N), float("nan"), device="cuda")))
    group = ops.BitLinearGroup(members, N, K)
    group.run()
    group.run()                                     # a second run over the same bound buffers
    torch.cuda.synchronize()
    for i, ((wp, ws, x), m) in enumerate(zip(host, members)):
        ref = oracle.bitlinear_forward(wp, ws, x, N)["y"]
        assert np.array_equal(m[3].cpu().numpy(), ref), f"member {i}"
    assert ops.device_error_flags() == 0
    group.close()
