"""Runs one BitLinear case a few times on cuda:0 -- the small, self-ending workload meant to be
put under a profiler (or timed by hand).

    python -m bitnet_mlx_rs_b200.profile_case --kind decode --M 1 --K 8192 --N 28672 --copies 3 --iters 2

`--copies` distinct weight buffers are rotated so that every launch streams its weights from
HBM rather than L2.  Prints the mean device time per call measured with CUDA events.
"""
from __future__ import annotations

import argparse

import torch

from . import ops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", choices=["decode", "prefill", "ffn"], default="decode")
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--N", type=int, default=28672)
    ap.add_argument("--copies", type=int, default=3)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--pdl", action="store_true")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(0)

    def packed(n, k):
        w = torch.randint(0, 256, (n * k // 4,), dtype=torch.uint8, device="cuda", generator=gen)
        ops.sanitize_packed(w)
        return w

    x = torch.randn((a.M, a.K), device="cuda", generator=gen)
    if a.kind == "ffn":
        hidden, ffn = a.K, a.N
        W = [(packed(ffn, hidden), packed(ffn, hidden), packed(hidden, ffn)) for _ in range(a.copies)]
        y, h = torch.empty((a.M, hidden), device="cuda"), torch.empty((a.M, ffn), device="cuda")
        call = lambda i: ops.ffn_forward(W[i][0], 0.02, W[i][1], 0.02, W[i][2], 0.02, x, ffn, out=y, h_out=h, pdl=a.pdl)
        nbytes = 3 * ffn * hidden // 4 + 4 * a.M * (2 * hidden + 2 * ffn) + 4 * a.M * (2 * ffn + hidden)
    else:
        W = [packed(a.N, a.K) for _ in range(a.copies)]
        y = torch.empty((a.M, a.N), device="cuda")
        call = lambda i: ops.bitlinear_forward(W[i], 0.02, x, a.N, out=y, path=a.kind, pdl=a.pdl)
        nbytes = a.N * a.K // 4 + 4 * a.M * a.K + 4 * a.M * a.N
    call(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n = 0
    for _ in range(a.iters):
        for i in range(a.copies):
            call(i)
            n += 1
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / n
    print(f"{a.kind} M={a.M} K={a.K} N={a.N}: {us:.2f} us per call, {nbytes / us / 1e3:.1f} GB/s algorithmic, "
          f"{2.0 * a.M * a.K * a.N / us / 1e6:.1f} TOPS; device flags {ops.device_error_flags()}")


if __name__ == "__main__":
    main()
