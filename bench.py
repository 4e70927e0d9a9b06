#!/usr/bin/env python
"""Benchmark of the BitLinear decode hot path (one JSON line on stdout).

Workload (N=1): the BitNet b1.58 2B-shaped FFN decode GEMVs -- gate/up 2560->6912,
squared-ReLU gating, down 6912->2560 with per-token re-quantisation -- at M in {1,4,8}
tokens over 30 distinct layers' weights (398 MB packed, larger than L2), seeded synthetic
ternary weights (P(0)=0.4, P(+-1)=0.3) and N(0,1) activations with 0.1 % x20 outliers.
One step = 3 token counts x 30 layers x one FFN block = 300 kernel launches
(2 per block at M = 1, 4 at M > 1 where a small quantiser launch precedes each decode launch).
The 90 blocks of a step are independent (own weights, own input), so the step is replayed as one
CUDA graph in which they are dealt round-robin to eight streams: each block's launches stay
ordered (with programmatic dependent launch), blocks of different streams overlap on the device.
`single_chain` in the output is the same step as ONE dependent chain of launches on one stream
(the latency a single sequence sees).

metric  = algorithmic HBM GB/s: bytes N*K/4 + 4*M*K + 4*M*N per BitLinear call, summed
          over the step, divided by device time (CUDA events, max over ranks).
e2e     = the same bytes over the time of the host-buffer calls
          (bitnet_backend_ffn_forward_host_async queued round-robin on four streams, joined by
          bitnet_backend_synchronize at the end of every step: pinned H2D of x, the launches,
          D2H of y, all inside the timed region).
N > 1   = independent token batches row-sharded over ranks, weights replicated, no
          collective: weak scaling.
--impl reference times the CPU restatement of the reference path (the oracle port) on
the host cores for the same metric.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, FFN, LAYERS = 2560, 6912, 30
TOKEN_COUNTS = (1, 4, 8)
METRIC = "bitlinear_w2a8_gemv_hbm_gbs"


def call_bytes(M, K, N):
    return N * K // 4 + 4 * M * K + 4 * M * N


def ffn_bytes(M):
    return 2 * call_bytes(M, HIDDEN, FFN) + call_bytes(M, FFN, HIDDEN)


def step_bytes(layers=LAYERS):
    return sum(ffn_bytes(M) for M in TOKEN_COUNTS) * layers


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def profiled_traffic(name="decode_kernel_ffn_gate_up_m1_ncu.md"):
    """DRAM bytes per launch of the dominant kernel as the committed ncu summary records them (a line
    `traffic_bytes_per_launch: N` in that file under profiles/); (None, None) without it."""
    import re
    f = ROOT / "profiles" / name
    if f.exists():
        m = re.search(r"traffic_bytes_per_launch\s*[:=]\s*(\d+)", f.read_text())
        if m:
            return int(m.group(1)), f"profiles/{f.name}"
    return None, None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); smax.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle port on the host cores
# ------------------------------------------------------------------------------------------

def cpu_ffn_sample(steps, warmup, threads=None):
    """Times FFN blocks (M in {1,4,8}, one layer's weights) with the threaded oracle port."""
    import numpy as np
    import oracle
    try:
        oracle.build(native=True)
        native = True
    except Exception:
        native = False
    threads = threads or os.cpu_count() or 1
    g, u, d = (oracle.gen_ternary_packed(0, 1000 + i, FFN * HIDDEN) for i in range(3))
    sg, su, sd = (oracle.gen_weight_scale(0, 1000 + i, k) for i, k in ((0, HIDDEN), (1, HIDDEN), (2, FFN)))
    xs = {M: oracle.gen_activations(0, 2000 + M, (M, HIDDEN)) for M in TOKEN_COUNTS}

    def one_step():
        for M in TOKEN_COUNTS:
            up = oracle.bitlinear_forward_mt(u, su, xs[M], FFN, threads, native)
            gate = oracle.bitlinear_forward_mt(g, sg, xs[M], FFN, threads, native)
            h = up * np.square(np.maximum(gate, 0)).astype(np.float32)
            oracle.bitlinear_forward_mt(d, sd, h, HIDDEN, threads, native)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    nbytes = step_bytes(layers=1)
    return {"value": nbytes / dt / 1e9, "seconds_per_step": dt, "threads": threads, "native": native,
            "sample": f"FFN block 2560->6912->2560 at M in {list(TOKEN_COUNTS)}, 1 layer of weights, {steps} timed passes"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_ffn_sample(max(args.steps, 1), args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xternary->int32, fp32 scales",
        "data": "synthetic",
        "config": {"workload": "BitNet b1.58 2B FFN decode GEMVs (gate/up 2560->6912, ReLU^2 gating, down 6912->2560), "
                               "M in {1,4,8}", "sample": r["sample"]},
        "cpu_baseline": {"value": r["value"], "unit": "GB/s", "cores": r["threads"], "kind": "port", "sample": r["sample"],
                         "native_build": r["native"]},
        "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# CUDA arm
# ------------------------------------------------------------------------------------------

def gen_packed_on_device(torch, n_values, gen):
    """Seeded ternary weights with P(-1)=0.3, P(0)=0.4, P(+1)=0.3, packed 4 per byte (code = w+1)."""
    u = torch.rand(n_values, device="cuda", generator=gen)
    codes = ((u >= 0.3).to(torch.uint8) + (u >= 0.7).to(torch.uint8)).view(-1, 4)
    shifts = torch.tensor([0, 2, 4, 6], dtype=torch.uint8, device="cuda")
    return (codes << shifts).sum(dim=1, dtype=torch.uint8).contiguous()


def gen_activations_on_device(torch, shape, gen):
    x = torch.randn(shape, device="cuda", generator=gen)
    out = torch.rand(shape, device="cuda", generator=gen) < 0.001
    return torch.where(out, x * 20.0, x).contiguous()


def run_cuda(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from bitnet_mlx_rs_b200 import _lib, cuda, ops

    _lib.load()   # raises if the CUDA library is missing: there is no fallback
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (the CPU arm is --impl reference)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.gpus != world and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    # layer 0 comes from the host generator so that the oracle can check it byte for byte
    import oracle
    host0 = [oracle.gen_ternary_packed(0, 1000 + i, FFN * HIDDEN) for i in range(3)]
    scales0 = [oracle.gen_weight_scale(0, 1000 + i, k) for i, k in ((0, HIDDEN), (1, HIDDEN), (2, FFN))]
    Wg, Wu, Wd, S = [], [], [], []
    for l in range(LAYERS):
        if l == 0:
            g, u, d = (torch.from_numpy(h).cuda() for h in host0)
            S.append(tuple(scales0))
        else:
            g, u, d = (gen_packed_on_device(torch, FFN * HIDDEN, gen) for _ in range(3))
            S.append((0.5 / HIDDEN ** 0.5, 0.6 / HIDDEN ** 0.5, 0.7 / FFN ** 0.5))
        Wg.append(g); Wu.append(u); Wd.append(d)
    X = {M: [gen_activations_on_device(torch, (M, HIDDEN), gen) for _ in range(LAYERS)] for M in TOKEN_COUNTS}
    x0 = oracle.gen_activations(0, 2008, (8, HIDDEN))
    X[8][0] = torch.from_numpy(x0).cuda()
    Y = {M: torch.empty((LAYERS, M, HIDDEN), device="cuda") for M in TOKEN_COUNTS}
    n_streams = max(1, args.streams)
    Hb = {M: [torch.empty((M, FFN), device="cuda") for _ in range(n_streams)] for M in TOKEN_COUNTS}
    calls = [(M, l) for M in TOKEN_COUNTS for l in range(LAYERS)]
    branch = [torch.cuda.Stream() for _ in range(n_streams)] if n_streams > 1 else []

    def step(pdl, concurrent=True):
        """The step's 90 independent FFN blocks: one chain on the current stream, or dealt round-robin
        to `n_streams` streams forked from it (each block's two to four launches stay in order on
        their stream; blocks on different streams may overlap on the device)."""
        cur = torch.cuda.current_stream()
        use = branch if (concurrent and branch) else []
        for st in use:
            st.wait_stream(cur)
        for i, (M, l) in enumerate(calls):
            k = i % n_streams if use else 0
            with torch.cuda.stream(use[k] if use else cur):
                ops.ffn_forward(Wg[l], S[l][0], Wu[l], S[l][1], Wd[l], S[l][2], X[M][l], FFN, out=Y[M][l], h_out=Hb[M][k],
                                pdl=pdl, throughput=bool(use))   # small CTAs when launches of several streams share the SMs
        for st in use:
            cur.wait_stream(st)

    # per FFN block: M = 1 runs two launches (gate/up pair, down), each quantising its own input;
    # M >= 2 adds one small quantiser launch in front of each (activations are quantised once, not per CTA)
    block_launches_per_step = sum((2 if M < 2 else 4) for M in TOKEN_COUNTS) * LAYERS

    # The same 90 blocks as ONE group (bitnet_ffn_group_*): a quantiser launch and a persistent decode launch
    # per stage, each streaming the weights of every block.  This is the headline form; the per-block forms
    # (eight streams, one chain) are timed beside it.
    group = None
    if not args.per_block:
        group = ops.FfnGroup([(Wg[l], S[l][0], Wu[l], S[l][1], Wd[l], S[l][2], X[M][l], Y[M][l]) for M, l in calls], HIDDEN, FFN)
    launches_per_step = 4 if group is not None else block_launches_per_step

    # parity spot check against the oracle on layer 0, M=8 (checker only, outside any timing)
    ry, _ = oracle.ffn_forward(host0[0], scales0[0], host0[1], scales0[1], host0[2], scales0[2], x0, FFN)
    step(False)
    torch.cuda.synchronize()
    if rank == 0:
        np.testing.assert_allclose(Y[8][0].cpu().numpy(), ry, rtol=1e-5, atol=0)
    if group is not None:
        per_block = {M: Y[M].clone() for M in TOKEN_COUNTS}
        for M in TOKEN_COUNTS:
            Y[M].fill_(float("nan"))
        group.run()
        torch.cuda.synchronize()
        if rank == 0:
            np.testing.assert_allclose(Y[8][0].cpu().numpy(), ry, rtol=1e-5, atol=0)
        for M in TOKEN_COUNTS:   # every block of the group, bit for bit against the per-block launches
            if not torch.equal(Y[M], per_block[M]):
                raise RuntimeError(f"grouped FFN blocks differ from the per-block launches at M={M}")
        del per_block

    # capture the step in a CUDA graph: try programmatic dependent launch first
    side = torch.cuda.Stream()

    def capture(concurrent):
        for pdl in ((True, False) if not args.no_pdl else (False,)):
            try:
                with torch.cuda.stream(side):
                    step(pdl, concurrent)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        step(pdl, concurrent)
                g.replay()
                torch.cuda.synchronize()
                return g, ("cuda_graph+pdl" if pdl else "cuda_graph")
            except Exception as ex:   # capture not possible in this mode: try the next one
                print(f"graph capture (pdl={pdl}, concurrent={concurrent}) failed: {ex}", file=sys.stderr)
                torch.cuda.synchronize()
        return None, "eager"

    def capture_group():
        try:
            with torch.cuda.stream(side):
                group.run(stream=side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    group.run(stream=side)
            g.replay()
            torch.cuda.synchronize()
            return g, "cuda_graph+pdl"
        except Exception as ex:
            print(f"graph capture of the grouped step failed: {ex}", file=sys.stderr)
            torch.cuda.synchronize()
            return None, "eager"

    if group is not None:
        graph, mode = capture_group()
        if args.eager or graph is None:
            graph, mode = None, "eager"
        mode += ", one group of 90 blocks: 4 launches per step (bitnet_ffn_group_run)"
    else:
        graph, mode = capture(True)
        if args.eager or graph is None:
            graph, mode = None, "eager"
        if graph is not None and n_streams > 1:
            mode += f", {n_streams} concurrent streams, BITNET_FLAG_THROUGHPUT"

    def run_step():
        if graph is not None:
            graph.replay()
        elif group is not None:
            group.run()
        else:
            step(False, False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    clocks = sampler.stop() if rank == 0 else None

    nbytes = step_bytes()

    def per_block_figure(concurrent):
        g1, mode1 = capture(concurrent)
        if g1 is None:
            return None
        for _ in range(3):
            g1.replay()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        c0.record()
        n1 = max(5, min(args.steps, 20))
        for _ in range(n1):
            g1.replay()
        c1.record()
        barrier()
        ms1 = c0.elapsed_time(c1) / n1
        return {"ms_per_step": ms1, "value": nbytes / (ms1 * 1e-3) / 1e9, "unit": "GB/s", "launch_mode": mode1,
                "launches_per_step": block_launches_per_step, "us_per_ffn_block": ms1 * 1e3 / len(calls)}

    # the same step as ONE dependent chain of per-block launches on one stream (what a single sequence sees),
    # and as per-block launches dealt to the streams
    chain, streamed = None, None
    if graph is not None and not args.eager:
        chain = per_block_figure(False)
        if group is not None and n_streams > 1:
            streamed = per_block_figure(True)
            if streamed:
                streamed["launch_mode"] += f", {n_streams} concurrent streams, BITNET_FLAG_THROUGHPUT"
    value = world * nbytes * args.steps / (ms_total * 1e-3) / 1e9
    per_gpu = value / world
    peak, peak_kind = measured_peaks()

    # ---- end to end through the host-buffer C-ABI calls --------------------------------------
    # The step's 90 FFN blocks as one bound batch (bitnet_backend_ffn_plan_*): host buffers in, host
    # buffers out, every step copies each x from page-locked host memory to the device and each y back,
    # inside the timed region.  The per-call asynchronous form of the same work is timed beside it.
    E2E_STREAMS = 4   # the reference's default stream pool size (backend.rs:32)
    backend = cuda.CudaBackend(cuda.CudaBackendConfig(device_id=local, memory_pool_size=2 << 30, num_streams=E2E_STREAMS))
    e2e_layers = LAYERS
    dw = [(backend.upload_packed(Wg[l].cpu().numpy(), FFN, HIDDEN, S[l][0]),
           backend.upload_packed(Wu[l].cpu().numpy(), FFN, HIDDEN, S[l][1]),
           backend.upload_packed(Wd[l].cpu().numpy(), HIDDEN, FFN, S[l][2])) for l in range(e2e_layers)]
    xh = {M: [X[M][l].cpu().numpy() for l in range(e2e_layers)] for M in TOKEN_COUNTS}
    yh = {M: [np.empty((M, HIDDEN), dtype=np.float32) for _ in range(e2e_layers)] for M in TOKEN_COUNTS}
    calls = [(M, l) for M in TOKEN_COUNTS for l in range(e2e_layers)]
    for M, l in calls:
        backend.pin_host(xh[M][l]); backend.pin_host(yh[M][l])
    plan = backend.ffn_plan([(*dw[l], xh[M][l], yh[M][l]) for M, l in calls], n_lanes=n_streams)

    def timed_host(fn, steps):
        for _ in range(3):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device="cuda")
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return world * nbytes * steps / float(dt.item()) / 1e9

    e2e_steps = max(3, min(args.steps, 50))
    for M, l in calls:
        yh[M][l].fill(np.nan)
    e2e_value = timed_host(plan.run, e2e_steps)
    if rank == 0:
        np.testing.assert_allclose(yh[8][LAYERS - 1], Y[8][LAYERS - 1].cpu().numpy(), rtol=1e-5, atol=0)
        np.testing.assert_allclose(yh[1][0], Y[1][0].cpu().numpy(), rtol=1e-5, atol=0)
        np.testing.assert_allclose(yh[4][7], Y[4][7].cpu().numpy(), rtol=1e-5, atol=0)
    plan.close()

    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(max_workers=E2E_STREAMS)

    def feed(sidx):
        # one host thread per stream (the C calls release the interpreter lock)
        for M, l in calls[sidx::E2E_STREAMS]:
            backend.ffn_forward_host_async(dw[l][0], dw[l][1], dw[l][2], xh[M][l], yh[M][l], stream_idx=sidx)

    def async_step():
        list(pool.map(feed, range(E2E_STREAMS)))
        backend.synchronize()

    e2e_async = timed_host(async_step, max(3, min(args.steps, 20)))
    for M, l in calls:
        backend.unpin_host(xh[M][l]); backend.unpin_host(yh[M][l])
    io_bytes = sum(M * HIDDEN * 4 for M in TOKEN_COUNTS) * LAYERS
    pool.shutdown()
    backend.close()

    # ---- supporting single-kernel figures (same kernel, other configs of the spec) ---------------
    extra = {}
    if rank == 0 and not args.no_extra:
        extra = single_kernel_figures(torch, ops, gen, peak)
    # ---- the sharded configs: the oversized layer split over the ranks, the model's sequences row-sharded ----
    del Wg, Wu, Wd, X, Y, Hb, dw
    torch.cuda.empty_cache()
    nsplit = model = None
    if world > 1 and not args.no_extra:
        barrier()
        nsplit = nsplit_figures(torch, dist, ops, world, rank)
    if not args.no_model:
        barrier()
        model = model_figures(torch, dist, local, world, peak, layers=args.model_layers or None)

    traffic, traffic_source = profiled_traffic("decode_group_kernel_ffn_gate_up_90_blocks_ncu.md") if group is not None else profiled_traffic()
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        r = cpu_ffn_sample(steps=max(args.steps, 1), warmup=max(args.warmup, 1))   # as many passes as the reference arm times
        cpu = {"value": r["value"], "unit": "GB/s", "cores": r["threads"], "kind": "port", "sample": r["sample"],
               "native_build": r["native"]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8xternary->int32, fp32 scales", "data": "synthetic",
            "config": {"workload": "BitNet b1.58 2B FFN decode GEMVs (gate/up 2560->6912, ReLU^2 gating, down 6912->2560), "
                                   "M in {1,4,8}, 30 layers of distinct weights per step",
                       "l2": "inputs larger than L2 (398 MB of packed weights per step)", "launch_mode": mode,
                       "parallelism": f"row-sharded x{world}, weights replicated, no collective"},
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "peak_kind": peak_kind,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch at M = 1, read from the
                         # committed ncu summary of that kernel (not measured by this run); algorithmic 8.89 MB
                         "traffic": traffic, "traffic_source": traffic_source,
                         "kernel": ("decode_group_kernel (one gate/up launch and one down launch over all 90 blocks; "
                                    if group is not None else "decode_kernel (gate/up pair and down launches; ") +
                                   f"algorithmic bytes per launch {step_bytes() / launches_per_step:.0f} on average); achieved "
                                   "= bytes of the whole step / CUDA-event time of the whole graph-replayed step (every "
                                   "launch in it is this kernel or its quantiser)"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
                    "steps": e2e_steps,
                    "api": "bitnet_backend_ffn_plan_run: the step's 90 FFN blocks bound to page-locked host buffers, run as three "
                           "groups; per group one launch copies its inputs host->device, four launches compute, one launch copies "
                           "its outputs device->host (copies of one group overlap the kernels of another)",
                    "per_call_async": {"value": e2e_async, "unit": "GB/s",
                                       "api": f"bitnet_backend_ffn_forward_host_async on {E2E_STREAMS} streams, one host thread "
                                              "each, + bitnet_backend_synchronize per step"}},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if chain:
            line["single_chain"] = chain
        if streamed:
            line["per_block_streams"] = streamed
        if cpu:
            line["cpu_baseline"] = cpu
        if extra:
            line["kernels"] = extra
        if nsplit:
            line["nsplit"] = nsplit
        if model:
            line["cfg4_model_decode"] = model
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def single_kernel_figures(torch, ops, gen, peak):
    """Device time of single BitLinear launches at the other decode shapes of the spec,
    rotating over enough weight copies to exceed L2."""
    out = {}
    for name, (M, K, N) in {"cfg1_m1_2560x2560": (1, 2560, 2560), "cfg5_m1_8192x28672": (1, 8192, 28672),
                            "cfg5_m16_8192x28672": (16, 8192, 28672)}.items():
        copies = max(2, min(96, int(400e6 // (N * K // 4)) + 1))
        W = [gen_packed_on_device(torch, N * K, gen) for _ in range(copies)]
        x = gen_activations_on_device(torch, (M, K), gen)
        y = torch.empty((M, N), device="cuda")
        def rotate():
            for w in W:
                ops.bitlinear_forward(w, 0.01, x, N, out=y, pdl=True)

        rotate()
        torch.cuda.synchronize()
        run, launch = rotate, "stream launches"
        try:   # one pass over all copies as a CUDA graph: launch overhead stays out of the figure
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    rotate()
            g.replay()
            torch.cuda.synchronize()
            run, launch = g.replay, "cuda graph"
        except Exception as ex:
            print(f"single-kernel figure {name}: graph capture failed ({ex}); timing stream launches", file=sys.stderr)
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
        gbs = call_bytes(M, K, N) / us / 1e3
        out[name] = {"us": us, "gbs": gbs, "frac_of_peak": gbs / peak, "weight_copies": copies, "launch": launch}
        del W
    # cfg1 as a batch: 96 independent single-token 2560 -> 2560 projections (weights of their own, 157 MB) as one group
    M, K, N, n = 1, 2560, 2560, 96
    members = [(gen_packed_on_device(torch, N * K, gen), 0.01, gen_activations_on_device(torch, (M, K), gen),
                torch.empty((M, N), device="cuda")) for _ in range(n)]
    group = ops.BitLinearGroup(members, N, K)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        group.run(stream=side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            group.run(stream=side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (10 * n)
    gbs = call_bytes(M, K, N) / us / 1e3
    out["cfg1_m1_2560x2560_group_of_96"] = {"us": us, "gbs": gbs, "frac_of_peak": gbs / peak, "members": n,
                                             "launch": "cuda graph, bitnet_bitlinear_group_run (2 launches for the group)"}
    group.close()
    out["cfg3_prefill_layer_m2048"] = prefill_layer_figures(torch, ops, gen)
    return out


MODEL = dict(num_layers=30, vocab_size=128256, hidden_size=2560, num_heads=20, num_kv_heads=5, head_dim=128,
             ffn_intermediate_size=6912)
MODEL_CONTEXT, MODEL_NEW_TOKENS, MODEL_SEQUENCES = 512, 128, 64


def model_step_bytes(seqs, context):
    """HBM bytes one decode step must move: every packed weight once (layers + language-model head), and each
    sequence's cached keys and values (bf16) at the given context length."""
    H, F, V, L = MODEL["hidden_size"], MODEL["ffn_intermediate_size"], MODEL["vocab_size"], MODEL["num_layers"]
    qd, kd = MODEL["num_heads"] * MODEL["head_dim"], MODEL["num_kv_heads"] * MODEL["head_dim"]
    weights = L * ((qd + 2 * kd) * H + H * qd + 3 * F * H) // 4 + V * H // 4
    kv = L * 2 * kd * 2 * context * seqs
    return weights, kv


class ModelBench:
    """The random-init 2B-shaped model (30 layers, hidden 2560, 20 heads / 5 KV heads, head_dim 128, FFN 6912, vocabulary
    128256, bf16 KV cache) on one GPU, built once; `run(seqs)` caches `context` random tokens per sequence (not timed),
    then generates `new_tokens` tokens per sequence greedily through bitnet_decoder_decode -- host token ids in, host
    token ids out: the wall time of that call is the figure."""

    def __init__(self, local, max_seqs, context=MODEL_CONTEXT, new_tokens=MODEL_NEW_TOKENS, layers=None):
        import numpy as np

        import oracle
        from bitnet_mlx_rs_b200 import cuda
        from bitnet_mlx_rs_b200.pipeline import ForwardPassConfig, ForwardPassPipeline

        self.local, self.context, self.new_tokens = local, context, new_tokens
        cfgd = dict(MODEL)
        if layers:
            cfgd["num_layers"] = layers
        cfg = self.cfg = ForwardPassConfig(max_seq_len=context + new_tokens, max_batch=max_seqs, **cfgd)
        H, F, V = cfg.hidden_size, cfg.ffn_intermediate_size, cfg.vocab_size
        qd, kd = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        self.backend = cuda.CudaBackend(cuda.CudaBackendConfig(device_id=local, memory_pool_size=24 << 30))
        self.pipe = pipe = ForwardPassPipeline(self.backend, cfg)
        block = oracle.gen_activations(0, 7000, (8192, H))
        pipe.load_embedding(np.tile(block, (V // 8192 + 1, 1))[:V])
        ones, zeros = np.ones(H, np.float32), np.zeros(H, np.float32)
        for l in range(cfg.num_layers):
            shapes = {"q": (qd, H), "k": (kd, H), "v": (kd, H), "o": (H, qd), "gate": (F, H), "up": (F, H), "down": (H, F)}
            lw = {}
            for i, (name, (n, k)) in enumerate(shapes.items()):
                lw[name] = oracle.gen_ternary_packed(0, 8000 + 10 * l + i, n * k)
                lw["s_" + {"gate": "g", "up": "u", "down": "d"}.get(name, name)] = oracle.gen_weight_scale(0, 8000 + 10 * l + i, k)
            lw.update(n1w=ones, n1b=zeros, n2w=ones, n2b=zeros)     # SubLNNormalization::new: ones and zeros
            pipe.load_layer(l, lw)
        pipe.load_lm_head(oracle.gen_ternary_packed(0, 8999, V * H), oracle.gen_weight_scale(0, 8999, H))

    def run(self, seqs, peak_gbs):
        import numpy as np

        from bitnet_mlx_rs_b200.pipeline import SamplingConfig
        V, context, new_tokens = self.cfg.vocab_size, self.context, self.new_tokens
        rng = np.random.default_rng(self.local)
        ids = rng.integers(0, V, size=(seqs, context)).astype(np.int32)
        self.pipe.reset()
        self.pipe.feed(ids[:, :context - 1])
        warm, _ = self.pipe.decode(ids[:, context - 1], 3, SamplingConfig(deterministic=True))     # records the step graph
        t0 = time.perf_counter()
        toks, steps = self.pipe.decode(warm[:, -1], new_tokens - 3, SamplingConfig(deterministic=True))
        dt = time.perf_counter() - t0
        assert steps == new_tokens - 3 and (toks >= 0).all() and (toks < V).all()
        ms_step = dt * 1e3 / steps
        weights, kv = model_step_bytes(seqs, context + new_tokens // 2)
        return {"sequences": seqs, "context": context, "new_tokens": steps, "ms_per_step": ms_step, "tokens_per_s": seqs * steps / dt,
                "seconds": dt, "hbm_bytes_per_step": weights + kv, "gbs": (weights + kv) / (ms_step * 1e-3) / 1e9,
                "frac_of_hbm_peak": (weights + kv) / (ms_step * 1e-3) / 1e9 / peak_gbs,
                "roofline_ms_per_step": (weights + kv) / (peak_gbs * 1e9) * 1e3}

    def close(self):
        self.pipe.close()
        self.backend.close()


def model_figures(torch, dist, local, world, peak_gbs, layers=None):
    """cfg4: 64 sequences with a 512-token context generating 128 tokens each.  weak = 64 sequences on EVERY GPU;
    strong = the 64 sequences row-sharded over the GPUs (64 / N each), weights replicated, no collective.  Times are
    the maximum over ranks; tokens/s are whole-job figures."""
    bench = ModelBench(local, MODEL_SEQUENCES, layers=layers)
    full = bench.run(MODEL_SEQUENCES, peak_gbs)
    share = full if world == 1 else bench.run(max(1, MODEL_SEQUENCES // world), peak_gbs)
    bench.close()

    def slowest(seconds):
        t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_full, t_share = slowest(full["seconds"]), slowest(share["seconds"])
    steps = full["new_tokens"]
    w, kv = model_step_bytes(MODEL_SEQUENCES, MODEL_CONTEXT + MODEL_NEW_TOKENS // 2)
    out = {"model": "random-init BitNet b1.58 2B shape: 30 layers, hidden 2560, 20 heads / 5 KV heads, head_dim 128, FFN 6912, "
                    "vocabulary 128256, bf16 KV cache; LM head as a BitLinear; greedy sampling on the device",
           "io": "token ids host->device before the call, generated ids device->host after it (bitnet_decoder_decode)",
           "weak": {"sequences_per_gpu": MODEL_SEQUENCES, "tokens_per_s": world * MODEL_SEQUENCES * steps / t_full,
                    "ms_per_step": t_full * 1e3 / steps, "frac_of_hbm_roofline": full["roofline_ms_per_step"] / (t_full * 1e3 / steps)},
           "strong": {"sequences_total": MODEL_SEQUENCES, "sequences_per_gpu": share["sequences"],
                      "tokens_per_s": world * share["sequences"] * steps / t_share, "ms_per_step": t_share * 1e3 / steps,
                      "speedup_vs_one_gpu": t_full / t_share,
                      "roofline_predicted_speedup": (w + kv) / (w + kv / world),
                      "frac_of_hbm_roofline": share["roofline_ms_per_step"] / (t_share * 1e3 / steps)}}
    return out


def nsplit_figures(torch, dist, ops, world, rank):
    """cfg5: the oversized layer K = 8192, N = 28672 at M in {1, 16, 256}, output features split over the ranks.  Two forms:
    every rank computes its column slice and the fp32 slices are all-gathered with NCCL; or every rank's kernel (the decode
    kernel up to 16 tokens, the persistent GEMM above) stores its slice straight into every GPU's output over NVLink and
    a barrier replaces the collective.  Before
    any timing each form's result is compared bit for bit with the single-GPU result of the same layer on this rank.
    Times: CUDA events, graph replay where it captures, maximum over ranks."""
    from bitnet_mlx_rs_b200 import parallel
    K, N = 8192, 28672
    n_local = N // world
    gen = torch.Generator(device="cuda").manual_seed(7)   # the same weights on every rank; each keeps its slice
    copies = max(2, -(-(160 << 20) // (n_local * K // 4)))   # rotate enough slices to exceed L2
    copies += copies % 2   # an even count: the two shared outputs then alternate across graph replays too
    layers, fused, full0 = [], [], None
    for c in range(copies):
        full = gen_packed_on_device(torch, N * K, gen)
        layers.append(parallel.NSplitBitLinear(full, 0.01, N, K))
        fused.append(parallel.FusedNSplitBitLinear(full, 0.01, N, K, max_tokens=256, share_outputs_with=fused[0] if fused else None))
        if c == 0:
            full0 = full
        del full
    out = {"layer": "K=8192 -> N=28672, N-split over %d GPUs (%d columns each)" % (world, n_local), "weight_copies_rotated": copies}

    def timed(fn, reps):
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3

    def graphed(body):
        """`body` replayed as one CUDA graph when it captures (launch overhead off the clock), else as it is."""
        try:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    body()
            g.replay()
            torch.cuda.synchronize()
            return g.replay, "cuda graph"
        except Exception as ex:   # capture is an optimisation of the measurement, not of the result
            print(f"N-split: graph capture failed ({type(ex).__name__}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            return body, "eager"

    for M in (1, 16, 256):
        x = gen_activations_on_device(torch, (M, K), gen)
        y_one = ops.bitlinear_forward(full0, 0.01, x, N)          # the whole layer on this GPU alone
        y_ag = layers[0].forward(x)
        same_ag = bool(torch.equal(y_ag, y_one))
        y_f = fused[0].forward(x).clone()
        same_fused = bool(torch.equal(y_f, y_one))
        flags = torch.tensor([int(same_ag), int(same_fused is not False)], device="cuda")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        entry = {"equals_single_gpu": bool(flags[0].item()) and bool(flags[1].item()),
                 "allgather_bytes_per_gpu": 4 * M * N * (world - 1) // world}
        y_buf = torch.empty((M, N), device="cuda")
        run1, mode1 = graphed(lambda: ops.bitlinear_forward(full0, 0.01, x, N, out=y_buf, pdl=True))
        entry["us_one_gpu"] = timed(run1, 20)
        entry["us_allgather"] = timed(lambda: [layers[i].forward(x) for i in range(copies)], 4) / copies
        runf, modef = graphed(lambda: [fused[i].forward(x) for i in range(copies)])
        entry["us_fused"] = timed(runf, 4) / copies
        entry["fused_launch"] = modef
        # without the barrier in front: the rotated layers alternate two outputs between them, calls are issued in
        # stream order, so a buffer is written again only after every rank passed the barrier of the call in between
        runf1, _ = graphed(lambda: [fused[i].forward(x, guard=False) for i in range(copies)])
        entry["us_fused_one_barrier"] = timed(runf1, 4) / copies
        out[f"m{M}"] = entry
    return out


def prefill_layer_figures(torch, ops, gen):
    """The seven BitLinear projections of one 2B decoder layer at M = 2048 tokens through the
    tensor-core path (quantiser launch + tcgen05 GEMM each), replayed from a CUDA graph."""
    M = 2048
    shapes = {"q": (2560, 2560), "k": (2560, 640), "v": (2560, 640), "o": (2560, 2560),
              "gate": (2560, 6912), "up": (2560, 6912), "down": (6912, 2560)}
    W = {k: gen_packed_on_device(torch, N * K, gen) for k, (K, N) in shapes.items()}
    X = {k: gen_activations_on_device(torch, (M, K), gen) for k, (K, N) in shapes.items()}
    Y = {k: torch.empty((M, N), device="cuda") for k, (K, N) in shapes.items()}

    branch = [torch.cuda.Stream() for _ in range(3)]

    def layer(concurrent):
        # the seven projections have their own inputs: one after the other on one stream, or dealt to
        # three streams so that one projection's quantiser and short GEMMs overlap another's GEMM
        cur = torch.cuda.current_stream()
        use = branch if concurrent else []
        for st in use:
            st.wait_stream(cur)
        for i, (k, (K, N)) in enumerate(shapes.items()):
            with torch.cuda.stream(use[i % len(use)] if use else cur):
                ops.bitlinear_forward(W[k], 0.01, X[k], N, out=Y[k], path="prefill")
        for st in use:
            cur.wait_stream(st)

    def timed(concurrent):
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            layer(concurrent)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                layer(concurrent)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    us_chain = timed(False)
    us = timed(True)
    int_ops = sum(2.0 * M * K * N for (K, N) in shapes.values())
    tops = int_ops / us / 1e6
    return {"us": us, "tops": tops, "int_ops": int_ops, "bound": "tensor", "launch_mode": "cuda graph, projections on 3 streams",
            "us_one_stream": us_chain, "tops_one_stream": int_ops / us_chain / 1e6,
            "frac_of_nominal_int8_peak_4500": tops / 4500.0,
            "note": "no measured int8 peak on this pool; 4500 TOPS is the nominal dense figure"}


def run_case(spec):
    """One BitLinear (or FFN) shape on cuda:0, timed with CUDA events -- the small, self-ending workload that the
    profiling commands under profiles/ run.  spec = kind:M:K:N[:copies[:iters]] with kind one of auto, decode, cluster,
    prefill, generic (a single BitLinear through that path), ffn (K = hidden, N = ffn) or ffngroup (`copies` independent
    FFN blocks of M tokens each as one grouped run).  `copies` distinct weight buffers are rotated so that every launch
    streams its weights from HBM rather than L2."""
    import torch

    from bitnet_mlx_rs_b200 import ops
    parts = spec.split(":")
    kind, M, K, N = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    copies = int(parts[4]) if len(parts) > 4 else 3
    iters = int(parts[5]) if len(parts) > 5 else 2
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = gen_activations_on_device(torch, (M, K), gen)
    if kind == "attn":
        # decode attention of the 2B shape: M sequences, K cached tokens each, bf16 cache, rotating `copies` caches
        nh, nkv, hd = MODEL["num_heads"], MODEL["num_kv_heads"], MODEL["head_dim"]
        caches = [(torch.randn((M, nkv, K + 8, hd), device="cuda", generator=gen).to(torch.bfloat16),
                   torch.randn((M, nkv, K + 8, hd), device="cuda", generator=gen).to(torch.bfloat16)) for _ in range(copies)]
        qkv = torch.randn((M, (nh + 2 * nkv) * hd), device="cuda", generator=gen)
        pos = torch.full((M,), K, dtype=torch.int32, device="cuda")
        call = lambda i: ops.attention_decode(qkv, caches[i][0], caches[i][1], pos, nh, nkv, hd, n_splits=N)   # noqa: E731  (N = splits, 0 = choose)
        nbytes = 2 * M * nkv * (K + 1) * hd * 2
        int_ops = 4.0 * M * nh * (K + 1) * hd
    elif kind == "ffngroup":
        W = [tuple(gen_packed_on_device(torch, K * N, gen) for _ in range(3)) for _ in range(copies)]
        xs = [gen_activations_on_device(torch, (M, K), gen) for _ in range(copies)]
        ys = [torch.empty((M, K), device="cuda") for _ in range(copies)]
        group = ops.FfnGroup([(W[i][0], 0.02, W[i][1], 0.02, W[i][2], 0.02, xs[i], ys[i]) for i in range(copies)], K, N)
        nbytes = copies * (2 * call_bytes(M, K, N) + call_bytes(M, N, K))
        int_ops = copies * 6.0 * M * K * N
    elif kind == "ffn":
        W = [tuple(gen_packed_on_device(torch, K * N, gen) for _ in range(3)) for _ in range(copies)]
        y, h = torch.empty((M, K), device="cuda"), torch.empty((M, N), device="cuda")
        call = lambda i: ops.ffn_forward(W[i][0], 0.02, W[i][1], 0.02, W[i][2], 0.02, x, N, out=y, h_out=h, pdl=True)   # noqa: E731
        nbytes = 2 * call_bytes(M, K, N) + call_bytes(M, N, K)
        int_ops = 6.0 * M * K * N
    else:
        W = [gen_packed_on_device(torch, N * K, gen) for _ in range(copies)]
        y = torch.empty((M, N), device="cuda")
        call = lambda i: ops.bitlinear_forward(W[i], 0.02, x, N, out=y, path=kind, pdl=True)   # noqa: E731
        nbytes = call_bytes(M, K, N)
        int_ops = 2.0 * M * K * N
    if kind == "ffngroup":   # one run covers all copies
        call = lambda i: group.run() if i == 0 else None   # noqa: E731
        nbytes, int_ops = nbytes / copies, int_ops / copies
    call(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # a graph of one pass over the copies keeps launch overhead out of the figure
    run, mode = None, "stream launches"
    try:
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(copies):
                    call(i)
        g.replay()
        torch.cuda.synchronize()
        run, mode = g.replay, "cuda graph"
    except Exception as ex:
        print(f"graph capture failed ({ex}); timing stream launches", file=sys.stderr)
        torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        if run:
            run()
        else:
            for i in range(copies):
                call(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (iters * copies)
    print(json.dumps({"case": spec, "us_per_call": us, "gbs": nbytes / us / 1e3, "tops": int_ops / us / 1e6, "launch": mode,
                      "device_flags": ops.device_error_flags()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--eager", action="store_true", help="launch kernels one by one instead of replaying a CUDA graph")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--streams", type=int, default=8, help="streams the per-block form deals the step's independent FFN blocks to (1 = one chain)")
    ap.add_argument("--per-block", action="store_true", help="headline from per-block launches on --streams streams instead of the grouped launch")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-extra", action="store_true", help="skip the single-kernel figures")
    ap.add_argument("--no-model", action="store_true", help="skip the model decode figure (cfg4)")
    ap.add_argument("--case", default="", metavar="kind:M:K:N[:copies[:iters]]",
                    help="time one BitLinear/FFN shape on GPU 0 and print it (the workload of the profiling commands)")
    ap.add_argument("--model-only", type=int, default=0, metavar="SEQS",
                    help="run only the model decode figure for this many sequences on GPU 0 and print it")
    ap.add_argument("--model-layers", type=int, default=0, help="with --model-only: fewer layers (quick look)")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
    elif args.model_only:
        mb = ModelBench(0, args.model_only, layers=args.model_layers or None)
        print(json.dumps(mb.run(args.model_only, measured_peaks()[0])))
        mb.close()
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
