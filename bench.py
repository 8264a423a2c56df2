#!/usr/bin/env python
"""Headline benchmark of the B200 ternary linear path.

Workload (named in the JSON line): the decode GEMV of BASELINE config 5 at its largest size --
K = N = 16384, M = 1 activation row per GPU -- run as a stack of LAYERS chained ternary linears
(each layer: per-token absmax int8 quantiser + 2-bit ternary GEMV + two-scale epilogue).  The stack
holds LAYERS x 64 MiB of packed weights, more than the 126 MB L2, so every step streams its
weights from HBM.  Weights are replicated on every GPU and rows (independent sequences) are sharded:
with N GPUs each rank runs its own row, no collective on the data path (weak scaling).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference ...                     # the reference's CPU path (oracle/_ref)

metric/unit: achieved HBM GB/s of algorithmic bytes (2-bit weights + fp32 x + fp32 y + scales).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM = 16384
N_DIM = 16384
LAYERS = 6
ROWS = 1
METRIC = "ternary_gemv_hbm_gbs"
UNIT = "GB/s"


def algorithmic_bytes(m: int, k: int, n: int) -> float:
    """2-bit weights + fp32 x read by the quantiser + fp32 y + (1 + M) scales."""
    return n * k / 4 + 4 * m * k + 4 * m * n + 4 * (1 + m)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs"), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.tmp.flush()
        clocks, max_clocks, reasons = [], [], set()
        with open(self.tmp.name) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    max_clocks.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.tmp.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(max_clocks) if max_clocks else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own BitLinear::forward on the host cores
# --------------------------------------------------------------------------------------------
class ReferenceSample:
    """`threads` column shards of a K-wide ternary layer (rows_per_thread outputs each), one shard per
    host thread, M = ROWS: a bounded sample of the workload on the reference's own CPU path
    (oracle/_ref, BitLinear::forward) or, where that build is absent, on the C port."""

    def __init__(self, threads: int, rows_per_thread: int, k: int = K_DIM):
        import oracle
        self.threads, self.rows = threads, rows_per_thread
        rng = np.random.default_rng(7)
        self.x = rng.standard_normal((ROWS, k)).astype(np.float32)
        self.sample = f"{threads} column shards x {rows_per_thread} rows of a {k}-wide layer, M={ROWS}"
        self.nbytes = algorithmic_bytes(ROWS, k, threads * rows_per_thread)
        if oracle.ref_available():
            self.kind = "reference"
            self.R = oracle.ref()
            self.handles = [self.R.layer_create((rng.standard_normal((rows_per_thread, k)) * 0.02).astype(np.float32))
                            for _ in range(threads)]
            self.ys = [np.zeros((ROWS, rows_per_thread), np.float32) for _ in range(threads)]
        else:
            self.kind = "port"
            self.P = oracle.port()
            w = (rng.standard_normal((threads * rows_per_thread, k)) * 0.02).astype(np.float32)
            _, self.scale, self.t, _ = self.P.pack_weights(w)
            # the port shards activation rows over threads: give every thread the same row
            self.xx = np.repeat(self.x, threads, axis=0)
            self.y = np.zeros((threads, self.t.shape[0]), np.float32)
            self.nbytes = algorithmic_bytes(threads, k, threads * rows_per_thread)

    def step(self) -> float:
        t0 = time.perf_counter()
        if self.kind == "reference":
            self.R.layers_forward_parallel(self.handles, self.x, self.ys)
        else:
            self.P.linear_forward_i8_mt(self.xx, self.t, self.scale, self.threads, y=self.y)
        return time.perf_counter() - t0

    def close(self):
        if self.kind == "reference":
            for h in self.handles:
                self.R.layer_destroy(h)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    t0 = time.perf_counter()
    ref = ReferenceSample(threads, 256)
    for _ in range(max(1, args.warmup)):
        ref.step()
    times = [ref.step() for _ in range(max(1, args.steps))]
    ref.close()
    wall = time.perf_counter() - t0
    med = statistics.median(times)
    gbs = ref.nbytes / med / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": med * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary -> int32", "data": "synthetic",
        "config": {"workload": f"C5 ternary decode GEMV K=N={K_DIM} M={ROWS}: reference CPU path, each step a bounded "
                               f"sample ({ref.sample})"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": ref.kind, "sample": ref.sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------
# this library
# --------------------------------------------------------------------------------------------
def build_layers(torch, layers: int, n: int, k: int, seed: int):
    """Synthetic N(0,0.02) weights, absmean-ternarised and packed on the device (data generation
    only: the library's own packer is the host routine checked by the tests), then relaid out
    into strips by the library."""
    from reimagined_b200 import capi
    L = capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    shifts = (2 * torch.arange(16, device="cuda", dtype=torch.int32)).view(1, 1, 16)
    out = []
    chunk = 1024
    for layer in range(layers):
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed * 1000 + layer)
        total = torch.zeros((), dtype=torch.float64, device="cuda")
        for r0 in range(0, n, chunk):
            w = torch.randn((min(chunk, n - r0), k), generator=gen, device="cuda") * 0.02
            total += w.abs().double().sum()
        absmean = (total / (n * k)).float()
        scale = absmean + 1e-8
        gen.manual_seed(seed * 1000 + layer)
        words = torch.empty((n, k // 16), dtype=torch.int32, device="cuda")
        for r0 in range(0, n, chunk):
            w = torch.randn((min(chunk, n - r0), k), generator=gen, device="cuda") * 0.02
            v = w / (scale + 1e-8)
            codes = (1 + (v > 0.5).int() - (v < -0.5).int()).view(-1, k // 16, 16)
            words[r0:r0 + codes.shape[0]] = (codes << shifts).sum(dim=2, dtype=torch.int32)
        strips = torch.empty(L.tbl_strip_bytes(n, k), dtype=torch.uint8, device="cuda")
        capi.check(L.tbl_relayout_strips(words.data_ptr(), n, k, strips.data_ptr(), st), "tbl_relayout_strips")
        torch.cuda.synchronize()
        out.append((strips, float(scale)))
        del words
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from reimagined_b200 import build as tbl_build
    tbl_build.build()
    from reimagined_b200 import capi
    L = capi.lib()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the ternary linear path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    m, k, n = ROWS, K_DIM, N_DIM
    layers = build_layers(torch, LAYERS, n, k, seed=5)
    x_host = torch.randn((m, k), generator=torch.Generator().manual_seed(100 + rank)).pin_memory()
    x_dev = x_host.cuda()
    bufs = [torch.empty((m, n), device="cuda"), torch.empty((m, n), device="cuda")]
    ws_bytes = L.tbl_linear_workspace_bytes(m, k, n)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream

    def chain_on(stream_ptr, src=None, outs=None, scratch=None):
        """One step: the input row runs through the LAYERS chained ternary linears."""
        h = x_dev if src is None else src
        outs = bufs if outs is None else outs
        scratch = ws if scratch is None else scratch
        for i, (strips, scale) in enumerate(layers):
            out = outs[i & 1]
            rc = L.tbl_linear_forward(h.data_ptr(), None, strips.data_ptr(), None, scale, m, k, n, 8, 0, None, None,
                                      out.data_ptr(), scratch.data_ptr(), ws_bytes, stream_ptr)
            if rc != 0:
                raise RuntimeError(f"tbl_linear_forward failed: {rc}")
            h = out
        return h

    def chain(src):
        return chain_on(sp, src)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    # warm up eagerly (one-time kernel attribute set-up happens here), then capture the step -- the
    # LAYERS launches of the chain -- in a CUDA graph, as a decode loop would
    for _ in range(max(3, args.warmup)):
        final = chain(x_dev)
    torch.cuda.synchronize()
    count0 = L.tbl_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=torch.cuda.Stream()):
        final = chain_on(torch.cuda.current_stream().cuda_stream)
    launches_per_step = L.tbl_launch_count() - count0

    def step_resident():
        graph.replay()

    # End to end: every step copies its input row from pinned host memory to the device, runs the chain and
    # copies the result back to pinned host memory; the three are nodes of one replayed graph.  Steps are
    # independent requests, so two lanes (own buffers, own stream) alternate and a lane's copies overlap the
    # other lane's kernels.
    class Lane:
        def __init__(self):
            self.stream = torch.cuda.Stream()
            self.x = torch.empty_like(x_dev)
            self.outs = [torch.empty((m, n), device="cuda"), torch.empty((m, n), device="cuda")]
            self.ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
            self.y_host = torch.empty((m, n)).pin_memory()
            self.x.copy_(x_host)
            self.resident = torch.cuda.CUDAGraph()          # inputs already in HBM, result left in HBM
            with torch.cuda.graph(self.resident, stream=self.stream):
                chain_on(torch.cuda.current_stream().cuda_stream, self.x, self.outs, self.ws)
            self.e2e = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.e2e, stream=self.stream):
                self.x.copy_(x_host, non_blocking=True)
                last = chain_on(torch.cuda.current_stream().cuda_stream, self.x, self.outs, self.ws)
                self.y_host.copy_(last, non_blocking=True)

    lanes = [Lane(), Lane()]

    def timed_lanes(steps, e2e):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for lane in lanes:
            lane.stream.wait_event(e0)
        for i in range(steps):
            lane = lanes[i & 1]
            with torch.cuda.stream(lane.stream):
                (lane.e2e if e2e else lane.resident).replay()
        for lane in lanes:
            stream.wait_stream(lane.stream)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    timed_lanes(max(3, args.warmup), True)
    timed_lanes(max(3, args.warmup), False)

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_single = timed(step_resident, args.steps)   # one request at a time: the kernel's own duration
    ms = timed_lanes(args.steps, False)            # two requests in flight, inputs resident
    launches = launches_per_step * args.steps      # kernels replayed by the graphs in each timed region
    ms_e2e = timed_lanes(args.steps, True)
    # the timed regions last milliseconds, nvidia-smi samples every 100 ms: keep the same replays running for
    # about 0.6 s more (untimed) so that the clock record is taken under this load
    probe_steps = max(args.steps, int(600.0 / max(ms / args.steps, 1e-3)))
    timed_lanes(probe_steps, False)
    clocks = sampler.stop()
    clocks["sampled_over"] = f"the timed regions plus {probe_steps} more untimed steps of the same replay"
    torch.cuda.synchronize()
    e2e_matches = all(bool(torch.equal(lane.y_host, final.cpu())) for lane in lanes)   # same input, same chain

    # per-launch duration of the dominant kernel: the single-request timed region replays, on one stream, a
    # graph that holds nothing but LAYERS launches of the strip GEMV (quantiser fused in its prologue), so the
    # CUDA-event time of that region divided by the launches in it is that kernel's average duration, launch
    # gaps included (with two requests in flight the kernels of the two chains overlap their heads and tails;
    # that shows in `value`, not in the roofline)
    kernel_ms = ms_single / launches
    status = L.tbl_device_status(sp)

    peak, peak_kind = measured_peaks()
    step_bytes = LAYERS * algorithmic_bytes(m, k, n)
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = world * step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    achieved = algorithmic_bytes(m, k, n) / (kernel_ms * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary(2-bit) -> int32", "data": "synthetic",
        "config": {"workload": f"C5 ternary decode GEMV K=N={k}, M={m} row per GPU, {LAYERS} chained layers per step "
                               f"({LAYERS * n * k // 4 >> 20} MiB of packed weights per step > 126 MB L2: inputs larger than L2)",
                   "parallelism": f"rows sharded over {world} GPU(s), weights replicated, no collective",
                   "launch": "the chain of a step is captured once in a CUDA graph and replayed; steps are independent "
                             "requests and two are kept in flight on two streams (value and e2e); the roofline's "
                             "kernel time is taken with one request at a time"},
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": m * k * 4, "d2h_bytes_per_step": m * n * 4,
                "ms_per_step": ms_e2e / args.steps, "matches_resident_result": e2e_matches},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "gemv_strip_kernel<1,true,2,1> (quantiser fused, single-row path)", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                     "kernel_us": kernel_ms * 1e3,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     # supplementary: the same bytes over the two-requests-in-flight region, where the head of
                     # one chain's kernel overlaps the tail of the other's (throughput, not a kernel duration)
                     "two_requests_in_flight": {"achieved": value / world, "frac": value / world / peak}},
        "device_status": status,
    }
    if rank == 0 and world == 1:
        threads = os.cpu_count() or 1
        ref = ReferenceSample(threads, 128)
        ref.step()
        med = statistics.median(ref.step() for _ in range(5))
        ref.close()
        one = ReferenceSample(1, 512)
        one.step()
        med1 = statistics.median(one.step() for _ in range(5))
        one.close()
        line["cpu_baseline"] = {"value": ref.nbytes / med / 1e9, "unit": UNIT, "cores": threads, "kind": ref.kind,
                                "sample": ref.sample + ", median of 5",
                                "single_thread": {"value": one.nbytes / med1 / 1e9, "cores": 1, "sample": one.sample}}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_strip_kernel launch at K = N = 16384, M = 1,
# from the ncu capture summarised in profiles/gemv_strip_16384x16384_m1.md
NCU_TRAFFIC_BYTES_PER_LAUNCH = 67235584 + 899328


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
