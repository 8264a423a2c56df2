#!/usr/bin/env python
"""Benchmark of the B200 ternary linear path: the whole metric in one JSON line.

Headline (`metric`, `value`, `roofline`, `e2e`): the decode GEMV of the standalone sweep at its largest size --
K = N = 16384, M = 1 activation row per GPU -- as a stack of LAYERS chained ternary linears (each layer:
per-token absmax int8 quantiser + 2-bit ternary GEMV + two-scale epilogue; layer i+1 consumes layer i's
output).  A step is ONE request going through the stack, i.e. one launch of the persistent kernel behind
`tbl_chain_forward`; the stack holds LAYERS x 64 MiB of packed weights, more than the 126 MB L2, so every
step streams its weights from HBM.  Weights are replicated on every GPU and rows (independent sequences) are
sharded: with N GPUs each rank runs its own row, no collective on the data path (weak scaling).

The other two thirds of the metric ride in the same line:
  "gemm"    prefill ternary x int8 GEMM on tcgen05 (standalone sweep M = 8192 at K = N = 8192 / 16384 and the two
            D768 prefill shapes, M = 4096): int8 TOPS, fraction of min(ops / 4.5 POPS, bytes / HBM), the
            torch._int_mm ceiling measured beside it; rows sharded over the ranks;
  "decode"  one full decode step of the D768 / 16-block hybrid (every op of the step, replayed from a CUDA graph)
            at batch 1 / 8 / 64: tokens/s and kernels per step; sequences sharded over the ranks;
  "colsplit" (N > 1 only) the 16384-wide layer split by output columns with one NCCL all-gather.
Results are verified against the CPU oracle BEFORE anything is timed, and the line carries SHA-256 digests of
the inputs and weights that were timed.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference ...                     # the reference's CPU path (oracle/_ref)

metric/unit: achieved HBM GB/s of algorithmic bytes (2-bit weights + fp32 x + fp32 y + scales).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_DIM = 16384
N_DIM = 16384
LAYERS = 16
ROWS = 1
METRIC = "ternary_gemv_hbm_gbs"
UNIT = "GB/s"
INT8_DENSE_PEAK_TOPS = 4500.0     # nominal dense int8 tensor peak of a B200


def algorithmic_bytes(m: int, k: int, n: int) -> float:
    """2-bit weights + fp32 x read by the quantiser + fp32 y + (1 + M) scales."""
    return n * k / 4 + 4 * m * k + 4 * m * n + 4 * (1 + m)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs"), "measured"
    return 6650.0, "fallback"


def profiled_traffic(name: str):
    """DRAM bytes of one launch from the ncu capture summarised next to this name under profiles/ (a small
    JSON written with the capture), or None when no capture of the current kernel has been taken."""
    path = os.path.join(ROOT, "profiles", name + ".json")
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        rec = json.load(f)
    return rec.get("dram_bytes_per_launch"), rec.get("capture")


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
def random_codes(torch, n: int, k: int, seed: int):
    """Canonical packed words of an [n, k] ternary matrix with uniformly random codes in {0, 1, 2} (device)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    shifts = (2 * torch.arange(16, device="cuda", dtype=torch.int32)).view(1, 1, 16)
    words = torch.empty((n, k // 16), dtype=torch.int32, device="cuda")
    chunk = max(1, (1 << 24) // k)
    for r0 in range(0, n, chunk):
        codes = torch.randint(0, 3, (min(chunk, n - r0), k // 16, 16), generator=gen, device="cuda", dtype=torch.int32)
        words[r0:r0 + codes.shape[0]] = (codes << shifts).sum(dim=2, dtype=torch.int32)
    return words


def build_layers(torch, layers: int, n: int, k: int, seed: int, keep_words: bool = False):
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
        out.append((strips, float(scale), words if keep_words else None))
        if not keep_words:
            del words
    return out


class Harness:
    """Timing helpers shared by the sections of the bench (one process per GPU)."""

    def __init__(self, torch, dist, world, rank):
        self.torch, self.dist, self.world, self.rank = torch, dist, world, rank
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        if self.world > 1:
            t = self.torch.tensor([ms], device="cuda")
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed(self, fn, steps: int) -> float:
        """ms for `steps` calls of fn on the current stream, barrier + synchronize on both sides, max over ranks."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record(self.stream)
        for _ in range(steps):
            fn()
        e1.record(self.stream)
        torch.cuda.synchronize()
        ms = self.max_over_ranks(e0.elapsed_time(e1))
        self.barrier()
        return ms

    def graph_of(self, fn, repeats: int = 1):
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=torch.cuda.Stream()):
            for i in range(repeats):
                fn(i)
        return g


def sha256_of(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().cpu().contiguous().numpy().tobytes())
    return h.hexdigest()


def verify_chain_against_oracle(torch, layers, x_host, y_dev):
    """The timed stack, layer by layer on the CPU oracle (exact BLAS form), against the device result: bit for bit."""
    import oracle
    from oracle import fast
    P = oracle.port()
    h = x_host.numpy().astype(np.float32)
    n, k = N_DIM, K_DIM
    for strips, scale, words in layers:
        t = P.unpack_i8(words.cpu().numpy().view(np.uint32).reshape(-1), n, k)
        h, *_ = fast.linear_forward(h, t, np.float32(scale))
        del t
    got = y_dev.cpu().numpy()
    return bool(np.array_equal(got.view(np.uint32), h.view(np.uint32))), float(np.abs(got - h).max())


def gemm_section(H: Harness, L, capi, peak_hbm):
    """Prefill ternary x int8 GEMM (tcgen05): rows of the activation matrix sharded over the ranks."""
    import oracle
    from oracle import fast
    torch = H.torch
    P = oracle.port()
    out = []
    sp = H.stream.cuda_stream
    for (M, K, N, label) in [(8192, 8192, 8192, "sweep M=8192 K=N=8192"), (8192, 16384, 16384, "sweep M=8192 K=N=16384"),
                             (4096, 768, 1536, "D768 prefill 768->1536"), (4096, 1536, 768, "D768 prefill 1536->768")]:
        m_local = M // H.world
        words = random_codes(torch, N, K, seed=N + K)
        w8 = torch.empty((N, K), dtype=torch.int8, device="cuda")
        capi.check(L.tbl_expand_weights_i8(words.data_ptr(), N, K, w8.data_ptr(), sp), "tbl_expand_weights_i8")
        gen = torch.Generator(device="cuda")
        gen.manual_seed(1000 + H.rank)
        x = torch.randn((m_local, K), generator=gen, device="cuda")
        y = torch.empty((m_local, N), device="cuda")
        ws_bytes = L.tbl_linear_workspace_bytes(m_local, K, N)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
        scale = 0.016

        def forward(_i=0):
            capi.check(L.tbl_linear_forward(x.data_ptr(), words.data_ptr(), None, w8.data_ptr(), scale, m_local, K, N, 8, 0,
                                            None, None, y.data_ptr(), ws.data_ptr(), ws_bytes,
                                            torch.cuda.current_stream().cuda_stream), "tbl_linear_forward")

        # verify before timing: 8 activation rows x 256 weight rows against the integer oracle, bit for bit
        forward()
        torch.cuda.synchronize()
        rows = np.linspace(0, m_local - 1, 8).astype(np.int64)
        cols = np.linspace(0, N - 1, 256).astype(np.int64)
        t_sel = P.unpack_i8(words[torch.from_numpy(cols).cuda()].cpu().numpy().view(np.uint32).reshape(-1), cols.size, K)
        want, *_ = fast.linear_forward(x[torch.from_numpy(rows).cuda()].cpu().numpy(), t_sel, np.float32(scale))
        got = y[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
        verified = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))

        # quantiser excluded: tbl_gemm on codes made once
        q = torch.empty((m_local, K), dtype=torch.int8, device="cuda")
        sc = torch.empty(m_local, device="cuda")
        capi.check(L.tbl_quantize_rows(x.data_ptr(), None, m_local, K, 8, 0, 0, q.data_ptr(), sc.data_ptr(), None, sp),
                   "tbl_quantize_rows")

        def gemm_only(_i=0):
            capi.check(L.tbl_gemm(q.data_ptr(), sc.data_ptr(), w8.data_ptr(), scale, None, None, m_local, K, N, y.data_ptr(),
                                  None, torch.cuda.current_stream().cuda_stream), "tbl_gemm")

        reps = 5 if M * K * N > 1 << 36 else 20
        for fn in (forward, gemm_only):
            for _ in range(3):
                fn()
        g_full, g_only = H.graph_of(forward, reps), H.graph_of(gemm_only, reps)
        ms_full = H.timed(g_full.replay, 3) / (3 * reps)
        ms_only = H.timed(g_only.replay, 3) / (3 * reps)
        # the library ceiling beside it: torch._int_mm (cuBLASLt int8) on the same operands
        int_mm_tops = None
        try:
            qa = q if m_local % 8 == 0 else None
            if qa is not None:
                wt = w8.t()
                for _ in range(2):
                    torch._int_mm(qa, wt)
                ms_lib = H.timed(lambda: torch._int_mm(qa, wt), 5) / 5
                int_mm_tops = 2.0 * M * N * K / (ms_lib * 1e-3) / 1e12
        except Exception:
            int_mm_tops = None
        ops = 2.0 * M * N * K
        bytes_ = N * K + M * K * 4 + M * N * 4              # int8 weights + fp32 x + fp32 y
        floor_ms = max(ops / (INT8_DENSE_PEAK_TOPS * 1e12), bytes_ / (peak_hbm * 1e9)) * 1e3 / H.world
        rec = {"shape": label, "M": M, "K": K, "N": N, "rows_per_gpu": m_local, "verified_vs_oracle": verified,
               "us": ms_full * 1e3, "tops": ops / (ms_full * 1e-3) / 1e12,
               "us_gemm_only": ms_only * 1e3, "tops_gemm_only": ops / (ms_only * 1e-3) / 1e12,
               "roofline": {"bound": "tensor" if ops / (INT8_DENSE_PEAK_TOPS * 1e12) > bytes_ / (peak_hbm * 1e9) else "hbm",
                            "attainable_us": floor_ms * 1e3, "frac": floor_ms / ms_only,
                            "frac_of_int8_peak": ops / (ms_only * 1e-3) / 1e12 / (INT8_DENSE_PEAK_TOPS * H.world),
                            "peak_tops": INT8_DENSE_PEAK_TOPS, "peak_kind": "nominal dense int8"},
               "torch_int_mm_tops": int_mm_tops,
               "frac_of_torch_int_mm": (ops / (ms_only * 1e-3) / 1e12 / int_mm_tops) if int_mm_tops else None}
        out.append(rec)
        del words, w8, x, y, q, g_full, g_only
        torch.cuda.empty_cache()
    return out


def decode_section(H: Harness, steps: int):
    """One full decode step of the D768 / 16-block hybrid per sequence; sequences sharded over the ranks."""
    import oracle
    from oracle.decode import PortDecoder
    from reimagined_b200 import capi
    from reimagined_b200.decode import D768_L16, DecodeEngine, synthetic_params
    torch = H.torch
    params = synthetic_params(D768_L16, seed=1)
    out = []
    context = 512
    for batch in (1, 8, 64):
        local = batch // H.world if batch >= H.world else (batch if H.rank == 0 else 0)
        rec = {"batch": batch, "sequences_per_gpu": batch // H.world if batch >= H.world else f"{batch} on rank 0",
               "context_tokens": context}
        us = 0.0
        if local > 0:
            eng = DecodeEngine(params, batch=local, capacity=context + steps + 8)
            gen = torch.Generator().manual_seed(batch)
            draw = lambda: torch.randint(0, D768_L16["vocab_size"], (local,), generator=gen, dtype=torch.int32).cuda()
            first = draw()
            logits = eng.step(first).clone()
            if batch == 1 and H.rank == 0:
                # verify before timing: the same first token through the CPU oracle's decode step
                _, want = PortDecoder(params, rows=1, capacity=4).step(first.cpu().numpy())
                got = logits.cpu().numpy()
                rec["verified_vs_oracle"] = bool(np.abs(got - want).max() <= 2e-3 * np.abs(want).max())
                rec["max_rel_err_vs_oracle"] = float(np.abs(got - want).max() / np.abs(want).max())
            rec["kernel_launches_per_step"] = eng.capture()
            for _ in range(context - 1):
                eng.step(draw())
            ids = [draw() for _ in range(steps)]
            torch.cuda.synchronize()
            it = iter(ids)
            ms = H.timed(lambda: eng.step(next(it)), steps)
            us = ms * 1e3 / steps
            rec["device_status"] = capi.lib().tbl_device_status(H.stream.cuda_stream)
            rec["packed_mb"] = round(eng.ternary_weights / 4 / 1e6, 2)
            del eng
        else:
            ms = H.timed(lambda: None, steps)
            us = ms * 1e3 / steps
        rec["us_per_step"] = us
        rec["tokens_per_s"] = batch / us * 1e6
        out.append(rec)
        torch.cuda.empty_cache()
    return out


def colsplit_section(H: Harness, L, capi, layers):
    """The 16384-wide layer split by output columns over the ranks, two ways: (1) each rank's linear writes its
    [M, N/g] block into its slot of the gather buffer, one in-place NCCL all-gather, one re-tile pass over local
    memory; (2) fused: the GEMM epilogue stores every tile into all ranks' copies of the output over NVLink
    (tbl_linear_forward_scatter), then one barrier across the ranks."""
    torch, dist = H.torch, H.dist
    from reimagined_b200 import sharding
    g, r = H.world, H.rank
    n, k = N_DIM, K_DIM
    n_local = n // g
    strips_full, scale, words = layers[0]
    sp = H.stream.cuda_stream
    shard_words = words[r * n_local:(r + 1) * n_local].contiguous()
    out = []
    for M in (128, 8192):
        gen = torch.Generator(device="cuda")
        gen.manual_seed(4242)                       # x is replicated: same on every rank
        x = torch.randn((M, k), generator=gen, device="cuda")
        w8 = torch.empty((n_local, k), dtype=torch.int8, device="cuda")
        capi.check(L.tbl_expand_weights_i8(shard_words.data_ptr(), n_local, k, w8.data_ptr(), sp), "tbl_expand_weights_i8")
        stacked = sharding.gather_buffer(M, n_local, g)
        y = torch.empty((M, n), device="cuda")
        ws_bytes = L.tbl_linear_workspace_bytes(M, k, n_local)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")

        def compute():
            capi.check(L.tbl_linear_forward(x.data_ptr(), shard_words.data_ptr(), None, w8.data_ptr(), scale, M, k, n_local, 8, 0,
                                            None, None, stacked[r].data_ptr(), ws.data_ptr(), ws_bytes,
                                            torch.cuda.current_stream().cuda_stream), "tbl_linear_forward")

        gather = lambda: sharding.gather_columns_inplace(stacked, r)
        retile = lambda: sharding.retile(stacked, y)
        for _ in range(3):
            compute(); gather(); retile()
        reps = 5
        ms_compute = H.timed(compute, reps) / reps
        ms_gather = H.timed(gather, reps) / reps
        ms_retile = H.timed(retile, reps) / reps
        ms_total = H.timed(lambda: (compute(), gather(), retile()), reps) / reps
        # the unsharded layer on one GPU (every rank runs it; the maximum is taken): strong-scaling reference and
        # bit-exact check of the gathered result on sampled rows
        w8_full = torch.empty((n, k), dtype=torch.int8, device="cuda")
        capi.check(L.tbl_expand_weights_i8(words.data_ptr(), n, k, w8_full.data_ptr(), sp), "tbl_expand_weights_i8")
        y_full = torch.empty((M, n), device="cuda")
        ws_full = torch.empty(max(L.tbl_linear_workspace_bytes(M, k, n), 256), dtype=torch.uint8, device="cuda")

        def unsharded():
            capi.check(L.tbl_linear_forward(x.data_ptr(), words.data_ptr(), None, w8_full.data_ptr(), scale, M, k, n, 8, 0, None,
                                            None, y_full.data_ptr(), ws_full.data_ptr(), ws_full.numel(),
                                            torch.cuda.current_stream().cuda_stream), "tbl_linear_forward")

        for _ in range(2):
            unsharded()
        ms_one = H.timed(unsharded, reps) / reps
        rows = torch.linspace(0, M - 1, 16).long().cuda()
        same = bool(torch.equal(y[rows], y_full[rows]))
        # (2) the exchange fused into the GEMM epilogue
        fused = None
        try:
            import ctypes
            peer = sharding.PeerOutput(M, n)
            order = [(r + 1 + i) % g for i in range(g)]
            dests = (ctypes.c_void_p * g)(*[peer.pointers[q] for q in order])

            def fused_step():
                capi.check(L.tbl_linear_forward_scatter(x.data_ptr(), w8.data_ptr(), scale, M, k, n_local, 8, 0, None, None, dests,
                                                        g, n, n_local * r, ws.data_ptr(), ws_bytes,
                                                        torch.cuda.current_stream().cuda_stream), "tbl_linear_forward_scatter")
                peer.barrier()

            for _ in range(3):
                fused_step()
            ms_fused = H.timed(fused_step, reps) / reps
            fused_same = bool(torch.equal(peer.tensor[rows], y_full[rows]))
            sent = M * n_local * 4 * (g - 1)
            fused = {"total_us": ms_fused * 1e3, "matches_unsharded_bit_for_bit": fused_same,
                     "bytes_stored_to_peers_per_gpu": sent, "nvlink_out_gbs_per_gpu": sent / (ms_fused * 1e-3) / 1e9,
                     "speedup_vs_one_gpu": ms_one / ms_fused, "strong_scaling_efficiency": ms_one / ms_fused / g,
                     "speedup_vs_all_gather_path": ms_total / ms_fused}
            del peer
        except Exception as exc:      # no peer mapping on this box: the all-gather path above stands alone
            fused = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        gathered_bytes = M * n * 4
        out.append({"M": M, "K": k, "N": n, "columns_per_gpu": n_local, "matches_unsharded_bit_for_bit": same,
                    "compute_us": ms_compute * 1e3, "all_gather_us": ms_gather * 1e3, "retile_us": ms_retile * 1e3,
                    "total_us": ms_total * 1e3, "all_gather_bytes": gathered_bytes,
                    "all_gather_bus_gbs": gathered_bytes * (g - 1) / g / (ms_gather * 1e-3) / 1e9,
                    "all_gather_share_of_total": ms_gather / ms_total,
                    "unsharded_one_gpu_us": ms_one * 1e3, "speedup_vs_one_gpu": ms_one / ms_total,
                    "strong_scaling_efficiency": ms_one / ms_total / g, "fused_epilogue_exchange": fused})
        del w8, w8_full, stacked, y, y_full, x
        torch.cuda.empty_cache()
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
    # peer mappings of the column-split output are plain (no NVLink multicast object is bound to them)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the ternary linear path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    H = Harness(torch, dist, world, rank)
    peak, peak_kind = measured_peaks()
    warmup = max(3, args.warmup)

    m, k, n = ROWS, K_DIM, N_DIM
    layers = build_layers(torch, LAYERS, n, k, seed=5, keep_words=True)
    x_host = torch.randn((m, k), generator=torch.Generator().manual_seed(100 + rank)).pin_memory()
    x_dev = x_host.cuda()
    y_dev = torch.empty((m, n), device="cuda")
    y_host = torch.empty((m, n)).pin_memory()
    views = (capi.LinearView * LAYERS)()
    for v, (strips, scale, words) in zip(views, layers):
        v.weight, v.magnitude, v.bias, v.w_i8 = None, None, None, None
        v.packed, v.strips = words.data_ptr(), strips.data_ptr()
        v.inputs, v.outputs, v.activation_bits, v.rms_input, v.weight_scale = k, n, 8, 0, scale
    ws_bytes = L.tbl_chain_workspace_bytes(views, LAYERS, m)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")

    def chain(src, dst):
        capi.check(L.tbl_chain_forward(views, LAYERS, None, src.data_ptr(), m, 0, dst.data_ptr(), ws.data_ptr(), ws_bytes,
                                       torch.cuda.current_stream().cuda_stream), "tbl_chain_forward")

    # ---- verify before timing, and fingerprint what is timed ----
    for _ in range(warmup):
        chain(x_dev, y_dev)
    torch.cuda.synchronize()
    verified, max_diff = (None, None)
    digests = None
    if rank == 0:
        verified, max_diff = verify_chain_against_oracle(torch, layers, x_host, y_dev)
        digests = {"input_sha256": sha256_of(x_host), "weights_sha256": sha256_of(*[w for _, _, w in layers])}
    expected = y_dev.clone()

    # ---- the step as a decode loop replays it: one graph node per launch ----
    count0 = L.tbl_launch_count()
    g_resident = H.graph_of(lambda _i: chain(x_dev, y_dev))
    launches_per_step = L.tbl_launch_count() - count0
    x_stage = torch.empty_like(x_dev)
    g_e2e = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_e2e, stream=torch.cuda.Stream()):
        x_stage.copy_(x_host, non_blocking=True)          # pinned host -> device, every step
        # device -> pinned host, every step: the last layer's epilogue stores its outputs straight into the
        # pinned (device-mapped) result buffer, so the read-back travels with the kernel instead of after it
        chain(x_stage, y_host)
    for g in (g_resident, g_e2e):
        for _ in range(warmup):
            g.replay()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = H.timed(g_resident.replay, args.steps)
    ms_e2e = H.timed(g_e2e.replay, args.steps)
    # the timed regions last milliseconds, nvidia-smi samples every 100 ms: keep the same replay running for
    # about 0.6 s more (untimed) so that the clock record is taken under this load
    probe_steps = max(args.steps, int(600.0 / max(ms / args.steps, 1e-3)))
    H.timed(g_resident.replay, probe_steps)
    clocks = sampler.stop()
    clocks["sampled_over"] = f"the timed regions plus {probe_steps} more untimed steps of the same replay"
    torch.cuda.synchronize()
    e2e_matches = bool(torch.equal(y_host, expected.cpu())) and bool(torch.equal(y_dev, expected))
    y_host.zero_()
    g_e2e.replay()                                       # once more into a cleared buffer: the result really arrives
    torch.cuda.synchronize()
    e2e_matches = e2e_matches and bool(torch.equal(y_host, expected.cpu()))
    status = L.tbl_device_status(H.stream.cuda_stream)

    step_bytes = LAYERS * algorithmic_bytes(m, k, n)
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = world * step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    # dominant kernel: the step is one launch of the persistent chain kernel (plus a 24 KB memset node that re-arms
    # its barrier words), so the CUDA-event time of the region divided by the launches in it is its duration
    kernel_ms = ms / args.steps
    achieved = step_bytes / (kernel_ms * 1e-3) / 1e9
    per_layer_traffic, capture = profiled_traffic("gemv_chain_16384x16384_m1")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x ternary(2-bit) -> int32", "data": "synthetic",
        "config": {"workload": f"C5 ternary decode GEMV K=N={k}, M={m} row per GPU, {LAYERS} chained layers per step "
                               f"({LAYERS * n * k // 4 >> 20} MiB of packed weights per step > 126 MB L2: inputs larger than L2)",
                   "parallelism": f"rows sharded over {world} GPU(s), weights replicated, no collective",
                   "launch": "one request at a time; a step is one persistent cooperative launch over the whole stack "
                             "(tbl_chain_forward), replayed from a CUDA graph"},
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": m * k * 4, "d2h_bytes_per_step": m * n * 4,
                "ms_per_step": ms_e2e / args.steps, "matches_resident_result": e2e_matches},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "gemv_chain_kernel (persistent, quantiser fused, one launch per step)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "kernel_us": kernel_ms * 1e3, "layers_per_launch": LAYERS,
                     "us_per_layer": kernel_ms * 1e3 / LAYERS,
                     "algorithmic_bytes_per_launch": step_bytes,
                     "traffic": per_layer_traffic * LAYERS if per_layer_traffic else None,
                     "traffic_capture": capture},
        "verified_vs_oracle_before_timing": verified, "max_abs_diff_vs_oracle": max_diff,
        "device_status": status,
    }
    if digests:
        line.update(digests)
    del g_resident, g_e2e
    torch.cuda.empty_cache()

    if not args.headline_only:
        if world > 1:
            line["colsplit"] = colsplit_section(H, L, capi, layers)
        del layers, views
        torch.cuda.empty_cache()
        line["gemm"] = gemm_section(H, L, capi, peak)
        line["decode"] = decode_section(H, min(args.steps, 50))

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the gemm / decode / colsplit sections (used for profiler captures of the headline kernel)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
