"""Time `tbl_linear_forward` on one synthetic shape: `python -m reimagined_b200.shapes --m 8 --n 4096 --k 4096`.

The decode path (M <= 64) runs on strip-major weights, the prefill path (M > 64) on the int8 expansion,
exactly as a caller of the C ABI would set them up.  Several weight buffers are rotated so that a call never
finds its weights in L2.  Prints one JSON line; also the committed way to put a given shape under a profiler.
"""
from __future__ import annotations

import argparse
import json


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--k", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true", help="launch from the stream instead of replaying a CUDA graph")
    args = ap.parse_args()

    import torch
    from . import capi

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the ternary linear path has no CPU fallback")
    L = capi.lib()
    torch.cuda.set_device(0)
    m, n, k = args.m, args.n, args.k
    if k % 16:
        raise SystemExit("K must be a multiple of 16")
    stream = torch.cuda.current_stream().cuda_stream
    packed = n * k // 4
    buffers = max(2, min(24, int(400e6 // (packed * (1 if m <= 64 else 4)))))
    weights = []
    for b in range(buffers):
        # random codes in {0, 1, 2} (two bits each, never 3)
        words = torch.randint(0, 2 ** 31 - 1, (n * k // 16,), dtype=torch.int32, device="cuda") & 0x2AAAAAAA
        if m <= 64 and k % 256 == 0:
            dev = torch.empty(L.tbl_strip_bytes(n, k), dtype=torch.uint8, device="cuda")
            capi.check(L.tbl_relayout_strips(words.data_ptr(), n, k, dev.data_ptr(), stream), "tbl_relayout_strips")
            weights.append((None, dev, None))
        elif m > 64:
            dev = torch.empty((n, k), dtype=torch.int8, device="cuda")
            capi.check(L.tbl_expand_weights_i8(words.data_ptr(), n, k, dev.data_ptr(), stream), "tbl_expand_weights_i8")
            weights.append((words, None, dev))
        else:
            weights.append((words, None, None))
    x = torch.randn((m, k), device="cuda")
    y = torch.empty((m, n), device="cuda")
    ws_bytes = L.tbl_linear_workspace_bytes(m, k, n)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")

    def call(i: int) -> None:
        words, strips, w8 = weights[i % buffers]
        capi.check(L.tbl_linear_forward(x.data_ptr(), None if words is None else words.data_ptr(),
                                        None if strips is None else strips.data_ptr(),
                                        None if w8 is None else w8.data_ptr(), 0.016, m, k, n, 8, 0, None, None,
                                        y.data_ptr(), ws.data_ptr(), ws_bytes, torch.cuda.current_stream().cuda_stream),
                   "tbl_linear_forward")

    for i in range(args.warmup):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.no_graph:
        e0.record()
        for i in range(args.iters):
            call(i)
        e1.record()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.iters):
                call(i)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.iters
    algorithmic = packed * (1 if m <= 64 else 4) + 4 * m * k + 4 * m * n + 4 * (1 + m)
    status = L.tbl_device_status(stream)
    print(json.dumps({"m": m, "n": n, "k": k, "us_per_call": round(us, 2), "gb_per_s": round(algorithmic / us / 1e3, 1),
                      "tops": round(2.0 * m * n * k / us / 1e6, 1), "weight_buffers": buffers,
                      "graph": not args.no_graph, "device_status": status}))


if __name__ == "__main__":
    main()
