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
    ap.add_argument("--canonical", action="store_true",
                    help="give the call only the canonical 2-bit words (no strip copy, no int8 expansion)")
    ap.add_argument("--moe", action="store_true",
                    help="time tbl_moe_forward instead: --m tokens, --k model width, --n expert hidden width")
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--no-i8", action="store_true", help="MoE: views without the int8 expansion (strip GEMV path)")
    ap.add_argument("--norm", action="store_true",
                    help="time tbl_row_norm instead: --m rows of --k elements (RMSNorm x weight)")
    ap.add_argument("--gated", action="store_true", help="row norm: SiLU gate first (the Mamba-2 epilogue)")
    ap.add_argument("--codes", choices=["no", "also", "only"], default="no",
                    help="row norm: also emit the int8 codes of the result, or only them (no fp32 store)")
    ap.add_argument("--chain", type=int, default=0,
                    help="time tbl_chain_forward instead: a stack of this many --n x --k layers (n == k) on --m rows")
    args = ap.parse_args()
    if args.chain:
        return chain(args)
    if args.moe:
        return moe(args)
    if args.norm:
        return norm(args)

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
    buffers = max(2, min(24, int(400e6 // (packed * (1 if m <= 64 or args.canonical else 4)))))
    weights = []
    for b in range(buffers):
        # random codes in {0, 1, 2} (two bits each, never 3)
        words = torch.randint(0, 2 ** 31 - 1, (n * k // 16,), dtype=torch.int32, device="cuda") & 0x2AAAAAAA
        if args.canonical:
            weights.append((words, None, None))
        elif m <= 64 and k % 256 == 0:
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
    algorithmic = packed * (1 if m <= 64 or args.canonical else 4) + 4 * m * k + 4 * m * n + 4 * (1 + m)
    status = L.tbl_device_status(stream)
    print(json.dumps({"m": m, "n": n, "k": k, "us_per_call": round(us, 2), "gb_per_s": round(algorithmic / us / 1e3, 1),
                      "tops": round(2.0 * m * n * k / us / 1e6, 1), "weight_buffers": buffers,
                      "graph": not args.no_graph, "device_status": status}))


def chain(args) -> None:
    """A stack of square ternary layers through tbl_chain_forward (one persistent launch when the shape allows it)."""
    import torch
    from . import capi

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the ternary linear path has no CPU fallback")
    L = capi.lib()
    torch.cuda.set_device(0)
    m, n, k, layers = args.m, args.n, args.k, args.chain
    if n != k or k % 16:
        raise SystemExit("--chain needs n == k, a multiple of 16")
    stream = torch.cuda.current_stream().cuda_stream
    keep = []
    views = (capi.LinearView * layers)()
    for v in views:
        words = torch.randint(0, 2 ** 31 - 1, (n * k // 16,), dtype=torch.int32, device="cuda") & 0x2AAAAAAA
        strips = None
        if k % 256 == 0:
            strips = torch.empty(L.tbl_strip_bytes(n, k), dtype=torch.uint8, device="cuda")
            capi.check(L.tbl_relayout_strips(words.data_ptr(), n, k, strips.data_ptr(), stream), "tbl_relayout_strips")
        keep.extend([words, strips])
        v.weight, v.magnitude, v.bias, v.w_i8 = None, None, None, None
        v.packed = words.data_ptr()
        v.strips = None if strips is None else strips.data_ptr()
        v.inputs, v.outputs, v.activation_bits, v.rms_input, v.weight_scale = k, n, 8, 0, 0.016
    x = torch.randn((m, k), device="cuda")
    y = torch.empty((m, n), device="cuda")
    ws_bytes = L.tbl_chain_workspace_bytes(views, layers, m)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")

    def call() -> None:
        capi.check(L.tbl_chain_forward(views, layers, None, x.data_ptr(), m, 0, y.data_ptr(), ws.data_ptr(), ws_bytes,
                                       torch.cuda.current_stream().cuda_stream), "tbl_chain_forward")

    for _ in range(args.warmup):
        call()
    torch.cuda.synchronize()
    before = L.tbl_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.no_graph:
        e0.record()
        for _ in range(args.iters):
            call()
        e1.record()
        launches = (L.tbl_launch_count() - before) // args.iters
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            call()
        launches = L.tbl_launch_count() - before
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            graph.replay()
        e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.iters
    algorithmic = layers * (n * k // 4 + 4 * m * k + 4 * m * n + 4 * (1 + m))
    print(json.dumps({"chain": True, "layers": layers, "m": m, "n": n, "k": k, "us_per_stack": round(us, 2),
                      "us_per_layer": round(us / layers, 2), "gb_per_s": round(algorithmic / us / 1e3, 1),
                      "kernel_launches": int(launches), "graph": not args.no_graph,
                      "device_status": L.tbl_device_status(stream)}))


def norm(args) -> None:
    """Row norm (optionally gated, optionally fused with the quantiser) on rotating buffers larger than L2 in total."""
    import torch
    from . import capi

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the ternary linear path has no CPU fallback")
    L = capi.lib()
    torch.cuda.set_device(0)
    rows, dim = args.m, args.k
    want_out, want_q = args.codes != "only", args.codes != "no"
    in_bytes = rows * dim * 4 * (2 if args.gated else 1)
    out_bytes = (rows * dim * 4 if want_out else 0) + (rows * dim + 8 * rows if want_q else 0)
    buffers = max(2, min(24, int(400e6 // (in_bytes + out_bytes)) + 1))
    sets = []
    for _ in range(buffers):
        sets.append((torch.randn((rows, dim), device="cuda"),
                     torch.randn((rows, dim), device="cuda") if args.gated else None,
                     torch.empty((rows, dim), device="cuda") if want_out else None,
                     torch.empty((rows, dim), dtype=torch.int8, device="cuda") if want_q else None))
    weight = torch.rand(dim, device="cuda") + 0.5
    scales = torch.empty(rows, device="cuda")
    sums = torch.empty(rows, dtype=torch.int32, device="cuda")

    def ptr(t):
        return None if t is None else t.data_ptr()

    def call(i: int) -> None:
        value, gate, out, q = sets[i % buffers]
        capi.check(L.tbl_row_norm(ptr(value), ptr(gate), ptr(weight), rows, dim, 1e-5, ptr(out), 8, ptr(q),
                                  ptr(scales) if want_q else None, ptr(sums) if want_q else None,
                                  torch.cuda.current_stream().cuda_stream), "tbl_row_norm")

    for i in range(args.warmup):
        call(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.iters):
            call(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.iters
    algorithmic = in_bytes + out_bytes + 4 * dim
    print(json.dumps({"row_norm": True, "rows": rows, "dim": dim, "gated": args.gated, "codes": args.codes,
                      "us_per_call": round(us, 2), "gb_per_s": round(algorithmic / us / 1e3, 1),
                      "algorithmic_mb": round(algorithmic / 1e6, 2), "buffers": buffers,
                      "device_status": L.tbl_device_status(torch.cuda.current_stream().cuda_stream)}))


def moe(args) -> None:
    """Expert FFN of a mixture-of-experts block: tokens x [m, k], E experts up k->n, squared ReLU, down n->k, top-k routing."""
    import torch
    from . import capi

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the ternary linear path has no CPU fallback")
    L = capi.lib()
    torch.cuda.set_device(0)
    rows, dim, hidden, E, topk = args.m, args.k, args.n, args.experts, args.topk
    stream = torch.cuda.current_stream().cuda_stream
    keep = []

    def make_view(n: int, k: int) -> capi.LinearView:
        words = torch.randint(0, 2 ** 31 - 1, (n * k // 16,), dtype=torch.int32, device="cuda") & 0x2AAAAAAA
        strips = None
        if k % 256 == 0:
            strips = torch.empty(L.tbl_strip_bytes(n, k), dtype=torch.uint8, device="cuda")
            capi.check(L.tbl_relayout_strips(words.data_ptr(), n, k, strips.data_ptr(), stream), "tbl_relayout_strips")
        w8 = torch.empty((n, k), dtype=torch.int8, device="cuda")      # for the grouped tensor-core GEMM
        capi.check(L.tbl_expand_weights_i8(words.data_ptr(), n, k, w8.data_ptr(), stream), "tbl_expand_weights_i8")
        keep.extend([words, strips, w8])
        v = capi.LinearView()
        v.weight, v.magnitude, v.bias = None, None, None
        v.packed = words.data_ptr()
        v.strips = None if strips is None else strips.data_ptr()
        v.w_i8 = None if args.no_i8 else w8.data_ptr()
        v.inputs, v.outputs, v.activation_bits, v.rms_input, v.weight_scale = k, n, 8, 1, 0.016
        return v

    views = [make_view(hidden, dim) for _ in range(E)] + [make_view(dim, hidden) for _ in range(E)]
    arr = (capi.LinearView * (2 * E))(*views)
    torch.manual_seed(0)          # the same routing every run
    x = torch.randn((rows, dim), device="cuda")
    # top-k routing weights: k distinct experts per token, weights summing to one
    scores = torch.rand((rows, E), device="cuda")
    top = scores.topk(topk, dim=1)
    routing = torch.zeros((rows, E), device="cuda")
    routing.scatter_(1, top.indices, top.values / top.values.sum(dim=1, keepdim=True))
    out = torch.empty((rows, dim), device="cuda")
    ws_bytes = L.tbl_moe_workspace_bytes(rows, dim, hidden, E, topk)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")

    def call() -> None:
        capi.check(L.tbl_moe_forward(arr, routing.data_ptr(), x.data_ptr(), rows, dim, hidden, E, topk, 1, 0,
                                     out.data_ptr(), ws.data_ptr(), ws_bytes, torch.cuda.current_stream().cuda_stream),
                   "tbl_moe_forward")

    for _ in range(args.warmup):
        call()
    torch.cuda.synchronize()
    before = L.tbl_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.no_graph:
        e0.record()
        for _ in range(args.iters):
            call()
        e1.record()
        launches = (L.tbl_launch_count() - before) // args.iters
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            call()
        launches = L.tbl_launch_count() - before
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            graph.replay()
        e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.iters
    active = int((routing.sum(dim=0) > 0).sum().item())
    packed_bytes = active * 2 * dim * hidden // 4
    ops = 2.0 * rows * topk * 2 * dim * hidden
    print(json.dumps({"moe": True, "tokens": rows, "dim": dim, "hidden": hidden, "experts": E, "topk": topk,
                      "active_experts": active, "us_per_call": round(us, 1), "kernel_launches": int(launches),
                      "packed_mb": round(packed_bytes / 1e6, 1), "packed_gb_per_s": round(packed_bytes / us / 1e3, 1),
                      "tops": round(ops / us / 1e6, 1), "device_status": L.tbl_device_status(stream)}))


if __name__ == "__main__":
    main()
