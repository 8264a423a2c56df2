"""The 107 ternary linears of one decode step of the D768 / 16-layer hybrid, chained and replayed from a CUDA graph:
`python -m reimagined_b200.decode_step --batch 1`.

Shapes follow the reference's model (d_model 768, 16 blocks each with a Mamba-2 branch: x/z projections
768->1536, B/C 768->16, dt 768->24, out 1536->768; blocks 8 and 16 add attention q 768->768, kv 768->1536,
out 768->768 and an FFN 768->3072->768 with squared ReLU; LM head 768->32000): 96.04 M ternary weights,
24.0 MB packed.  Only the linears run -- the state-space scan, attention over the KV cache, norms and gates
between them are not part of this library -- so the figure is the linear path's share of a token, an upper
bound on tokens/s, with real data dependencies (every linear consumes an earlier linear's output).
Projections that share an input go through `tbl_grouped_forward_rows` (one launch for five up to batch 8).
With `--norms` the norms that feed those linears run too (`tbl_row_norm`): the block RMSNorm x weight before each
projection group, attention group and FFN, the final norm before the LM head, and the Mamba-2 epilogue -- SiLU
gate, RMSNorm x weight, one launch -- before the out-projection (the x branch stands in for the scan's output,
the z branch is the gate).  The norms hand fp32 rows to the linears: at decode sizes the linear quantises in its
own prologue at no extra launch, so the norm's int8-code output (made for the prefill GEMM) would only add one.
Weights are synthetic (random codes).  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json

D, EXPAND, STATE, HEADS, FFN, VOCAB, LAYERS = 768, 2, 16, 24, 3072, 32000, 16
HYBRID_LAYERS = (7, 15)     # 0-based: the 8th and 16th blocks carry attention + FFN


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--norms", action="store_true", help="also run the norms either side of the linears")
    args = ap.parse_args()

    import torch
    from . import capi

    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the ternary linear path has no CPU fallback")
    L = capi.lib()
    torch.cuda.set_device(0)
    B = args.batch
    stream = torch.cuda.current_stream().cuda_stream
    keep = []          # device buffers referenced by raw pointers below
    total_weights = 0

    def make_linear(n: int, k: int, squared_relu: bool = False):
        nonlocal total_weights
        total_weights += n * k
        words = torch.randint(0, 2 ** 31 - 1, (n * k // 16,), dtype=torch.int32, device="cuda") & 0x2AAAAAAA
        strips = torch.empty(L.tbl_strip_bytes(n, k), dtype=torch.uint8, device="cuda")
        capi.check(L.tbl_relayout_strips(words.data_ptr(), n, k, strips.data_ptr(), stream), "tbl_relayout_strips")
        keep.extend([words, strips])
        return {"n": n, "k": k, "words": words, "strips": strips, "scale": 0.016}

    def view(lin) -> capi.LinearView:
        v = capi.LinearView()
        v.weight = None
        v.packed = lin["words"].data_ptr()
        v.strips = lin["strips"].data_ptr()
        v.magnitude = None
        v.bias = None
        v.inputs, v.outputs = lin["k"], lin["n"]
        v.activation_bits, v.rms_input, v.weight_scale = 8, 0, lin["scale"]
        return v

    inner = D * EXPAND
    blocks = []
    for layer in range(LAYERS):
        blk = {"proj": [make_linear(inner, D), make_linear(inner, D), make_linear(STATE, D), make_linear(STATE, D),
                        make_linear(HEADS, D)],
               "out": make_linear(D, inner)}
        if layer in HYBRID_LAYERS:
            blk["attn"] = [make_linear(D, D), make_linear(2 * D, D)]
            blk["attn_out"] = make_linear(D, D)
            blk["ffn_up"] = make_linear(FFN, D)
            blk["ffn_down"] = make_linear(D, FFN)
        blocks.append(blk)
    head = make_linear(VOCAB, D)

    ws_bytes = max(L.tbl_linear_workspace_bytes(B, FFN, VOCAB), L.tbl_grouped_rows_workspace_bytes(5, min(B, 64), D))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    hidden = [torch.randn((B, D), device="cuda"), torch.empty((B, D), device="cuda")]
    # slot i of a group buffer receives linear i's [B, n] output, contiguous with row pitch n
    proj_out = torch.empty((5, B * inner), device="cuda")
    attn_out = torch.empty((2, B * 2 * D), device="cuda")
    ffn_mid = torch.empty((B, FFN), device="cuda")
    logits = torch.empty((B, VOCAB), device="cuda")
    # --norms: per-block weights of the norms, the normalised row and the gated epilogue's output
    block_norm_w = [torch.rand(D, device="cuda") + 0.5 for _ in range(LAYERS + 2 * len(HYBRID_LAYERS) + 1)]
    gated_norm_w = [torch.rand(inner, device="cuda") + 0.5 for _ in range(LAYERS)]
    normed = torch.empty((B, D), device="cuda")
    gated_out = torch.empty((B, inner), device="cuda")

    def linear(lin, x_ptr: int, y_ptr: int) -> None:
        capi.check(L.tbl_linear_forward(x_ptr, None, lin["strips"].data_ptr(), None, lin["scale"], B, lin["k"],
                                        lin["n"], 8, 0, None, None, y_ptr, ws.data_ptr(), ws_bytes,
                                        torch.cuda.current_stream().cuda_stream), "tbl_linear_forward")

    def group(lins, x, out) -> None:
        """Several linears on the same input rows: one grouped call (up to 64 rows), else one call each."""
        if B <= 64:
            arr = (capi.LinearView * len(lins))(*[view(l) for l in lins])
            capi.check(L.tbl_grouped_forward_rows(arr, len(lins), x.data_ptr(), B, out.data_ptr(), out.shape[1], 0,
                                                  ws.data_ptr(), ws_bytes, torch.cuda.current_stream().cuda_stream),
                       "tbl_grouped_forward_rows")
        else:
            for i, l in enumerate(lins):
                linear(l, x.data_ptr(), out[i].data_ptr())

    def block_norm(x, weight):
        """RMSNorm x weight of the residual stream into `normed` (identity without --norms)."""
        if not args.norms:
            return x
        capi.check(L.tbl_row_norm(x.data_ptr(), None, weight.data_ptr(), B, D, 1e-5, normed.data_ptr(), 8, None, None,
                                  None, torch.cuda.current_stream().cuda_stream), "tbl_row_norm")
        return normed

    def mamba_epilogue(blk, weight, y_ptr: int) -> None:
        """x branch (gated by the z branch and normalised with --norms) -> out projection."""
        if not args.norms:
            return linear(blk["out"], proj_out[0].data_ptr(), y_ptr)
        capi.check(L.tbl_row_norm(proj_out[0].data_ptr(), proj_out[1].data_ptr(), weight.data_ptr(), B, inner, 1e-5,
                                  gated_out.data_ptr(), 8, None, None, None, torch.cuda.current_stream().cuda_stream),
                   "tbl_row_norm")
        linear(blk["out"], gated_out.data_ptr(), y_ptr)

    def step() -> None:
        cur = 0
        norm_w = iter(block_norm_w)
        for layer, blk in enumerate(blocks):
            group(blk["proj"], block_norm(hidden[cur], next(norm_w)), proj_out)
            mamba_epilogue(blk, gated_norm_w[layer], hidden[cur ^ 1].data_ptr())
            cur ^= 1
            if "attn" in blk:
                group(blk["attn"], block_norm(hidden[cur], next(norm_w)), attn_out)
                linear(blk["attn_out"], attn_out[0].data_ptr(), hidden[cur ^ 1].data_ptr())
                cur ^= 1
                linear(blk["ffn_up"], block_norm(hidden[cur], next(norm_w)).data_ptr(), ffn_mid.data_ptr())
                linear(blk["ffn_down"], ffn_mid.data_ptr(), hidden[cur ^ 1].data_ptr())
                cur ^= 1
        linear(head, block_norm(hidden[cur], next(norm_w)).data_ptr(), logits.data_ptr())

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    before = L.tbl_launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    launches = L.tbl_launch_count() - before
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.iters
    packed_mb = total_weights / 4 / 1e6
    workload = "D768/L16 decode step, the 107 ternary linears" + (" and the 37 norms that feed them" if args.norms
                                                                       else " only")
    print(json.dumps({"workload": workload, "batch": B, "linears": 107, "norms": 37 if args.norms else 0, "kernel_launches_per_step": int(launches), "us_per_step": round(us, 1),
                      "tokens_per_s_linears_only": round(B / us * 1e6, 1), "ternary_weights": total_weights,
                      "packed_mb": round(packed_mb, 2), "packed_gb_per_s": round(packed_mb / us * 1e3, 1),
                      "device_status": L.tbl_device_status(stream)}))


if __name__ == "__main__":
    main()
