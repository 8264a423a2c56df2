"""Generates tests/golden/*.npz by running the REFERENCE's own C++ (oracle/_ref/libnsos_ref.so,
built by oracle/Makefile from the reference checkout) on seeded inputs.

    python tests/golden/make_golden.py [name-prefix]      # only fixtures whose name starts with the prefix

Only runs where the reference checkout is available; the produced fixtures are committed and are
what the CPU-only and GPU tests compare against on machines without the reference.
Inputs come from numpy's PCG64 (seeded); each fixture stores a SHA-256 of its inputs so a change
of generator would be noticed, plus the inputs themselves when they are small.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def make_inputs(seed, N, K, M, affine):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    mag = (1.0 + 0.25 * rng.standard_normal(N)).astype(np.float32) if affine else None
    bias = (0.1 * rng.standard_normal(N)).astype(np.float32) if affine else None
    return w, x, mag, bias


# name, seed, N, K, M, exact_linear, affine, bits, store_inputs
LINEAR_CASES = [
    ("c1_exact_768", 0, 768, 768, 1, True, False, 8, False),
    ("c1_default_768", 0, 768, 768, 1, False, True, 8, False),
    ("small_33x48_m3", 11, 33, 48, 3, True, False, 8, True),
    ("small_17x1024_m5", 12, 17, 1024, 5, True, False, 8, True),
    ("tail_64x52_m2", 13, 64, 52, 2, True, False, 8, True),
    ("affine_32x64_m8", 14, 32, 64, 8, False, True, 8, True),
    ("bits4_48x256_m4", 15, 48, 256, 4, True, False, 4, True),
    ("bits2_48x256_m4", 16, 48, 256, 4, True, False, 2, True),
    ("mid_96x512_m24", 17, 96, 512, 24, False, True, 8, True),
    ("gemm_160x256_m130", 18, 160, 256, 130, True, False, 8, True),
]


def row_norm_fixtures(R, only):
    """Block norm and gated Mamba-2 epilogue norm from the reference's own Tensor ops (ref_row_norm)."""
    for name, seed, rows, dim, gated, weighted, eps in ROW_NORM_CASES:
        if not name.startswith(only):
            continue
        rng = np.random.default_rng(seed)
        value = rng.standard_normal((rows, dim)).astype(np.float32)
        gate = (2.5 * rng.standard_normal((rows, dim))).astype(np.float32) if gated else None
        weight = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32) if weighted else None
        out = R.row_norm(value, gate, weight, eps)
        rec = dict(seed=seed, eps=np.float32(eps), value=value, out=out)
        if gated:
            rec["gate"] = gate
        if weighted:
            rec["weight"] = weight
        np.savez_compressed(os.path.join(OUT, name + ".npz"), **rec)
        print(name, "out[0,:3]", out[0, :3])


# name, seed, rows, dim, gated, weighted, eps
ROW_NORM_CASES = [
    ("rownorm_block_3x768", 31, 3, 768, False, True, 1e-6),
    ("rownorm_plain_2x50", 32, 2, 50, False, False, 1e-5),
    ("rownorm_gated_4x1536", 33, 4, 1536, True, True, 1e-5),
    ("rownorm_gated_2x33", 34, 2, 33, True, True, 1e-6),
]


TINY_MODEL = dict(num_layers=2, d_model=64, vocab_size=96, n_heads=1, n_kv_heads=1, mamba_d_state=16, mamba_expand=2,
                  mamba_conv_kernel=4, mamba_head_dim=64, mamba_n_groups=1, attention_period=2, attention_slot=1)
TINY_TOKENS = [5, 90, 17, 17, 0, 63, 41, 8]


def model_fixtures(only):
    """From the reference's whole model (oracle/_ref/libnsos_model_ref.so): a two-block hybrid (one Mamba-2 block,
    one Mamba-2 + attention + FFN block) stepped token by token through JambaModel::forward_ids_last, with its
    parameters, the residual stream after every block, its own edge-linear pack, and MoERouter::forward."""
    if not oracle.model_ref_available():
        print("model reference library not built: decode / edge-pack / router fixtures skipped")
        return
    MR = oracle.model_ref()
    if "decode_tiny".startswith(only) or "edge_pack_tiny".startswith(only):
        m = MR.model(TINY_MODEL, seed=11)
        params = m.export()
        twin = MR.model(TINY_MODEL, seed=11)
        logits, hidden = [], []
        for tok in TINY_TOKENS:
            lg = m.step(tok)                       # public API
            hd, lg2 = twin.step_trace(tok)         # block by block on a twin with the same seed
            assert np.array_equal(lg.view(np.uint32), lg2.view(np.uint32))
            logits.append(lg)
            hidden.append(hd)
        rec = {"param:" + k: v for k, v in params.items()}
        rec.update(tokens=np.asarray(TINY_TOKENS, np.int32), logits=np.stack(logits), hidden=np.stack(hidden),
                   cfg=np.asarray([TINY_MODEL[k] for k in oracle.MODEL_CFG_FIELDS], np.int32))
        np.savez_compressed(os.path.join(OUT, "decode_tiny.npz"), **rec)
        print("decode_tiny logits[0,:3]", logits[0][:3], "logits[-1,:3]", logits[-1][:3])
        path = os.path.join(OUT, "edge_pack_tiny.bin")
        m.save_edge_pack(path)
        print("edge_pack_tiny.bin", os.path.getsize(path), "bytes")
        m.close()
        twin.close()
    if "router_".startswith(only[:7]) or not only:
        for name, seed, rows, D, E, k in [("router_40x64_e8_top2", 41, 40, 64, 8, 2), ("router_9x32_e4_top1", 42, 9, 32, 4, 1)]:
            rng = np.random.default_rng(seed)
            x = rng.standard_normal((rows, D)).astype(np.float32)
            x[1] = x[0]                                       # two identical rows
            gate = (rng.standard_normal((E, D)) * 0.02).astype(np.float32)
            gate[1] = gate[0]                                 # a tie between experts 0 and 1 on every row
            lg, w = MR.router(x, gate, k)
            np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, gate=gate, top_k=k, logits=lg, weights=w)
            print(name, "weights[0]", w[0])


def main():
    only = sys.argv[1] if len(sys.argv) > 1 else ""
    model_fixtures(only)
    R = oracle.ref()
    row_norm_fixtures(R, only)
    for name, seed, N, K, M, exact, affine, bits, store in LINEAR_CASES:
        if not name.startswith(only):
            continue
        w, x, mag, bias = make_inputs(seed, N, K, M, affine)
        words, scale = R.pack(w)
        y = R.linear_forward(w, x, exact_linear=exact, magnitude=mag, bias=bias, bits=bits)
        rec = dict(seed=seed, N=N, K=K, M=M, exact_linear=exact, affine=affine, bits=bits,
                   input_sha=sha(w, x), words=words, weight_scale=np.float32(scale), y=y)
        if store:
            rec.update(w=w, x=x)
        if affine:
            rec.update(magnitude=mag, bias=bias)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), **rec)
        print(name, "scale", scale, "y[0,:3]", y[0, :3])

    if not "moe_6x64x128_e4".startswith(only):
        return
    # MoE expert FFN (default-mode experts: RMS input norm, magnitude 1, no bias), top-2 of 4
    rng = np.random.default_rng(21)
    rows, D, H, E, top_k = 6, 64, 128, 4, 2
    x = rng.standard_normal((rows, D)).astype(np.float32)
    up = (rng.standard_normal((E, H, D)) * 0.02).astype(np.float32)
    down = (rng.standard_normal((E, D, H)) * 0.02).astype(np.float32)
    logits = rng.standard_normal((rows, E)).astype(np.float32)
    routing = oracle.port().router_topk(logits, top_k)
    out = R.moe_forward(x, routing, up, down)
    np.savez_compressed(os.path.join(OUT, "moe_6x64x128_e4.npz"), x=x, up=up, down=down, routing=routing,
                        out=out, top_k=top_k)
    print("moe out[0,:3]", out[0, :3])


if __name__ == "__main__":
    main()
