"""The Gotivik decoder beside the dense (Qwen3 layer) decoder at equal sizes: prefill and decode throughput of both
through the same step function, and each kernel of the new design alone against its roofline, beside the like kernel
of the dense decoder (the closest existing model: softmax attention over the paged cache and a dense feed-forward).

    python -m lily_b200.bench.gotivik_bench [--sizes small mid] [--layers 4] [--no-kernels] [--no-models] [--table]
    python bench.py --design gotivik ...          (the same, as one JSON line)

Random weights in bfloat16.  A size gives both models the same width, layers, query and key/value heads.  The Gotivik
layers alternate as [differential, differential, windowed, differential]: the differential attention has the size's
heads with two maps of 64 columns each and values of 128 (so its projections have the dense layer's shapes), a cap of
50 and a query temperature; the windowed attention has heads of 128 with 64 rotated columns (YaRN), a convolution of
4 taps on q, k and v, the size's window and 64 kept first positions.  The feed-forward ``down(relu(up x)^2)`` is
3/2 of the dense layer's width, which gives it the gated feed-forward's weights and work.
Timing as in ``design_bench``: device time by CUDA events after warm-up, weights and caches larger than L2, kernels
over rotated inputs replayed from a graph.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import List

import torch

from lily_b200.bench.design_bench import SIZES, dense_config, model_throughput
from lily_b200.bench.kbench import peaks, time_ms

KEPT = 64          # first positions the windowed layers keep in sight
CAP = 50.0


def gotivik_config(z: dict, layers: int) -> dict:
    head = z["head"]
    diff = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": head // 2, "vdim": head, "scale": (head // 2) ** -0.5,
            "diff": 0.2, "softcap": CAP, "q_temp": {"coef": 0.25, "every": 1024}}
    conv = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": head, "vdim": head, "scale": head ** -0.5, "conv": 4,
            "mask": {"size": z["window"], "keep_first": KEPT},
            "rot": {"dims": head // 2, "base": 1000000.0, "scaling": {"factor": 4.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    ff = {"kind": "dense", "ff": z["ff"] * 3 // 2}
    kinds = [("attention_2", diff), ("attention_2", diff), ("attention", conv), ("attention_2", diff)]
    return {"architecture": "Gotivik", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.7,
            "layers": [{"type": t, "mixer": m, "mlp": ff} for t, m in (kinds[i % 4] for i in range(layers))]}


def kernel_table(z: dict, tokens: int, batch: int, context: int, reps: int = 30, copies: int = 3) -> List[dict]:
    """Each kernel of the design alone, prefill shape (``tokens`` of one request) and decode shape (``batch`` requests of
    one token), with the like kernel of the dense decoder beside it."""
    from lily_b200.csrc import ops

    dev, dt = "cuda", torch.bfloat16
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    width, nq, nkv, dd, page = z["width"], z["heads"], z["kv_heads"], z["head"], 64
    half = dd // 2
    window = z["window"]
    rows: List[dict] = []

    def add(name, like, fns, bytes_moved, flops=0.0, shape=""):
        ms = time_ms(fns, reps, graph=True)
        row = {"kernel": name, "like": like, "shape": shape, "us": round(ms * 1e3, 2),
               "hbm_frac": round(bytes_moved / ms / 1e6 / pk["hbm_gbs"], 3)}
        if flops:
            row["flop_frac"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
            row["flop_peak"] = "bf16 tensor"
        row["roofline_frac"] = max(row["hbm_frac"], row.get("flop_frac", 0.0))
        row["bound"] = row.get("flop_peak", "hbm") if row.get("flop_frac", 0.0) > row["hbm_frac"] else "hbm"
        rows.append(row)

    q_cols, kv_cols = nq * dd, nkv * dd
    projected = q_cols + 2 * kv_cols
    for label, n, reqs in (("prefill", tokens, 1), ("decode", batch, batch)):
        per = n // reqs
        pages_per = -(-(per + 1) // page)
        cu = torch.arange(0, n + 1, per, device=dev, dtype=torch.int32)
        slots = torch.arange(1, reqs + 1, device=dev, dtype=torch.int32)
        token_req = torch.arange(reqs, device=dev, dtype=torch.int32).repeat_interleave(per)
        positions = torch.arange(per, device=dev, dtype=torch.int32).repeat(reqs)
        table = (torch.arange(reqs * pages_per, device=dev, dtype=torch.int32) + 1).view(reqs, pages_per)
        caches = [torch.zeros(reqs * pages_per + 1, 2, nkv, page, dd, device=dev, dtype=dt) for _ in range(copies)]
        # ---- the sublayer's two norms and the add in one pass, beside the dense decoder's add + norm
        resid = [rnd(n, width) for _ in range(copies)]
        deltas = [rnd(n, width).to(dt) for _ in range(copies)]
        post, gain = rnd(width), torch.ones(width, device=dev, dtype=dt)
        add("add_normed_rmsnorm", "add_rmsnorm", [lambda r=r, x=x: ops.add_normed_rmsnorm(r, x, post, 1e-6, 0.7, gain, 1e-6, dt)
                                                  for r, x in zip(resid, deltas)], n * width * (8 + 2 + 2), shape=label)
        add("add_rmsnorm (dense)", "-", [lambda r=r, x=x: ops.add_rmsnorm(r, x, gain, 1e-6, dt) for r, x in zip(resid, deltas)],
            n * width * (8 + 2 + 2), shape=label)
        # ---- the feed-forward's activation beside the gated one
        ff = z["ff"] * 3 // 2
        ups = [rnd(n, ff).to(dt) for _ in range(copies)]
        add("activation relu2", "silu_mul", [lambda x=x: ops.activation(x, dt, "relu2") for x in ups], n * ff * 4, shape=label)
        gus = [rnd(n, 2 * z["ff"]).to(dt) for _ in range(copies)]
        add("silu_mul (dense)", "-", [lambda x=x: ops.silu_mul(x, dt) for x in gus], n * z["ff"] * 6, shape=label)
        # ---- the convolution over q, k and v
        projs = [rnd(n, projected).to(dt) for _ in range(copies)]
        taps = 4
        conv_w = rnd(projected, taps) / 2
        states = [torch.zeros(reqs + 1, (taps - 1) * projected, device=dev) for _ in range(copies)]
        chunk_req, chunk_start = ops.token_chunks([per] * reqs, ops.SSM_CHUNK, dev)
        add("causal_conv (no activation)", "-", [lambda x=x, s=s: ops.causal_conv(x, 0, projected, conv_w, None, s, 0, chunk_req, chunk_start,
                                                                                 cu, slots, ops.SSM_CHUNK, activation="none")
                                                 for x, s in zip(projs, states)], n * projected * 4, shape=label)
        # ---- queries and cache rows of the differential attention beside the rotation + cache write
        gated = [rnd(n, projected + nq).to(dt) for _ in range(copies)]
        add("diff_prepare", "qk_norm_rope_write", [lambda x=x, c=c: ops.diff_prepare(x, positions, token_req, table, c, nq, nkv, half, dd, 2, page, 0.25, 1024)
                                                   for x, c in zip(gated, caches)], n * (projected * 2 + 2 * q_cols * 2 + 2 * kv_cols * 2), shape=label)
        cos, sin = (torch.rand(per + 1, half // 2, device=dev, generator=g) for _ in range(2))
        add("qk_norm_rope_write (dense)", "-", [lambda x=x, c=c: ops.qk_norm_rope_write(x, None, None, 1e-6, cos, sin, positions, token_req, table, c,
                                                                                       nq, nkv, dd, half, page)
                                                for x, c in zip(projs, caches)], n * (projected * 2 + q_cols * 2 + 2 * kv_cols * 2), shape=label)
        maps_out = [rnd(n, 2 * q_cols).to(dt) for _ in range(copies)]
        add("diff_combine", "sigmoid_gate", [lambda m=m, x=x: ops.diff_combine(m, x, projected, nq, dd, 2, 0.3, 0.5, 1e-6)
                                             for m, x in zip(maps_out, gated)], n * (2 * q_cols * 2 + q_cols * 2), shape=label)
        outs = [rnd(n, q_cols).to(dt) for _ in range(copies)]
        gates = [rnd(n, q_cols).to(dt) for _ in range(copies)]
        add("sigmoid_gate (like)", "-", [lambda o=o, x=x: ops.sigmoid_gate(o, x) for o, x in zip(outs, gates)], n * q_cols * 6, shape=label)

    # ---- attention: window with kept first positions, and the two maps, beside the dense heads
    def prefill(heads, keep, cap, name, like):
        pages = -(-tokens // page)
        cu1 = torch.tensor([0, tokens], device=dev, dtype=torch.int32)
        pre = torch.zeros(1, device=dev, dtype=torch.int32)
        span = min(window, tokens) if window else tokens
        pairs = tokens * span - span * (span - 1) / 2 if window else tokens * (tokens + 1) / 2
        opts = {"keep_first": keep} if keep else {}
        if cap:
            opts["softcap"] = cap
        fns = []
        for _ in range(copies):
            cache = rnd(pages + 1, 2, nkv, page, dd).to(dt)
            table = (torch.randperm(pages, device=dev, generator=g) + 1).view(1, pages).to(torch.int32)
            q = rnd(tokens, heads * dd).to(dt)
            out = torch.empty_like(q)
            tile = ops.prefill_tile_rows(dt, dd, page, tokens, **opts)
            tr, ts = ops.prefill_tiles([0], [tokens], 0, tile, dev)
            fns.append(lambda q=q, cache=cache, table=table, out=out, tr=tr, ts=ts, tile=tile: ops.attention_prefill(
                q, cache, table, cu1, pre, tr, ts, out, heads, nkv, dd, page, dd ** -0.5, window if not cap else None, tile_rows=tile, **opts))
        if cap:
            pairs = tokens * (tokens + 1) / 2
        add(name, like, fns, tokens * (2 * nkv + 2 * heads) * dd * 2, 4.0 * heads * dd * pairs, shape=f"{tokens} tokens")

    def decode(heads, keep, cap, name, like):
        pages = -(-context // page)
        seen = context if cap else min(window, context) + keep
        opts = {"keep_first": keep} if keep else {}
        fns = []
        for _ in range(copies):
            cache = rnd(batch * pages + 1, 2, nkv, page, dd).to(dt)
            table = (torch.randperm(batch * pages, device=dev, generator=g) + 1).view(batch, pages).to(torch.int32)
            q = rnd(batch, heads * dd).to(dt)
            out = torch.empty_like(q)
            seq = torch.full((batch,), context, device=dev, dtype=torch.int32)
            plan = ops.plan_decode_attention(dt, batch, heads, nkv, dd, seen, fusable=False, **opts)
            scratch = torch.empty(max(1, plan.scratch_floats), device=dev)
            capped = {"softcap": cap} if cap else {}
            fns.append(lambda q=q, cache=cache, table=table, out=out, seq=seq, scratch=scratch, plan=plan: ops.attention_decode(
                q, cache, table, seq, out, scratch, plan.splits, heads, nkv, dd, page, dd ** -0.5, None if cap else window,
                stages=plan.stages, **capped, **opts))
        add(name, like, fns, batch * seen * 2 * nkv * dd * 2 + 2 * batch * heads * dd * 2, 4.0 * batch * heads * dd * seen,
            shape=f"{batch} x {context}")

    prefill(nq, KEPT, None, "attention_prefill (window, kept first)", "attention_prefill")
    prefill(nq, 0, None, "attention_prefill (dense heads, same window)", "-")
    prefill(2 * nq, 0, CAP, "attention_prefill (two maps a head, cap, causal)", "attention_prefill")
    prefill(nq, 0, CAP, "attention_prefill (dense heads, cap, causal)", "-")
    decode(nq, KEPT, None, "attention_decode (window, kept first)", "attention_decode")
    decode(nq, 0, None, "attention_decode (dense heads, same window)", "-")
    decode(2 * nq, 0, CAP, "attention_decode (two maps a head, cap, causal)", "attention_decode")
    decode(nq, 0, CAP, "attention_decode (dense heads, cap, causal)", "-")
    return rows


def run(sizes, layers, tokens, batch, context, steps, kernels=True, models=True) -> dict:
    out = {"design": "Gotivik", "beside": "the dense (Qwen3 layer) decoder at equal width, heads and layers",
           "dtype": "bf16", "data": "synthetic: seeded random weights", "peaks": peaks(), "layers": layers,
           "prefill_tokens": tokens, "decode_batch": batch, "context": context, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z}
        if models:
            entry["gotivik"] = model_throughput(gotivik_config(z, layers), tokens, batch, context, steps)
            entry["dense"] = model_throughput(dense_config(z, layers, context), tokens, batch, context, steps)
        if kernels:
            entry["kernels"] = kernel_table(z, tokens, batch, context)
        out["sizes"][name] = entry
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", nargs="+", default=["small", "mid"], choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-models", action="store_true")
    ap.add_argument("--table", action="store_true", help="print the kernels as a table on stderr as well")
    a = ap.parse_args(argv)
    out = run(a.sizes, a.layers, a.tokens, a.batch, a.context, a.steps, kernels=not a.no_kernels, models=not a.no_models)
    if a.table:
        for name, entry in out["sizes"].items():
            for k in ("gotivik", "dense"):
                if k in entry:
                    print(name, k, entry[k], file=sys.stderr)
            for row in entry.get("kernels", []):
                print(f"{name:6s} {row['kernel']:52s} {row['shape']:14s} {row['us']:10.2f} us  hbm {row['hbm_frac']:.3f}"
                      + (f"  {row['flop_peak']} {row['flop_frac']:.3f}" if "flop_frac" in row else "") + f"  ({row['bound']})",
                      file=sys.stderr)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
