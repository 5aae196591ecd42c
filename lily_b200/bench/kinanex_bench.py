"""The Kinanex decoder beside the Zirurax decoder (the closest existing model: softmax attention and a state-space
recurrence in every layer) and the dense (Qwen3 layer) decoder at equal sizes: prefill and decode throughput through
the same step function, and each kernel of the new design alone against its roofline, beside its like.

    python -m lily_b200.bench.kinanex_bench [--sizes small mid] [--layers 4] [--no-kernels] [--no-models] [--table]
    python bench.py --design kinanex ...          (the same, as one JSON line)

Random weights in bfloat16.  A size gives all models the same width, layers and query heads.  The Kinanex layers
alternate as [delta, attention + feed-forward, mamba1, attention + feed-forward]: the delta rule has the size's heads
with keys and values of the size's head width (its state is heads x head x head float32 a request); the selective scan
has 2 x width channels of 16 state entries and a step rank of width / 16; the attention has the size's heads with keys
and values of the head width, biases, q/k norm, half of the head rotated, the sink and mixed heads (the kernel table also
has the attention with values of 40 columns, a shape the CUDA-core kernels take); the
feed-forward has the dense layer's width.
Timing as in ``design_bench``: device time by CUDA events after warm-up, weights and caches larger than L2, kernels
over rotated inputs replayed from a graph.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import List

import torch

from lily_b200.bench.design_bench import SIZES, dense_config, model_throughput, zirurax_config
from lily_b200.bench.kbench import peaks, time_ms

SCAN_STATE = 16


def value_dim(z: dict) -> int:
    return z["head"]


def kinanex_config(z: dict, layers: int) -> dict:
    head = z["head"]
    delta = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": head, "vdim": head, "conv": 4}
    scan = {"inner": 2 * z["width"], "state": SCAN_STATE, "dt_rank": z["width"] // 16, "conv": 4}
    att = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": head, "vdim": value_dim(z), "scale": head ** -0.5, "v_mix": True,
           "rot": {"dims": head // 2, "base": 1000000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    ff = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    kinds = [("delta", delta, None), ("attention", att, ff), ("mamba1", scan, None), ("attention", att, ff)]
    return {"architecture": "Kinanex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in (kinds[i % 4] for i in range(layers))]}


def kernel_table(z: dict, tokens: int, batch: int, context: int, reps: int = 30, copies: int = 3) -> List[dict]:
    """Each kernel of the design alone, prefill shape (``tokens`` of one request) and decode shape (``batch`` requests of
    one token), with its like beside it."""
    from lily_b200.csrc import ops

    dev, dt = "cuda", torch.bfloat16
    pk = peaks()
    props = torch.cuda.get_device_properties(0)
    fp32_tflops = props.multi_processor_count * 128 * 2 * (props.clock_rate if hasattr(props, "clock_rate") else 1965000) / 1e9
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    width, nq, nkv, dd, page = z["width"], z["heads"], z["kv_heads"], z["head"], 64
    dv = value_dim(z)
    rows: List[dict] = []

    def add(name, like, fns, bytes_moved, flops=0.0, flop_peak=None, shape=""):
        ms = time_ms(fns, reps, graph=True)
        row = {"kernel": name, "like": like, "shape": shape, "us": round(ms * 1e3, 2),
               "hbm_frac": round(bytes_moved / ms / 1e6 / pk["hbm_gbs"], 3)}
        if flops:
            row["flop_frac"] = round(flops / ms / 1e9 / (flop_peak or pk["bf16_tflops"]), 3)
            row["flop_peak"] = "fp32 fma" if flop_peak else "bf16 tensor"
        row["roofline_frac"] = max(row["hbm_frac"], row.get("flop_frac", 0.0))
        row["bound"] = row.get("flop_peak", "hbm") if row.get("flop_frac", 0.0) > row["hbm_frac"] else "hbm"
        rows.append(row)

    for label, n, reqs in (("prefill", tokens, 1), ("decode", batch, batch)):
        per = n // reqs
        pages_per = -(-(per + 1) // page)
        cu = torch.arange(0, n + 1, per, device=dev, dtype=torch.int32)
        slots = torch.arange(1, reqs + 1, device=dev, dtype=torch.int32)
        token_req = torch.arange(reqs, device=dev, dtype=torch.int32).repeat_interleave(per)
        positions = torch.arange(per, device=dev, dtype=torch.int32).repeat(reqs)
        table = (torch.arange(reqs * pages_per, device=dev, dtype=torch.int32) + 1).view(reqs, pages_per)
        # ---- the delta rule beside the two recurrences the package has
        hd = nq * dd
        qkv_cols = 2 * nkv * dd + hd
        qkvs = [rnd(n, qkv_cols).to(dt) for _ in range(copies)]
        projs = [rnd(n, 8 + 2 * nq).to(dt) for _ in range(copies)]
        a_log, dt_bias = rnd(nq) - 2, rnd(nq)
        states = [torch.zeros(reqs + 1, nq * dd * dd, device=dev) for _ in range(copies)]
        add("delta_rule", "wkv_scan", [lambda x=x, p=p, s=s: ops.delta_rule(x, p, 8, 8 + nq, a_log, dt_bias, s, cu, slots, reqs, nq, nkv, dd, dd,
                                                                             1e-6, dd ** -0.5)
                                       for x, p, s in zip(qkvs, projs, states)],
            n * (qkv_cols * 2 + hd * 4) + 2 * reqs * nq * dd * dd * 4, 8.0 * n * hd * dd, fp32_tflops, shape=label)
        rkv = [(rnd(n, hd).to(dt), (rnd(n, hd) / 8).to(dt), rnd(n, hd).to(dt), -torch.rand(n, hd, device=dev, generator=g)) for _ in range(copies)]
        u = rnd(nq, dd)
        wstates = [torch.zeros(reqs + 1, nq * dd * dd + width, device=dev) for _ in range(copies)]
        plan = ops.wkv_plan([per] * reqs, dev)
        room = torch.empty(max(1, ops.wkv_workspace_floats(plan, nq, dd)), device=dev)
        add("wkv_scan (like)", "-", [lambda x=x, s=s: ops.wkv_scan(x[0], x[1], x[2], x[3], u, s, cu, slots, reqs, nq, dd, plan=plan, workspace=room)
                                     for x, s in zip(rkv, wstates)],
            n * hd * (3 * 2 + 4 + 4) + 2 * reqs * hd * dd * 4, 4.0 * n * hd * dd, fp32_tflops, shape=label)
        # ---- the selective scan beside the state-space scan of the Zirurax decoder
        inner, ns, rank = 2 * width, SCAN_STATE, width // 16
        xs = [rnd(n, inner).to(dt) for _ in range(copies)]
        lows = [rnd(n, rank + 2 * ns).to(dt) for _ in range(copies)]
        steps = [rnd(n, inner) for _ in range(copies)]
        zs = [rnd(n, 2 * inner).to(dt) for _ in range(copies)]
        a_mat, d_skip = -torch.rand(inner, ns, device=dev, generator=g) - 0.1, rnd(inner)
        sstates = [torch.zeros(reqs + 1, inner * ns, device=dev) for _ in range(copies)]
        cplan = ops.scan_plan([per] * reqs, dev, inner * ns)                   # long portions run as chunks, as in the model
        croom = torch.empty(max(1, ops.selective_workspace_floats(cplan, inner, ns)), device=dev)
        add("selective_scan", "ssd_scan", [lambda x=x, lo=lo, st=st, zz=zz, s=s: ops.selective_scan(x, lo, rank, st, zz, inner, a_mat, d_skip, s, cu, slots, reqs,
                                                                                                    plan=cplan, workspace=croom)
                                           for x, lo, st, zz, s in zip(xs, lows, steps, zs, sstates)],
            n * (inner * (2 + 4 + 2 + 2) + (rank + 2 * ns) * 2) + 2 * reqs * inner * ns * 4, 6.0 * n * inner * ns, fp32_tflops, shape=label)
        s_inner, s_state = z["s_heads"] * z["s_head"], z["state"]
        channels = s_inner + 2 * z["groups"] * s_state
        projected = 2 * s_inner + 2 * z["groups"] * s_state + z["s_heads"]
        xbcs = [rnd(n, channels).to(dt) for _ in range(copies)]
        sprojs = [rnd(n, projected).to(dt) for _ in range(copies)]
        vecs = [rnd(z["s_heads"]) - 2 for _ in range(3)]
        zstates = [torch.zeros(reqs + 1, s_inner * s_state + 3 * channels, device=dev) for _ in range(copies)]
        splan = ops.scan_plan([per] * reqs, dev, s_inner * s_state)
        sroom = torch.empty(max(1, ops.scan_workspace_floats(splan, z["s_heads"], z["s_head"], s_state)), device=dev)
        add("ssd_scan (like)", "-", [lambda x=x, p=p, s=s: ops.ssd_scan(x, p, s_inner + channels, vecs[0], vecs[1], vecs[2], s, cu, slots, reqs,
                                                                        z["s_heads"], z["s_head"], s_state, z["groups"], plan=splan, workspace=sroom)
                                     for x, p, s in zip(xbcs, sprojs, zstates)],
            n * (channels * 2 + s_inner * 4) + 2 * reqs * s_inner * s_state * 4, 6.0 * n * s_inner * s_state, fp32_tflops, shape=label)
        # ---- the layer scale on the way into the stream beside the dense decoder's add + norm
        resid = [rnd(n, width) for _ in range(copies)]
        deltas = [rnd(n, width).to(dt) for _ in range(copies)]
        post, gain = rnd(width), torch.ones(width, device=dev, dtype=dt)
        add("add_normed_rmsnorm (gain alone)", "add_rmsnorm", [lambda r=r, x=x: ops.add_normed_rmsnorm(r, x, post, 1e-6, 1.0, gain, 1e-6, dt, normalise=False)
                                                                for r, x in zip(resid, deltas)], n * width * (8 + 2 + 2), shape=label)
        add("add_rmsnorm (dense)", "-", [lambda r=r, x=x: ops.add_rmsnorm(r, x, gain, 1e-6, dt) for r, x in zip(resid, deltas)],
            n * width * (8 + 2 + 2), shape=label)
        # ---- the clamped gate beside the dense decoder's
        gus = [rnd(n, 2 * z["ff"]).to(dt) for _ in range(copies)]
        add("clamped gate * (up + 1)", "silu_mul", [lambda x=x: ops.silu_mul(x, dt, activation="swish_clamped", limit=7.0, alpha=1.702) for x in gus],
            n * z["ff"] * 6, shape=label)
        add("silu_mul (dense)", "-", [lambda x=x: ops.silu_mul(x, dt) for x in gus], n * z["ff"] * 6, shape=label)
        # ---- rotation + cache write with normed, blended values beside the plain one (same sizes)
        cols = (nq + nkv) * dd + nkv * dv
        aqkv = [rnd(n, cols).to(dt) for _ in range(copies)]
        cache_shape = (reqs * pages_per + 1, 2, nkv, page, dd) if dv == dd else (reqs * pages_per + 1, nkv * page * (dd + dv))
        caches = [torch.zeros(cache_shape, device=dev, dtype=dt) for _ in range(copies)]
        keeps = [rnd(n, nkv * dv) for _ in range(copies)]
        qg, kg = torch.ones(dd, device=dev), torch.ones(dd, device=dev)
        cos, sin = (torch.rand(per + 1, dd // 4, device=dev, generator=g) for _ in range(2))
        add("qk_norm_rope_write (values normed, blended)", "qk_norm_rope_write",
            [lambda x=x, c=c, k=k: ops.qk_norm_rope_write(x, qg, kg, 1e-6, cos, sin, positions, token_req, table, c, nq, nkv, dd, dd // 2, page, dv=dv,
                                                           v_norm=True, v_keep=k, v_blend=0.4) for x, c, k in zip(aqkv, caches, keeps)],
            n * (cols * 2 + nq * dd * 2 + nkv * (dd + dv) * 2 + nkv * dv * 4), shape=label)
        add("qk_norm_rope_write (like)", "-",
            [lambda x=x, c=c: ops.qk_norm_rope_write(x, qg, kg, 1e-6, cos, sin, positions, token_req, table, c, nq, nkv, dd, dd // 2, page, dv=dv)
             for x, c in zip(aqkv, caches)], n * (cols * 2 + nq * dd * 2 + nkv * (dd + dv) * 2), shape=label)
        # the sums in the layout the attention leaves them in for these sizes (planes a kv head, or wide float32 rows)
        sums = [ops.all_values_sums(dt, n, nq, nkv, dd, dv, dev).normal_() for _ in range(copies)]
        mix = torch.eye(nq, device=dev) + rnd(nq, nq) / 8
        add("head_mix", "sigmoid_gate", [lambda s=s: ops.head_mix(s, mix, nq, nkv, dv, dt) for s in sums],
            n * nq * dv * (nkv * sums[0].element_size() + 2), 2.0 * n * nq * nq * dv, fp32_tflops, shape=label)

    # ---- attention: the sink and the values of all kv heads, beside the same kernel without them and the dense heads
    def prefill(name, like, d_v, **how):
        pages = -(-tokens // page)
        cu1 = torch.tensor([0, tokens], device=dev, dtype=torch.int32)
        pre = torch.zeros(1, device=dev, dtype=torch.int32)
        pairs = tokens * (tokens + 1) / 2
        wide = nkv * d_v if how.get("all_values") else d_v
        sized = {} if d_v == dd else {"dv": d_v}
        fns = []
        for _ in range(copies):
            shape = (pages + 1, 2, nkv, page, dd) if d_v == dd else (pages + 1, nkv * page * (dd + d_v))
            cache = rnd(*shape).to(dt)
            tbl = (torch.randperm(pages, device=dev, generator=g) + 1).view(1, pages).to(torch.int32)
            q = rnd(tokens, nq * dd).to(dt)
            out = ops.all_values_sums(dt, tokens, nq, nkv, dd, d_v, dev) if how.get("all_values") else torch.empty((tokens, nq * d_v), device=dev, dtype=dt)
            tile = ops.prefill_tile_rows(dt, dd, page, tokens, **sized, **how)
            tr, ts = ops.prefill_tiles([0], [tokens], 0, tile, dev)
            fns.append(lambda q=q, cache=cache, tbl=tbl, out=out, tr=tr, ts=ts, tile=tile: ops.attention_prefill(
                q, cache, tbl, cu1, pre, tr, ts, out, nq, nkv, dd, page, dd ** -0.5, None, tile_rows=tile, **sized, **how))
        # the work counted is the design's own: scores once, weighted sums over every kv head's values
        add(name, like, fns, tokens * (nkv * (dd + d_v) + nq * dd) * 2 + tokens * nq * wide * out.element_size(),
            2.0 * nq * (dd + wide) * pairs, shape=f"{tokens} tokens")

    def decode(name, like, d_v, **how):
        pages = -(-context // page)
        wide = nkv * d_v if how.get("all_values") else d_v
        sized = {} if d_v == dd else {"dv": d_v}
        fns = []
        for _ in range(copies):
            shape = (batch * pages + 1, 2, nkv, page, dd) if d_v == dd else (batch * pages + 1, nkv * page * (dd + d_v))
            cache = rnd(*shape).to(dt)
            tbl = (torch.randperm(batch * pages, device=dev, generator=g) + 1).view(batch, pages).to(torch.int32)
            q = rnd(batch, nq * dd).to(dt)
            out = ops.all_values_sums(dt, batch, nq, nkv, dd, d_v, dev) if how.get("all_values") else torch.empty((batch, nq * d_v), device=dev, dtype=dt)
            seq = torch.full((batch,), context, device=dev, dtype=torch.int32)
            on_cores = bool(how) and not ops.sink_on_tensor_cores(dt, dd, d_v)
            seen = ops.all_values_decode_rows(dt, batch, nkv, dd, d_v) if how.get("all_values") else batch
            plan = ops.plan_decode_attention(dt, seen, nq, nkv, dd, context, fusable=False,
                                             **({"dv": wide, "cuda_cores": True} if on_cores else sized))
            scratch = torch.empty(max(1, plan.scratch_floats), device=dev)
            fns.append(lambda q=q, cache=cache, tbl=tbl, out=out, seq=seq, scratch=scratch, plan=plan: ops.attention_decode(
                q, cache, tbl, seq, out, scratch, plan.splits, nq, nkv, dd, page, dd ** -0.5, None, stages=plan.stages, **sized, **how))
        add(name, like, fns, batch * context * nkv * (dd + d_v) * 2 + 2 * batch * nq * dd * 2, 2.0 * batch * nq * (dd + wide) * context,
            shape=f"{batch} x {context}")

    prefill("attention_prefill (sink, values of all kv heads)", "attention_prefill", dv, sink=True, all_values=True)
    prefill("attention_prefill (sink alone)", "attention_prefill", dv, sink=True)
    prefill("attention_prefill (dense heads)", "-", dd)
    decode("attention_decode (sink, values of all kv heads)", "attention_decode", dv, sink=True, all_values=True)
    decode("attention_decode (sink alone)", "attention_decode", dv, sink=True)
    decode("attention_decode (dense heads)", "-", dd)
    # a value size of its own (values of 40 columns a head beside keys of the head width): the CUDA-core kernels take these shapes
    prefill("attention_prefill (sink, all kv heads; values of 40: CUDA cores)", "attention_prefill", 40, sink=True, all_values=True)
    decode("attention_decode (sink, all kv heads; values of 40: CUDA cores)", "attention_decode", 40, sink=True, all_values=True)
    return rows


def run(sizes, layers, tokens, batch, context, steps, kernels=True, models=True) -> dict:
    out = {"design": "Kinanex", "beside": "the Zirurax decoder and the dense (Qwen3 layer) decoder at equal width, heads and layers",
           "dtype": "bf16", "data": "synthetic: seeded random weights", "peaks": peaks(), "layers": layers,
           "prefill_tokens": tokens, "decode_batch": batch, "context": context, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z}
        if models:
            entry["kinanex"] = model_throughput(kinanex_config(z, layers), tokens, batch, context, steps)
            entry["zirurax"] = model_throughput(zirurax_config(z, layers), tokens, batch, context, steps)
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
            for k in ("kinanex", "zirurax", "dense"):
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
