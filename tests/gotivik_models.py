"""Small Gotivik configurations and random weights for the tests, made here from the design alone (no code of
``lily_b200`` decides a name or a shape)."""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from zirurax_models import tokens, write_model_dir  # noqa: F401  (the same container and token helper)


def conv_attention(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, conv=3, window: Optional[int] = 11, keep_first=3,
                   rot_dims=8, base=100.0, scaling=None, ff: Optional[int] = 40, weights_of=None) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        mixer["conv"] = conv
    if window:
        mixer["mask"] = {"size": window, "keep_first": keep_first}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            mixer["rot"]["scaling"] = scaling
    out = {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def diff_attention(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.35, diff=0.3, softcap: Optional[float] = 6.0, q_temp=(0.4, 7),
                   ff: Optional[int] = 40, weights_of=None) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if softcap:
        mixer["softcap"] = softcap
    if q_temp:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    out = {"type": "attention_2", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


SCALING = {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 0.5}      # the ramp lies inside 8 rotated dimensions

# Sizes that differ in every respect from layer to layer: head counts and sizes for keys and values, 1 to 4 taps and
# none, partial, full and no rotation, with and without scaling, window, kept first positions, cap, temperature and
# feed-forward; layers that use another layer's tensors, one of them a layer further on.
VARIED = {"architecture": "Gotivik", "vocab": 131, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
          "layers": [diff_attention(),
                     conv_attention(heads=6, kv_heads=3, dim=16, vdim=8, conv=3, window=11, keep_first=3, rot_dims=8,
                                    scaling=SCALING, ff=None),
                     diff_attention(weights_of=0),
                     conv_attention(heads=2, kv_heads=2, dim=12, vdim=20, conv=2, window=None, rot_dims=12, scale=0.25, ff=56,
                                    weights_of=5),
                     conv_attention(heads=6, kv_heads=3, dim=16, vdim=8, conv=3, window=11, keep_first=3, rot_dims=8,
                                    scaling=SCALING, ff=None, weights_of=1),
                     conv_attention(heads=2, kv_heads=2, dim=12, vdim=20, conv=2, window=None, rot_dims=12, scale=0.25, ff=56),
                     diff_attention(heads=3, kv_heads=1, dim=16, vdim=16, scale=0.2, diff=0.8, softcap=None, q_temp=None, ff=24),
                     conv_attention(heads=2, kv_heads=1, dim=8, vdim=8, conv=0, window=5, keep_first=0, rot_dims=0, ff=32),
                     conv_attention(heads=1, kv_heads=1, dim=24, vdim=16, conv=4, window=20, keep_first=17, rot_dims=24,
                                    base=50.0, ff=32),
                     # a single tap: a gain on every channel, nothing carried from step to step
                     conv_attention(heads=2, kv_heads=1, dim=8, vdim=24, conv=1, window=7, keep_first=1, rot_dims=4, ff=None)]}

# Sharp attention: a large scale puts nearly all weight on the best visible key, so a key that is wrongly seen or
# wrongly dropped at a window's edge or among the kept first positions changes the output outright.
SHARP = {"architecture": "Gotivik", "vocab": 97, "width": 32, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
         "layers": [conv_attention(heads=2, kv_heads=1, dim=16, vdim=16, scale=3.0, conv=2, window=9, keep_first=2, rot_dims=16, ff=32),
                    diff_attention(heads=2, kv_heads=1, dim=8, vdim=16, scale=2.5, diff=0.5, softcap=40.0, q_temp=(0.5, 16), ff=32),
                    conv_attention(heads=2, kv_heads=1, dim=16, vdim=16, scale=3.0, conv=4, window=17, keep_first=6, rot_dims=16, ff=32)]}

# Head sizes the tensor-core attention kernels take, wider layers.
WIDE = {"architecture": "Gotivik", "vocab": 257, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
        "layers": [diff_attention(heads=4, kv_heads=2, dim=32, vdim=64, scale=0.2, diff=0.4, softcap=20.0, q_temp=(0.3, 64), ff=192),
                   conv_attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.15, conv=4, window=40, keep_first=5, rot_dims=32,
                                  base=10000.0, scaling={"factor": 2.0, "original": 64, "fast": 8.0, "slow": 1.0}, ff=128),
                   diff_attention(heads=2, kv_heads=1, dim=64, vdim=128, scale=0.12, diff=0.6, softcap=None, q_temp=(0.5, 100), ff=None),
                   conv_attention(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.1, conv=3, window=None, rot_dims=64, ff=256),
                   diff_attention(heads=4, kv_heads=2, dim=32, vdim=64, scale=0.2, diff=0.4, softcap=20.0, q_temp=(0.3, 64), ff=192,
                                  weights_of=0)]}


def owner(cfg: dict, i: int) -> int:
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def shapes(cfg: dict) -> Dict[str, tuple]:
    w = cfg["width"]
    out = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, ly in enumerate(cfg["layers"]):
        if ly.get("weights_of") is not None:
            continue
        m, p = ly["mixer"], f"l{i}"
        out.update({f"{p}.norm1": (w,), f"{p}.norm1b": (w,)})
        if ly["type"] == "attention":
            q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            out.update({f"{p}.mix.q": (q, w), f"{p}.mix.k": (k, w), f"{p}.mix.v": (v, w), f"{p}.mix.o": (w, m["heads"] * m["vdim"])})
            if m.get("conv"):
                out.update({f"{p}.mix.q.conv": (q, m["conv"]), f"{p}.mix.k.conv": (k, m["conv"]), f"{p}.mix.v.conv": (v, m["conv"])})
        else:
            out.update({f"{p}.mix.q": (m["heads"] * 2 * m["dim"], w), f"{p}.mix.k": (m["kv_heads"] * 2 * m["dim"], w),
                        f"{p}.mix.v": (m["kv_heads"] * m["vdim"], w), f"{p}.mix.g": (m["heads"], w),
                        f"{p}.mix.o": (w, m["heads"] * m["vdim"])})
            out.update({f"{p}.mix.{n}": (m["dim"],) for n in ("lq1", "lk1", "lq2", "lk2")})
        if ly["mlp"]:
            out.update({f"{p}.norm2": (w,), f"{p}.norm2b": (w,), f"{p}.mlp.up": (ly["mlp"]["ff"], w), f"{p}.mlp.down": (w, ly["mlp"]["ff"])})
    return out


def make_weights(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Random weights at scales that keep every mechanism alive: projections of unit gain, gains around one, taps of
    the size of one, vectors whose products give a lambda away from its starting value."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        n = lambda: torch.randn(shape, generator=g)
        if name == "embed":
            t = n()
        elif name.endswith(("norm1", "norm1b", "norm2", "norm2b", "final.norm")):
            t = 1.0 + 0.2 * n()
        elif name.endswith(".conv"):
            t = 0.6 * n()
        elif name.endswith(("lq1", "lk1", "lq2", "lk2")):
            t = 0.5 * n()
        else:
            t = n() / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out
