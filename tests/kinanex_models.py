"""Small Kinanex configurations and random weights for the tests, made here from the design alone (no code of
``lily_b200`` decides a name or a shape)."""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from zirurax_models import tokens, write_model_dir  # noqa: F401  (the same container and token helper)


def mlp(ff: Optional[int], limit: float = 2.0):
    return None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}


def delta(heads=4, kv_heads=2, dim=16, vdim=8, conv=3, ff: Optional[int] = None, limit=2.0) -> dict:
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp(ff, limit)}


def mamba(inner=40, state=6, dt_rank=5, conv=4, ff: Optional[int] = None, limit=2.0) -> dict:
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp(ff, limit)}


def attention(heads=4, kv_heads=2, dim=16, vdim=12, scale=0.3, v_mix=True, rot_dims=8, base=100.0, scaling=None,
              ff: Optional[int] = 40, limit=2.0) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            mixer["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": mixer, "mlp": mlp(ff, limit)}


SCALING = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}       # all three bands among four frequencies of base 100

# Sizes that differ from layer to layer: head counts and sizes that are no powers of two, 1 to 4 taps, partial, full
# and no rotation, with and without scaling, attention layers that share values and one that does not, layers with
# and without feed-forward, limits that bite and one that never does, an attention layer first and a recurrence last.
VARIED = {"architecture": "Kinanex", "vocab": 131, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
          "layers": [attention(heads=6, kv_heads=3, dim=12, vdim=10, v_mix=False, rot_dims=12, ff=None),
                     delta(heads=4, kv_heads=2, dim=12, vdim=20, conv=2, ff=56, limit=0.7),
                     attention(heads=4, kv_heads=2, dim=16, vdim=12, rot_dims=8, scaling=SCALING, ff=40, limit=1.5),
                     mamba(inner=40, state=6, dt_rank=5, conv=4, ff=None),
                     attention(heads=2, kv_heads=2, dim=24, vdim=12, rot_dims=0, scale=0.2, ff=24, limit=50.0),
                     delta(heads=3, kv_heads=3, dim=20, vdim=7, conv=1, ff=None),
                     attention(heads=4, kv_heads=2, dim=8, vdim=12, rot_dims=8, base=50.0, scale=0.4, ff=None),
                     mamba(inner=24, state=19, dt_rank=1, conv=2, ff=32, limit=1.0),
                     delta(heads=2, kv_heads=1, dim=8, vdim=16, conv=4, ff=None)]}

# Sharp attention: a large scale puts nearly all weight on the best visible key (or on the sink when no key scores
# above zero), so a key that is wrongly seen, a sink left out or heads mixed the wrong way round change the output outright.
SHARP = {"architecture": "Kinanex", "vocab": 97, "width": 32, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
         "layers": [attention(heads=2, kv_heads=1, dim=16, vdim=16, scale=3.0, rot_dims=16, ff=32),
                    delta(heads=2, kv_heads=2, dim=16, vdim=16, conv=2, ff=None),
                    attention(heads=4, kv_heads=1, dim=8, vdim=16, scale=2.5, rot_dims=4, ff=32)]}

# Wider layers, head sizes of 32 to 128, one kv head (the model norm's and the logits' constants at 1).
WIDE = {"architecture": "Kinanex", "vocab": 257, "width": 128, "norm": {"eps": 1e-6},
        "layers": [delta(heads=4, kv_heads=2, dim=64, vdim=32, conv=4, ff=None),
                   attention(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.15, rot_dims=32, base=10000.0,
                             scaling={"factor": 6.0, "low": 1.0, "high": 3.0, "original": 64}, ff=192, limit=1.5),
                   mamba(inner=192, state=16, dt_rank=8, conv=3, ff=None),
                   delta(heads=2, kv_heads=2, dim=128, vdim=40, conv=3, ff=128, limit=3.0),
                   attention(heads=8, kv_heads=4, dim=32, vdim=16, scale=0.2, v_mix=False, rot_dims=32, ff=None),
                   attention(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.15, rot_dims=64, ff=128, limit=0.5)]}


# Values that other configurations happen to make equal or 1: one head, as many kv heads as heads, values wider than
# keys, a single tap and a single state entry, a step rank above the state size, a recurrence first and an attention last.
ODD = {"architecture": "Kinanex", "vocab": 53, "width": 40, "norm": {"eps": 1e-4}, "logit_scale": 3.0,
       "layers": [mamba(inner=24, state=1, dt_rank=7, conv=1, ff=None),
                  delta(heads=1, kv_heads=1, dim=40, vdim=72, conv=4, ff=48, limit=1.2),
                  attention(heads=3, kv_heads=3, dim=20, vdim=28, rot_dims=20, scale=0.25, ff=None),
                  delta(heads=6, kv_heads=1, dim=8, vdim=4, conv=2, ff=None),
                  attention(heads=5, kv_heads=1, dim=16, vdim=16, v_mix=False, rot_dims=6, scale=0.3, ff=16, limit=0.4),
                  attention(heads=3, kv_heads=3, dim=12, vdim=28, rot_dims=0, scale=0.5, ff=None)]}

# No attention at all: a model without a paged cache.
RECURRENT = {"architecture": "Kinanex", "vocab": 61, "width": 32, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
             "layers": [delta(heads=2, kv_heads=2, dim=16, vdim=16, conv=3, ff=32), mamba(inner=48, state=8, dt_rank=4, conv=3, ff=None)]}


def shapes(cfg: dict) -> Dict[str, tuple]:
    w = cfg["width"]
    out = {"embed": (cfg["vocab"], w), "embed.norm": (w,), "final.norm": (w,)}
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}"
        out.update({f"{p}.norm1": (w,), f"{p}.ls1": (w,)})
        if ly["type"] == "attention":
            q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            out.update({f"{p}.mix.q": (q, w), f"{p}.mix.k": (k, w), f"{p}.mix.v": (v, w), f"{p}.mix.q.b": (q,), f"{p}.mix.k.b": (k,),
                        f"{p}.mix.v.b": (v,), f"{p}.mix.q.norm": (m["dim"],), f"{p}.mix.k.norm": (m["dim"],),
                        f"{p}.mix.talk": (m["heads"], m["heads"]), f"{p}.mix.o": (w, m["heads"] * m["vdim"])})
            if m.get("v_mix"):
                out[f"{p}.mix.vmix"] = ()
        elif ly["type"] == "delta":
            qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({f"{p}.mix.q": (qk, w), f"{p}.mix.k": (qk, w), f"{p}.mix.v": (v, w), f"{p}.mix.q.conv": (qk, m["conv"]),
                        f"{p}.mix.k.conv": (qk, m["conv"]), f"{p}.mix.v.conv": (v, m["conv"]), f"{p}.mix.b": (m["heads"], w),
                        f"{p}.mix.a": (m["heads"], w), f"{p}.mix.A_log": (m["heads"],), f"{p}.mix.dt_bias": (m["heads"],),
                        f"{p}.mix.norm": (m["vdim"],), f"{p}.mix.g": (v, w), f"{p}.mix.o": (w, v)})
        else:
            n, s, r = m["inner"], m["state"], m["dt_rank"]
            out.update({f"{p}.mix.in": (2 * n, w), f"{p}.mix.conv": (n, m["conv"]), f"{p}.mix.conv.b": (n,),
                        f"{p}.mix.x": (r + 2 * s, n), f"{p}.mix.dt": (n, r), f"{p}.mix.dt.b": (n,), f"{p}.mix.A_log": (n, s),
                        f"{p}.mix.D": (n,), f"{p}.mix.o": (w, n)})
        if ly["mlp"]:
            ff = ly["mlp"]["ff"]
            out.update({f"{p}.norm2": (w,), f"{p}.ls2": (w,), f"{p}.mlp.gate": (ff, w), f"{p}.mlp.up": (ff, w), f"{p}.mlp.down": (w, ff)})
    return out


def make_weights(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Random weights at scales that keep every mechanism alive: projections of unit gain, gains around one, taps of
    the size of one, decays from nearly none to fast, a head-mixing matrix far from the identity, blends near a half."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        n = lambda: torch.randn(shape, generator=g)
        if name == "embed":
            t = n()
        elif name.endswith(("norm1", "norm2", "final.norm", "embed.norm", "q.norm", "k.norm", "mix.norm", ".D")):
            t = 1.0 + 0.2 * n()
        elif name.endswith((".ls1", ".ls2")):
            t = 0.6 + 0.2 * n()
        elif name.endswith(".conv"):
            t = 0.6 * n()
        elif name.endswith(".talk"):
            t = 0.5 * torch.eye(shape[0]) + 0.4 * n()
        elif name.endswith(".vmix"):
            t = torch.sigmoid(n())
        elif name.endswith("mix.A_log") and len(shape) == 1:
            t = torch.linspace(-3.0, 1.0, shape[0])[torch.randperm(shape[0], generator=g)]        # slow and fast heads
        elif name.endswith("mix.A_log"):
            t = torch.log(torch.linspace(0.2, 4.0, shape[1])).expand(shape).clone() + 0.3 * n()
        elif name.endswith(("dt_bias", "dt.b", ".b")) and len(shape) == 1:
            t = 0.5 * n()
        else:
            t = n() / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out
