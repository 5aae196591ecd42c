"""Plain, slow implementation of the Kinanex decoder, for tests only.

Whole sequences, no cache, one function per mechanism, float32 on the CPU unless
``precision(torch.float64)`` is in force.  It reads the raw ``config.json`` dictionary and the
checkpoint's own tensor names and shares no code with ``lily_b200``.

The design in this file's notation.  The stream starts as ``N(embed[token])``; a layer is

    x <- x + s_1 * mixer(N_1(x))        x <- x + s_2 * ff(N_2(x))        N(y) = y / rms(y) * w

with ``s`` a gain per column (the second line only where the layer has a feed-forward).  The mixer is one of

* ``delta``: a matrix S per head updated by the gated delta rule, ``S <- a S; S <- S + k (b (v - S^T k))^T``, read out
  as ``S^T q`` after the write; q, k, v pass a short causal convolution and SiLU, q and k are made unit vectors;
* ``mamba1``: a selective scan with a state vector per channel, ``s <- exp(dt A) s + dt x B``, ``y = s . C + D x``;
* ``attention``: grouped-query attention with biases, q/k norm, partial rotation (Llama-3 frequency scaling), values
  brought to unit root mean square and blended with the first such layer's values, a softmax whose denominator holds
  one more unit, and the heads' weights mixed by a matrix before they meet the values.

The feed-forward is ``down(g sigmoid(1.702 g) (u + 1))`` with clamped g and u.  The logits are the final norm times the
embedding table times a constant.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

Tensor = torch.Tensor

_COMPUTE = [torch.float32]


class precision:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        _COMPUTE.append(self.dtype)

    def __exit__(self, *exc):
        _COMPUTE.pop()


def _c(t: Tensor) -> Tensor:
    return t.to(_COMPUTE[-1])


def rms(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def unit(x: Tensor, eps: float = 1e-6) -> Tensor:
    """x / sqrt(sum(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def short_convolution(u: Tensor, taps: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """y[t, c] = sum_j taps[c, j] u[t - (J - 1) + j, c] (+ bias[c]); rows before the start are zero."""
    n, J = u.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros((J - 1, u.shape[1]), dtype=u.dtype), u])
    y = torch.zeros_like(u)
    for j in range(J):
        y = y + padded[j:j + n] * taps[:, j]
    return y if bias is None else y + bias


# --------------------------------------------------------------------------- the delta-rule mixer

def delta_rule(q: Tensor, k: Tensor, v: Tensor, a: Tensor, b: Tensor) -> Tensor:
    """One head.  q, k [n, d]; v [n, dv]; a, b [n].  Returns o [n, dv]."""
    n, d = q.shape
    S = torch.zeros((d, v.shape[1]), dtype=q.dtype)
    out = []
    for t in range(n):
        S = a[t] * S
        u = b[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def delta_mixer(h: Tensor, w: Dict[str, Tensor], p: str, mx: dict, eps: float) -> Tensor:
    n = h.shape[0]
    H, G, d, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    act = lambda name: F.silu(short_convolution(h @ _c(w[f"{p}.{name}"]).T, _c(w[f"{p}.{name}.conv"])))
    q = unit(act("q").view(n, G, d)) * d ** -0.5
    k = unit(act("k").view(n, G, d))
    v = act("v").view(n, H, dv)
    beta = torch.sigmoid(h @ _c(w[f"{p}.b"]).T)                                              # [n, H]
    decay = torch.exp(-torch.exp(_c(w[f"{p}.A_log"])) * F.softplus(h @ _c(w[f"{p}.a"]).T + _c(w[f"{p}.dt_bias"])))
    heads = [delta_rule(q[:, j // (H // G)], k[:, j // (H // G)], v[:, j], decay[:, j], beta[:, j]) for j in range(H)]
    o = rms(torch.stack(heads, 1), eps) * _c(w[f"{p}.norm"])                                 # [n, H, dv]
    o = o * F.silu(h @ _c(w[f"{p}.g"]).T).view(n, H, dv)
    return o.reshape(n, H * dv) @ _c(w[f"{p}.o"]).T


# --------------------------------------------------------------------------- the selective-scan mixer

def selective_scan(x: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, D: Tensor) -> Tensor:
    """x, dt [n, c]; A [c, s]; B, C [n, s]; D [c].  Returns y [n, c]."""
    S = torch.zeros_like(A)
    out = []
    for t in range(x.shape[0]):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        out.append(S @ C[t] + D * x[t])
    return torch.stack(out)


def mamba_mixer(h: Tensor, w: Dict[str, Tensor], p: str, mx: dict) -> Tensor:
    inner, rank, state = int(mx["inner"]), int(mx["dt_rank"]), int(mx["state"])
    xz = h @ _c(w[f"{p}.in"]).T
    x, z = xz[:, :inner], xz[:, inner:]
    x = F.silu(short_convolution(x, _c(w[f"{p}.conv"]), _c(w[f"{p}.conv.b"])))
    low = x @ _c(w[f"{p}.x"]).T
    dt = F.softplus(low[:, :rank] @ _c(w[f"{p}.dt"]).T + _c(w[f"{p}.dt.b"]))
    B, C = low[:, rank:rank + state], low[:, rank + state:rank + 2 * state]
    y = selective_scan(x, dt, -torch.exp(_c(w[f"{p}.A_log"])), B, C, _c(w[f"{p}.D"]))
    return (y * F.silu(z)) @ _c(w[f"{p}.o"]).T


# --------------------------------------------------------------------------- attention

def rotary_frequencies(rot: dict) -> Tensor:
    """f_i = base^(-2i/dims), float64; rescaled by wavelength when the entry has 'scaling'."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, lo, hi, L = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        wavelength = 2.0 * math.pi / f
        s = (L / wavelength - lo) / (hi - lo) if hi != lo else torch.zeros_like(f)
        blend = (1.0 - s) * f / factor + s * f
        f = torch.where(wavelength < L / hi, f, torch.where(wavelength > L / lo, f / factor, blend))
    return f


def rotate(x: Tensor, rot: Optional[dict], positions: Tensor) -> Tensor:
    """x [n, heads, d]: column i < dims/2 turns with column i + dims/2 by the angle position * f_i."""
    if not rot or not int(rot["dims"]):
        return x
    dims = int(rot["dims"])
    half = dims // 2
    angle = positions.to(torch.float32)[:, None] * rotary_frequencies(rot).to(torch.float32)[None, :]      # float32 angles
    cos, sin = _c(angle.cos())[:, None, :], _c(angle.sin())[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], -1)


def sink_softmax(scores: Tensor, mask: Tensor) -> Tensor:
    """p_j = exp(s_j) / (1 + sum_visible exp(s_j)) over the last axis."""
    s = scores.masked_fill(~mask, float("-inf"))
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def attention_values(h: Tensor, w: Dict[str, Tensor], p: str, mx: dict, eps: float) -> Tensor:
    """A layer's own values [n, kv_heads, dv], each head at unit root mean square."""
    n = h.shape[0]
    v = (h @ _c(w[f"{p}.v"]).T + _c(w[f"{p}.v.b"])).view(n, int(mx["kv_heads"]), int(mx["vdim"]))
    return rms(v, eps)


def attention_mixer(h: Tensor, w: Dict[str, Tensor], p: str, mx: dict, eps: float, v: Tensor) -> Tensor:
    """``v`` [n, kv_heads, dv]: the values the layer attends over (normed and, where it applies, blended)."""
    n = h.shape[0]
    H, G, d, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    pos = torch.arange(n)
    q = (h @ _c(w[f"{p}.q"]).T + _c(w[f"{p}.q.b"])).view(n, H, d)
    k = (h @ _c(w[f"{p}.k"]).T + _c(w[f"{p}.k.b"])).view(n, G, d)
    q = rotate(rms(q, eps) * _c(w[f"{p}.q.norm"]), mx.get("rot"), pos)
    k = rotate(rms(k, eps) * _c(w[f"{p}.k.norm"]), mx.get("rot"), pos)
    kv_of = torch.arange(H) // (H // G)
    scores = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * float(mx["scale"])
    weights = sink_softmax(scores, (pos[None, :] <= pos[:, None])[None])                     # [H, n, n]
    weights = torch.einsum("hg,gij->hij", _c(w[f"{p}.talk"]), weights)
    o = torch.einsum("hij,jhe->ihe", weights, v[:, kv_of])
    return o.reshape(n, H * dv) @ _c(w[f"{p}.o"]).T


# --------------------------------------------------------------------------- feed-forward, model

def feed_forward(h: Tensor, w: Dict[str, Tensor], p: str, limit: float) -> Tensor:
    g = torch.clamp(h @ _c(w[f"{p}.gate"]).T, max=limit)
    u = torch.clamp(h @ _c(w[f"{p}.up"]).T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _c(w[f"{p}.down"]).T


def forward(cfg: dict, w: Dict[str, Tensor], tokens: Sequence[int], streams: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [tokens, vocab] of one whole sequence; ``streams`` collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = rms(_c(w["embed"])[torch.as_tensor(list(tokens), dtype=torch.long)], eps) * _c(w["embed.norm"])
    first_values = None
    for i, entry in enumerate(cfg["layers"]):
        p, mx = f"l{i}", entry["mixer"]
        h = rms(x, eps) * _c(w[f"{p}.norm1"])
        if entry["type"] == "delta":
            a = delta_mixer(h, w, f"{p}.mix", mx, eps)
        elif entry["type"] == "mamba1":
            a = mamba_mixer(h, w, f"{p}.mix", mx)
        elif entry["type"] == "attention":
            v = attention_values(h, w, f"{p}.mix", mx, eps)
            if mx.get("v_mix"):
                if first_values is None:
                    first_values = v
                else:
                    lam = _c(w[f"{p}.mix.vmix"])
                    v = (1.0 - lam) * v + lam * first_values
            a = attention_mixer(h, w, f"{p}.mix", mx, eps, v)
        else:
            raise ValueError(entry["type"])
        x = x + _c(w[f"{p}.ls1"]) * a
        if entry.get("mlp") is not None:
            h = rms(x, eps) * _c(w[f"{p}.norm2"])
            x = x + _c(w[f"{p}.ls2"]) * feed_forward(h, w, f"{p}.mlp", float(entry["mlp"]["limit"]))
        if streams is not None:
            streams.append(x.clone())
    return (rms(x, eps) * _c(w["final.norm"])) @ _c(w["embed"]).T * float(cfg.get("logit_scale", 1.0))
