"""Plain, slow implementation of the Gotivik decoder, for tests only.

Whole sequences, no cache, one function per mechanism, float32 on the CPU unless
``precision(torch.float64)`` is in force.  It reads the raw ``config.json`` dictionary and the
checkpoint's own tensor names and shares no code with ``lily_b200``.

The design in this file's notation.  With ``m`` the residual multiplier, a layer is

    x <- x + m * N_1b(mixer(N_1(x)))        x <- x + m * N_2b(ff(N_2(x)))        N(y) = y / rms(y) * w

(the second line only where the layer has a feed-forward).  A layer may borrow another layer's weights.  The mixer is
either a grouped-query softmax attention whose q, k and v pass a short causal convolution over time and whose q and
k are then rotated by position (frequencies rescaled in the YaRN manner), over a sliding window that also keeps a
sequence's first positions; or a differential attention: two softmax maps with their own q and k over shared
values, combined as ``a1 - lambda a2``, brought to unit root mean square per head and gated per head.  The
feed-forward is ``down(relu(up h)^2)``.  The logits are the final norm times the embedding table.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

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


def relu_squared(z: Tensor) -> Tensor:
    r = torch.clamp(z, min=0.0)
    return r * r


# --------------------------------------------------------------------------- rotation

def yarn_frequencies(rot: dict):
    """Returns (frequencies [dims / 2], the factor both cos and sin are multiplied by).

    f_i = base^(-2i/dims).  With scaling (factor s, trained length L, turns ``fast`` and ``slow``): the feature index at
    which a wave makes t turns over L is idx(t) = dims ln(L / (2 pi t)) / (2 ln base); between lo = idx(fast) (rounded
    down, at least 0) and hi = idx(slow) (rounded up, at most dims - 1) a ramp r_i goes from 0 to 1, and the frequency is
    f_i (1 - r_i) + f_i r_i / s.  The tables are stretched by 0.1 ln(s) + 1."""
    dims = int(rot["dims"])
    base = float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    stretch = 1.0
    if sc:
        s, length = float(sc["factor"]), float(sc["original"])

        def idx(turns: float) -> float:
            return dims * math.log(length / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(idx(float(sc["fast"]))), 0)
        hi = min(math.ceil(idx(float(sc["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / s * ramp + f * (1.0 - ramp)
        stretch = 0.1 * math.log(s) + 1.0
    return f.to(torch.float32), stretch


def rotate_halves(x: Tensor, positions: Tensor, freqs: Tensor, stretch: float) -> Tensor:
    """x [tokens, heads, dim]: feature i of the first 2 n is paired with feature i + n (n = len(freqs)) and the pair
    (u, v) turned by the angle position * f_i: (u cos - v sin, v cos + u sin); the other features pass."""
    n = freqs.numel()
    ang = positions.to(torch.float32)[:, None] * freqs[None, :]          # float32 angles
    cos = _c(ang.cos() * stretch)[:, None, :]
    sin = _c(ang.sin() * stretch)[:, None, :]
    u, v = x[..., :n], x[..., n:2 * n]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., 2 * n:]], dim=-1)


# --------------------------------------------------------------------------- short convolution

def causal_conv(u: Tensor, w: Tensor) -> Tensor:
    """u [tokens, channels], w [channels, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    taps = w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, u.shape[1]), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + u.shape[0]] * w[:, j][None, :]
    return y


# --------------------------------------------------------------------------- attention

def visible(n: int, window: Optional[int], keep_first: int) -> Tensor:
    """[queries, keys] bool: key j is seen from i when j <= i and (i - j < window or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, mask: Tensor, softcap: Optional[float] = None) -> Tensor:
    """q [tokens, heads, d], k [tokens, kv_heads, d], v [tokens, kv_heads, dv] -> [tokens, heads, dv]; query head h
    reads kv head h // (heads / kv_heads)."""
    heads, kv_heads = q.shape[1], k.shape[1]
    rep = heads // kv_heads
    out = []
    for h in range(heads):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


def windowed_attention(h: Tensor, w: Dict[str, Tensor], p: str, mx: dict) -> Tensor:
    """The mixer 'attention' on h [tokens, width]."""
    n = h.shape[0]
    H, G, d, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    q, k, v = h @ _c(w[f"{p}.q"]).T, h @ _c(w[f"{p}.k"]).T, h @ _c(w[f"{p}.v"]).T
    if mx.get("conv"):
        q, k, v = (causal_conv(t, _c(w[f"{p}.{name}.conv"])) for t, name in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(n, H, d), k.view(n, G, d), v.view(n, G, dv)
    rot = mx.get("rot")
    if rot and rot.get("dims"):
        f, stretch = yarn_frequencies(rot)
        pos = torch.arange(n)
        q, k = rotate_halves(q, pos, f, stretch), rotate_halves(k, pos, f, stretch)
    mask = mx.get("mask") or {}
    window = int(mask["size"]) if mask.get("size") else None
    o = softmax_attention(q, k, v, float(mx["scale"]), visible(n, window, int(mask.get("keep_first") or 0)))
    return o.reshape(n, H * dv) @ _c(w[f"{p}.o"]).T


def query_temperature(n: int, qt: Optional[dict]) -> Tensor:
    """1 + coef ln(floor((p + 1) / every) + 1) for p = 0 .. n - 1, float32."""
    if not qt:
        return torch.ones(n, dtype=torch.float32)
    p = torch.arange(n, dtype=torch.float32)
    return 1.0 + float(qt["coef"]) * torch.log(torch.floor((p + 1.0) / float(qt["every"])) + 1.0)


def differential_lambda(w: Dict[str, Tensor], p: str, diff: float) -> float:
    a = float((w[f"{p}.lq1"].double() * w[f"{p}.lk1"].double()).sum())
    b = float((w[f"{p}.lq2"].double() * w[f"{p}.lk2"].double()).sum())
    return math.exp(a) - math.exp(b) + diff


def differential_attention(h: Tensor, w: Dict[str, Tensor], p: str, mx: dict, eps: float) -> Tensor:
    """The mixer 'attention_2' on h [tokens, width]."""
    n = h.shape[0]
    H, G, d, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    diff = float(mx["diff"])
    q = (h @ _c(w[f"{p}.q"]).T).view(n, H, 2, d) * _c(query_temperature(n, mx.get("q_temp")))[:, None, None, None]
    k = (h @ _c(w[f"{p}.k"]).T).view(n, G, 2, d)
    v = (h @ _c(w[f"{p}.v"]).T).view(n, G, dv)
    mask = visible(n, None, 0)
    cap = float(mx["softcap"]) if mx.get("softcap") else None
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, float(mx["scale"]), mask, cap)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, float(mx["scale"]), mask, cap)
    o = a1 - differential_lambda(w, p, diff) * a2
    o = rms(o, eps) * (1.0 - diff)
    gate = torch.sigmoid(h @ _c(w[f"{p}.g"]).T)                          # [tokens, heads]
    o = o * gate[:, :, None]
    return o.reshape(n, H * dv) @ _c(w[f"{p}.o"]).T


# --------------------------------------------------------------------------- feed-forward, layer, model

def feed_forward(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    return relu_squared(h @ _c(w[f"{p}.up"]).T) @ _c(w[f"{p}.down"]).T


def owner(cfg: dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    seen = set()
    while cfg["layers"][i].get("weights_of") is not None and i not in seen:
        seen.add(i)
        i = int(cfg["layers"][i]["weights_of"])
    return i


def layer(x: Tensor, w: Dict[str, Tensor], cfg: dict, i: int) -> Tensor:
    entry = cfg["layers"][i]
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    p = f"l{owner(cfg, i)}"
    h = rms(x, eps) * _c(w[f"{p}.norm1"])
    if entry["type"] == "attention":
        a = windowed_attention(h, w, f"{p}.mix", entry["mixer"])
    elif entry["type"] == "attention_2":
        a = differential_attention(h, w, f"{p}.mix", entry["mixer"], eps)
    else:
        raise ValueError(entry["type"])
    x = x + m * (rms(a, eps) * _c(w[f"{p}.norm1b"]))
    if entry.get("mlp") is not None:
        h = rms(x, eps) * _c(w[f"{p}.norm2"])
        x = x + m * (rms(feed_forward(h, w, f"{p}.mlp"), eps) * _c(w[f"{p}.norm2b"]))
    return x


def forward(cfg: dict, w: Dict[str, Tensor], tokens: Sequence[int], streams: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [tokens, vocab] of one whole sequence; ``streams`` collects the residual stream after every layer run."""
    x = _c(w["embed"])[torch.as_tensor(list(tokens), dtype=torch.long)]
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        if streams is not None:
            streams.append(x.clone())
    eps = float(cfg["norm"]["eps"])
    return (rms(x, eps) * _c(w["final.norm"])) @ _c(w["embed"]).T
