"""Typed configuration of the Gotivik decoder, read from its ``config.json``.

The file lists the layers one by one; every layer names its type and carries the sizes and constants of its mixer
and of its feed-forward (or ``null`` for none), so layers of one model may differ.  A layer with ``weights_of: j`` has
no tensors of its own and uses layer j's, with a cache and state of its own.  Keys read here:

    architecture, vocab, width, norm.eps, residual_mult (optional, 1), max_positions (optional)
    layers[i].type          "attention" | "attention_2"
    layers[i].weights_of    optional: the layer whose tensors this one uses
    layers[i].mixer         attention:    heads, kv_heads, dim, vdim, scale, conv (optional: taps),
                                          mask.{size, keep_first} (optional),
                                          rot.{dims, base, scaling.{factor, original, fast, slow}} (rot and scaling optional)
                            attention_2:  heads, kv_heads, dim, vdim, scale, diff, softcap (optional),
                                          q_temp.{coef, every} (optional)
    layers[i].mlp           null, or {kind: "dense", ff}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union

from lily_b200.config.model_config import ConfigError, RopeScaling
from lily_b200.config.zirurax_config import _need


def _heads(d: Dict[str, Any], where: str):
    heads, kv_heads, dim, vdim = (_need(d, k, where) for k in ("heads", "kv_heads", "dim", "vdim"))
    if min(heads, kv_heads, dim, vdim) < 1 or heads % kv_heads:
        raise ConfigError(f"{where}: {heads} heads over {kv_heads} kv heads of sizes {dim} / {vdim}")
    return heads, kv_heads, dim, vdim


@dataclass(frozen=True)
class ConvAttentionConfig:
    """Softmax attention with a short convolution on q, k and v, rotation and a window that keeps the first positions."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                         # taps of the convolution; 0: none
    window: Optional[int]
    keep_first: int
    rotary_dims: int                  # 0: no rotation
    rotary_base: float
    rotary_scaling: RopeScaling

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "ConvAttentionConfig":
        heads, kv_heads, dim, vdim = _heads(d, where)
        rot = d.get("rot") or {}
        sc = rot.get("scaling")
        scaling = RopeScaling()
        if sc:
            scaling = RopeScaling("yarn", factor=_need(sc, "factor", f"{where}.rot.scaling", float),
                                  original_max_position_embeddings=_need(sc, "original", f"{where}.rot.scaling", int),
                                  fast_turns=_need(sc, "fast", f"{where}.rot.scaling", float),
                                  slow_turns=_need(sc, "slow", f"{where}.rot.scaling", float))
            if not (scaling.factor > 0 and scaling.original_max_position_embeddings > 0 and scaling.fast_turns > 0
                    and scaling.slow_turns > 0):
                raise ConfigError(f"{where}.rot.scaling: factor, original, fast and slow must be positive")
        mask = d.get("mask") or {}
        out = cls(heads, kv_heads, dim, vdim, _need(d, "scale", where, float), int(d.get("conv") or 0),
                  int(mask["size"]) if mask.get("size") else None, int(mask.get("keep_first") or 0),
                  int(rot.get("dims") or 0), float(rot.get("base") or 10000.0), scaling)
        if out.rotary_dims < 0 or out.rotary_dims % 2 or out.rotary_dims > out.dim:
            raise ConfigError(f"{where}.rot.dims {out.rotary_dims} must be even and within dim {out.dim}")
        if out.rotary_dims and not out.rotary_base > 1.0:
            raise ConfigError(f"{where}.rot.base must be above one")
        if (out.window is not None and out.window < 1) or out.keep_first < 0:
            raise ConfigError(f"{where}.mask: size must be positive and keep_first not negative")
        if not (0 <= out.conv <= 8):
            raise ConfigError(f"{where}.conv: {out.conv} taps (1 to 8, or none)")
        return out


@dataclass(frozen=True)
class DiffAttentionConfig:
    """Differential attention: two maps a head, query temperature by position, capped scores, a gate per head."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    softcap: Optional[float]
    q_temp_coef: float
    q_temp_every: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "DiffAttentionConfig":
        heads, kv_heads, dim, vdim = _heads(d, where)
        qt = d.get("q_temp") or {}
        softcap = d.get("softcap")
        out = cls(heads, kv_heads, dim, vdim, _need(d, "scale", where, float), _need(d, "diff", where, float),
                  float(softcap) if softcap else None,
                  _need(qt, "coef", f"{where}.q_temp", float) if qt else 0.0,
                  _need(qt, "every", f"{where}.q_temp") if qt else 1)
        if out.q_temp_every < 1:
            raise ConfigError(f"{where}.q_temp.every must be positive")
        return out


MIXERS = {"attention": ConvAttentionConfig, "attention_2": DiffAttentionConfig}


@dataclass(frozen=True)
class GotivikLayerConfig:
    type: str
    mixer: Union[ConvAttentionConfig, DiffAttentionConfig]
    ff: Optional[int]                 # None: the layer has no feed-forward
    weights_of: Optional[int]         # None: the layer has tensors of its own


@dataclass
class GotivikConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: List[GotivikLayerConfig]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], generation: Optional[Dict[str, Any]] = None,
                  architecture: Optional[str] = None) -> "GotivikConfig":
        listed = cfg.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json lacks the list 'layers'")
        layers = []
        for i, layer in enumerate(listed):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}.type {kind!r} is not a layer type of this architecture (have: {', '.join(MIXERS)})")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not a feed-forward of this architecture (have: dense)")
            owner = layer.get("weights_of")
            layers.append(GotivikLayerConfig(kind, MIXERS[kind].from_dict(layer.get("mixer") or {}, f"{where}.mixer"),
                                             None if mlp is None else _need(mlp, "ff", f"{where}.mlp"),
                                             None if owner is None else int(owner)))
        out = cls(architecture=architecture or str(cfg.get("architecture", "Gotivik")),
                  vocab=_need(cfg, "vocab", "config"), width=_need(cfg, "width", "config"),
                  eps=_need(cfg.get("norm") or {}, "eps", "norm", float),
                  residual_mult=float(cfg["residual_mult"]) if cfg.get("residual_mult") is not None else 1.0,
                  layers=layers, max_positions=int(cfg.get("max_positions") or (1 << 17)),
                  torch_dtype=str(cfg.get("torch_dtype") or "bfloat16"))
        if out.vocab < 1 or out.width < 1 or not out.eps > 0:
            raise ConfigError("vocab and width must be positive, norm.eps above zero")
        for i in range(len(layers)):
            out.owner(i)
        return out

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it names another with ``weights_of``)."""
        seen = {i}
        while self.layers[i].weights_of is not None:
            j = self.layers[i].weights_of
            if not (0 <= j < len(self.layers)) or j in seen:
                raise ConfigError(f"layers[{i}].weights_of = {j} names no layer with tensors of its own")
            if self.layers[j].type != self.layers[i].type:
                raise ConfigError(f"layers[{i}] ({self.layers[i].type}) cannot use the tensors of layers[{j}] ({self.layers[j].type})")
            seen.add(j)
            i = j
        return i

    def summary(self) -> str:
        own = sum(1 for layer in self.layers if layer.weights_of is None)
        return (f"{self.architecture} layers={len(self.layers)} (with tensors of their own: {own}) width={self.width} "
                f"vocab={self.vocab} eps={self.eps} residual_mult={self.residual_mult}")
