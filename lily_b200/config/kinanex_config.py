"""Typed configuration of the Kinanex decoder, read from its ``config.json``.

The file lists the layers one by one; every layer names its type and carries the sizes and constants of its mixer
and of its feed-forward (or ``null`` for none), so layers of one model may differ.  Keys read here:

    architecture, vocab, width, norm.eps, logit_scale (optional, 1), max_positions (optional)
    layers[i].type          "delta" | "mamba1" | "attention"
    layers[i].mixer         delta:      heads, kv_heads, dim, vdim, conv (taps)
                            mamba1:     inner, state, dt_rank, conv (taps)
                            attention:  heads, kv_heads, dim, vdim, scale, v_mix (optional),
                                        rot.{dims, base, scaling.{factor, low, high, original}} (rot and scaling optional)
    layers[i].mlp           null, or {kind: "dense", ff, limit}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union

from lily_b200.config.model_config import ConfigError, RopeScaling
from lily_b200.config.zirurax_config import _need

MAX_TAPS = 8


def _taps(d: Dict[str, Any], where: str) -> int:
    taps = _need(d, "conv", where)
    if not (1 <= taps <= MAX_TAPS):
        raise ConfigError(f"{where}.conv: {taps} taps (1 to {MAX_TAPS})")
    return taps


@dataclass(frozen=True)
class DeltaConfig:
    """Gated delta rule: ``kv_heads`` query/key heads of ``dim``, ``heads`` value heads of ``vdim``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "DeltaConfig":
        out = cls(*(_need(d, k, where) for k in ("heads", "kv_heads", "dim", "vdim")), _taps(d, where))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: {out.heads} heads over {out.kv_heads} kv heads of sizes {out.dim} / {out.vdim}")
        return out


@dataclass(frozen=True)
class SelectiveScanConfig:
    """Selective scan with a state vector per channel (the first Mamba)."""

    inner: int
    state: int
    dt_rank: int
    conv: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "SelectiveScanConfig":
        out = cls(*(_need(d, k, where) for k in ("inner", "state", "dt_rank")), _taps(d, where))
        if min(out.inner, out.state, out.dt_rank) < 1:
            raise ConfigError(f"{where}: inner, state and dt_rank must be positive")
        return out


@dataclass(frozen=True)
class TalkingAttentionConfig:
    """Softmax attention with biases, q/k norm, values at unit root mean square (blended with the first such layer's
    where ``v_mix``), one more unit in the softmax's denominator and the heads' weights mixed by a matrix."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    v_mix: bool
    rotary_dims: int                  # 0: no rotation
    rotary_base: float
    rotary_scaling: RopeScaling

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "TalkingAttentionConfig":
        rot = d.get("rot") or {}
        sc = rot.get("scaling")
        scaling = RopeScaling()
        if sc:
            scaling = RopeScaling("llama3", _need(sc, "factor", f"{where}.rot.scaling", float),
                                  _need(sc, "low", f"{where}.rot.scaling", float),
                                  _need(sc, "high", f"{where}.rot.scaling", float),
                                  int(_need(sc, "original", f"{where}.rot.scaling", float)))
            if not (scaling.factor > 0 and scaling.original_max_position_embeddings > 0 and scaling.low_freq_factor > 0
                    and scaling.high_freq_factor > 0):
                raise ConfigError(f"{where}.rot.scaling: factor, low, high and original must be positive")
        out = cls(*(_need(d, k, where) for k in ("heads", "kv_heads", "dim", "vdim")), _need(d, "scale", where, float),
                  bool(d.get("v_mix")), int(rot.get("dims") or 0), float(rot.get("base") or 10000.0), scaling)
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: {out.heads} heads over {out.kv_heads} kv heads of sizes {out.dim} / {out.vdim}")
        if out.rotary_dims < 0 or out.rotary_dims % 2 or out.rotary_dims > out.dim:
            raise ConfigError(f"{where}.rot.dims {out.rotary_dims} must be even and within dim {out.dim}")
        if out.rotary_dims and not out.rotary_base > 1.0:
            raise ConfigError(f"{where}.rot.base must be above one")
        return out


MIXERS = {"delta": DeltaConfig, "mamba1": SelectiveScanConfig, "attention": TalkingAttentionConfig}


@dataclass(frozen=True)
class ClampedFFConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class KinanexLayerConfig:
    type: str
    mixer: Union[DeltaConfig, SelectiveScanConfig, TalkingAttentionConfig]
    mlp: Optional[ClampedFFConfig]    # None: the layer has no feed-forward


@dataclass
class KinanexConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: List[KinanexLayerConfig]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], generation: Optional[Dict[str, Any]] = None,
                  architecture: Optional[str] = None) -> "KinanexConfig":
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
            ff = None
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not a feed-forward of this architecture (have: dense)")
                ff = ClampedFFConfig(_need(mlp, "ff", f"{where}.mlp"), _need(mlp, "limit", f"{where}.mlp", float))
                if ff.ff < 1 or not ff.limit > 0:
                    raise ConfigError(f"{where}.mlp: ff and limit must be positive")
            layers.append(KinanexLayerConfig(kind, MIXERS[kind].from_dict(layer.get("mixer") or {}, f"{where}.mixer"), ff))
        out = cls(architecture=architecture or str(cfg.get("architecture", "Kinanex")),
                  vocab=_need(cfg, "vocab", "config"), width=_need(cfg, "width", "config"),
                  eps=_need(cfg.get("norm") or {}, "eps", "norm", float),
                  logit_scale=float(cfg["logit_scale"]) if cfg.get("logit_scale") is not None else 1.0,
                  layers=layers, max_positions=int(cfg.get("max_positions") or (1 << 17)),
                  torch_dtype=str(cfg.get("torch_dtype") or "bfloat16"))
        if out.vocab < 1 or out.width < 1 or not out.eps > 0:
            raise ConfigError("vocab and width must be positive, norm.eps above zero")
        blended = [layer.mixer for layer in layers if layer.type == "attention" and layer.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (blended[0].kv_heads, blended[0].vdim) for m in blended):
            raise ConfigError("layers that blend their values with the first such layer's need its kv_heads and vdim")
        return out

    def summary(self) -> str:
        kinds = ", ".join(f"{sum(1 for x in self.layers if x.type == k)} {k}" for k in MIXERS)
        return (f"{self.architecture} layers={len(self.layers)} ({kinds}) width={self.width} vocab={self.vocab} "
                f"eps={self.eps} logit_scale={self.logit_scale}")
