"""RMSNorm fused with the residual add.

``forward(residual, delta)`` adds ``delta`` into the float32 residual stream in place and
returns the normalised activations in the compute dtype: the fused-add convention of
lily/layers/layernorm.py:11-47 with the sum kept in float32.  With ``rows`` only those rows are
normalised (the final norm before the logits).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict

from lily_b200.parts.base import BuildContext, Norm, TensorSpec, register_part


@dataclass
class NormedDelta:
    """A sublayer's output that enters the residual stream as ``mult * (rms(delta) * gain)``, its own root mean
    square (with ``eps``) taken over the row first (a norm behind the sublayer as well as ahead of it).  A block hands
    it on as its pending delta; the norm that follows folds it into the stream in the pass in which it normalises."""

    delta: Any                 # [tokens, size] in the compute dtype, or float32 partial sums [splits, tokens, size]
    gain: Any                  # float32 [size]
    eps: float
    mult: float = 1.0
    normalise: bool = True     # False: ``mult * (delta * gain)``, a gain per column without the division (a layer scale)


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"
    suffix: str = ".weight"        # the gain's name is the part's prefix followed by this ("" where the prefix is the name)
    offset: float = 0.0            # the checkpoint stores the gain minus this (1.0: gains stored around zero); the sum
                                   # is formed once, in float32, when the gain is loaded


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: RMSNormSpec, prefix: str, ctx: BuildContext):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.weight = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {f"{self.prefix}{self.spec.suffix}": TensorSpec((self.spec.size,), role="vector", init="gain")}

    def load(self, get) -> None:
        self.weight = get(f"{self.prefix}{self.spec.suffix}")
        if self.spec.offset:
            self.weight = (self.weight.float() + self.spec.offset).contiguous()

    def forward(self, residual, delta=None, delta_bias=None, rows=None, write_residual=True, also=None, out_dtype=None):
        """``delta`` may be a tuple of tensors to be summed; ``delta_bias`` a float32 vector added to every row;
        ``also`` another norm of this kind and size whose output of the same rows is wanted too (returns a pair)."""
        if isinstance(delta, NormedDelta):
            if delta_bias is not None or also is not None:
                raise ValueError("a normalised delta comes alone: no stream vector and no second norm in the same pass")
            return self.ctx.ops.add_normed_rmsnorm(residual, delta.delta, delta.gain, delta.eps, delta.mult, self.weight,
                                                   self.spec.eps, out_dtype or self.ctx.dtype, rows=rows,
                                                   write_residual=write_residual and rows is None,
                                                   **({} if delta.normalise else {"normalise": False}))
        deltas = [d for d in delta if d is not None] if isinstance(delta, (tuple, list)) else ([delta] if delta is not None else [])
        if delta_bias is None and also is None and len(deltas) <= 1:
            return self.ctx.ops.add_rmsnorm(residual, deltas[0] if deltas else None, self.weight, self.spec.eps,
                                            out_dtype or self.ctx.dtype, rows=rows, write_residual=write_residual)
        if rows is not None:
            # gathered rows: the sum goes into the stream first, then the plain form reads the rows
            self.ctx.ops.add_rmsnorm_multi(residual, deltas, [], self.spec.eps, self.ctx.dtype, bias=delta_bias)
            return self.ctx.ops.add_rmsnorm(residual, None, self.weight, self.spec.eps, out_dtype or self.ctx.dtype, rows=rows)
        if also is not None and (also.spec.eps != self.spec.eps or also.spec.size != self.spec.size):
            raise ValueError("two norms share a pass over the rows only with one size and one eps")
        gains = [self.weight.float()] + ([also.weight.float()] if also is not None else [])
        outs = self.ctx.ops.add_rmsnorm_multi(residual, deltas, gains, self.spec.eps, out_dtype or self.ctx.dtype,
                                              bias=delta_bias, write_residual=write_residual)
        return outs if also is not None else outs[0]
