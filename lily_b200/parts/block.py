"""Block arrangements.  The pre-norm block: ``r += mixer(norm_in(r)); r += feed_forward(norm_post(r))``; the parallel
block (``ParallelBlockSpec``): one norm, several mixers and the feed-forward side by side on its output; the sandwich
block (``SandwichBlockSpec``): a norm on both sides of each sublayer and a multiplier on what enters the stream.

The residual stream ``r`` is float32 and updated in place; each add is fused into the norm that
follows it, so a block receives the pending delta of the block before it and returns its own
(lily/models/llama.py:108-117 with the fused-add convention of lily/layers/layernorm.py:34-36).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Tuple

from lily_b200.parts.base import Block, BlockSpec, BuildContext, RunSlots, TensorSpec, build_part, register_part
from lily_b200.parts.norm import NormedDelta


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, prefix: str, ctx: BuildContext):
        self.spec = spec
        p = spec.prefix
        self.norm_in = build_part("norm", spec.norm_in, f"{p}.{spec.norm_in_name}", ctx)
        self.mixer = build_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}", ctx)
        self.norm_post = build_part("norm", spec.norm_post, f"{p}.{spec.norm_post_name}", ctx)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, f"{p}.{spec.feed_forward_name}", ctx)
        self.mixers = (self.mixer,)
        self.parts = (self.norm_in, self.mixer, self.norm_post, self.feed_forward)

    def tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.parts:
            out.update(part.tensors())
        return out

    def load(self, get) -> None:
        for part in self.parts:
            part.load(get)

    def forward(self, residual, delta, batch, run: RunSlots):
        x = self.norm_in.forward(residual, delta, delta_bias=run.stream_bias)
        a = self.mixer.forward(x, batch, run.caches[0], run.states[0], run.write_cache)
        y = self.norm_post.forward(residual, a)
        return self.feed_forward.forward(y, batch)


@dataclass(frozen=True)
class ParallelBlockSpec:
    """One norm whose output every sublayer reads: ``h = norm(r)``, ``r += mean_k(rms(mixer_k(h)) * gain_k) + ff(h)``.
    ``mixers`` lists (name under the block's prefix, mixer spec, name of the mixer's output gain); the feed-forward
    may be absent.  The mixers run side by side on the same ``h``; each output is divided by its root mean square
    over the model width (``eps``) and multiplied by its own gain before the mean is taken.
    A gain name of None leaves the mixer's output as it is (one mixer then: ``r += mixer(h) + ff(.)``, the sum formed
    in float32 by the next residual add).  ``ff_norm`` gives the feed-forward a norm of its own over the same ``r``
    (``r += mixer(norm(r)) + ff(ff_norm(r))``); both norms share one pass over the rows."""

    prefix: str
    hidden_size: int
    mixers: Tuple[Tuple[str, Any, str], ...]
    feed_forward: Any
    norm: Any
    eps: float
    kind: str = "parallel"
    norm_name: str = "norm1"
    feed_forward_name: str = "mlp"
    ff_norm: Any = None
    ff_norm_name: str = "norm2"


@register_part("block", "parallel")
class ParallelBlock(Block):
    def __init__(self, spec: ParallelBlockSpec, prefix: str, ctx: BuildContext):
        if not spec.mixers:
            raise ValueError("a parallel block has at least one mixer")
        self.spec, self.ctx = spec, ctx
        p = spec.prefix
        self.norm = build_part("norm", spec.norm, f"{p}.{spec.norm_name}", ctx)
        self.mixers = tuple(build_part("mixer", m, f"{p}.{name}", ctx) for name, m, _ in spec.mixers)
        self.feed_forward = None if spec.feed_forward is None else \
            build_part("feed_forward", spec.feed_forward, f"{p}.{spec.feed_forward_name}", ctx)
        self.ff_norm = None
        if spec.ff_norm is not None and self.feed_forward is not None:
            self.ff_norm = build_part("norm", spec.ff_norm, f"{p}.{spec.ff_norm_name}", ctx)
        self.parts = (self.norm, *self.mixers) + ((self.feed_forward,) if self.feed_forward is not None else ()) + \
            ((self.ff_norm,) if self.ff_norm is not None else ())
        plain = [gain is None for _, _, gain in spec.mixers]
        if any(plain) and (not all(plain) or len(plain) != 1):
            raise ValueError("a parallel block takes its mixers' outputs as they are only when it has one mixer")
        self.plain_sum = all(plain)
        self.gain_names = [] if self.plain_sum else [f"{p}.{gain}" for _, _, gain in spec.mixers]
        self.gains = []

    def tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.parts:
            out.update(part.tensors())
        for name in self.gain_names:
            out[name] = TensorSpec((self.spec.hidden_size,), role="vector", init="gain")
        return out

    def load(self, get) -> None:
        for part in self.parts:
            part.load(get)
        self.gains = [get(name).float().contiguous() for name in self.gain_names]

    def forward(self, residual, delta, batch, run: RunSlots):
        if self.ff_norm is not None:
            h, h_ff = self.norm.forward(residual, delta, delta_bias=run.stream_bias, also=self.ff_norm)
        else:
            h = h_ff = self.norm.forward(residual, delta, delta_bias=run.stream_bias)
        outs = [m.forward(h, batch, run.caches[k], run.states[k], run.write_cache) for k, m in enumerate(self.mixers)]
        f = self.feed_forward.forward(h_ff, batch) if self.feed_forward is not None else None
        if self.plain_sum:
            return (outs[0], f) if f is not None else outs[0]          # summed in float32 by the next residual add
        # float32, as one plane of partial sums: the next norm adds it into the residual stream
        return self.ctx.ops.normed_mean(outs, self.gains, self.spec.eps, add=f)


@dataclass(frozen=True)
class SandwichBlockSpec:
    """A norm ahead of and behind each sublayer: ``r += mult * norm_1b(mixer(norm_1(r)))``, then, where the block has a
    feed-forward, ``r += mult * norm_2b(ff(norm_2(r)))``.  The norm behind a sublayer and the add are folded into the
    pass of the norm that comes next (``NormedDelta``), in this block or in the one after it.
    ``post_divides`` False: what stands behind a sublayer is a gain per column alone (a layer scale,
    ``r += mult * gain_1b * mixer(norm_1(r))``), named like the norms behind the sublayers and folded the same way."""

    prefix: str
    mixer: Any
    feed_forward: Any                         # None: the block ends behind its mixer
    norm: Any                                 # the spec of all four norms (size, eps, gain naming)
    mult: float = 1.0
    kind: str = "sandwich"
    mixer_name: str = "mix"
    feed_forward_name: str = "mlp"
    norm_names: Tuple[str, str, str, str] = ("norm1", "norm1b", "norm2", "norm2b")
    post_divides: bool = True


@register_part("block", "sandwich")
class SandwichBlock(Block):
    def __init__(self, spec: SandwichBlockSpec, prefix: str, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        p = spec.prefix
        n1, n1b, n2, n2b = spec.norm_names
        self.norm_in = build_part("norm", spec.norm, f"{p}.{n1}", ctx)
        self.norm_in_post = build_part("norm", spec.norm, f"{p}.{n1b}", ctx)
        self.mixer = build_part("mixer", spec.mixer, f"{p}.{spec.mixer_name}", ctx)
        self.mixers = (self.mixer,)
        self.parts = (self.norm_in, self.norm_in_post, self.mixer)
        self.feed_forward = self.norm_ff = self.norm_ff_post = None
        if spec.feed_forward is not None:
            self.norm_ff = build_part("norm", spec.norm, f"{p}.{n2}", ctx)
            self.norm_ff_post = build_part("norm", spec.norm, f"{p}.{n2b}", ctx)
            self.feed_forward = build_part("feed_forward", spec.feed_forward, f"{p}.{spec.feed_forward_name}", ctx)
            self.parts += (self.norm_ff, self.norm_ff_post, self.feed_forward)
        self.post_gains = []

    def tensors(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for part in self.parts:
            out.update(part.tensors())
        return out

    def load(self, get) -> None:
        for part in self.parts:
            part.load(get)
        # the gains of the norms behind the sublayers enter a float32 sum
        self.post_gains = [n.weight.float().contiguous() for n in (self.norm_in_post, self.norm_ff_post) if n is not None]

    def forward(self, residual, delta, batch, run: RunSlots):
        eps, mult, divides = self.spec.norm.eps, float(self.spec.mult), self.spec.post_divides
        h = self.norm_in.forward(residual, delta, delta_bias=run.stream_bias)
        a = NormedDelta(self.mixer.forward(h, batch, run.caches[0], run.states[0], run.write_cache), self.post_gains[0], eps, mult, divides)
        if self.feed_forward is None:
            return a
        h = self.norm_ff.forward(residual, a)
        return NormedDelta(self.feed_forward.forward(h, batch), self.post_gains[1], eps, mult, divides)
