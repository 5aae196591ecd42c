"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``, no bias; act is SiLU (SwiGLU) unless the spec names
another (``"gelu_tanh"``); the fused kernels take either.

gate and up are one matrix ``[2 * inter, hidden]`` so that one product feeds the SiLU*mul
(lily/models/llama.py:31-47, stacking llama.py:164-165).  In bfloat16, when the intermediate size
is a multiple of 128, the rows alternate between 128 gate rows and the 128 up rows of the same
outputs: a 256-row tile of the product then holds both halves of 128 outputs, and for more than a
few tokens the tcgen05 kernel applies SiLU*mul in its epilogue, so the ``[tokens, 2 * inter]``
intermediate never reaches memory.  Otherwise gate rows come first, then up rows.  For up to 8
tokens (decode) one weight-streaming kernel forms both sums and SiLU*mul from either layout; the
reference streams these products through its own kernel as well (lily/csrc/bf16_skinny.cu:45-96).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, FeedForward, TensorSpec, register_part


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"
    activation: str = "silu"              # "silu" | "gelu_tanh" | "swish_clamped"
    # "swish_clamped": down(g sigmoid(alpha g) (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit)
    limit: float = 0.0
    alpha: float = 1.702
    # names of the gate, up and down weights under the part's prefix; None: "<x>_proj.weight"
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, f"{role}_proj.weight")


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec: SwiGLUSpec, prefix: str, ctx: BuildContext):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_gate_up = None
        self.w_down = None
        self.block = None          # rows of gate / up alternate in runs of this many (None: all gate, then all up)

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i, p = self.spec.hidden_size, self.spec.intermediate_size, self.prefix
        n = self.spec.name
        return {f"{p}.{n('gate')}": TensorSpec((i, h)), f"{p}.{n('up')}": TensorSpec((i, h)),
                f"{p}.{n('down')}": TensorSpec((h, i))}

    def load(self, get) -> None:
        p, i = self.prefix, self.spec.intermediate_size
        name = self.spec.name
        gate = get(f"{p}.{name('gate')}")
        h = self.spec.hidden_size
        self.w_gate_up = torch.empty((2 * i, h), dtype=gate.dtype, device=gate.device)
        self.block = b = self.ctx.ops.gate_up_interleave(gate.dtype, i)
        if b:
            runs = self.w_gate_up.view(i // b, 2, b, h)
            runs[:, 0].copy_(gate.view(i // b, b, h))
            del gate
            runs[:, 1].copy_(get(f"{p}.{name('up')}").view(i // b, b, h))
        else:
            self.w_gate_up[:i].copy_(gate)
            del gate
            self.w_gate_up[i:].copy_(get(f"{p}.{name('up')}"))
        self.w_down = get(f"{p}.{name('down')}").contiguous()

    def forward(self, x, batch):
        ops = self.ctx.ops
        product = ops.linear_auto                                # partial sums for a few tokens, else [M, N]
        how = {} if self.spec.activation == "silu" else {"activation": self.spec.activation}
        if self.spec.activation == "swish_clamped":
            how.update(limit=self.spec.limit, alpha=self.spec.alpha)
        few = ops.swiglu_skinny_need(x.shape[0], self.spec.intermediate_size, self.spec.hidden_size, x.dtype, self.block)
        if few is not None and batch.workspace is not None:
            # a few tokens: one kernel streams the fused matrix and applies the activation and the product to its own sums
            act = ops.swiglu_skinny(x, self.w_gate_up, self.block, batch.workspace.floats("swiglu", few[0]),
                                    batch.workspace.counters("swiglu", few[1]), **how)
        elif self.block and ops.gate_up_fused_pays(x.shape[0], self.w_gate_up.shape[0]) and ops.gemm_tc_takes(x, self.w_gate_up):
            act = ops.gemm_tc(x, self.w_gate_up, silu_mul_block=True, **how)
        else:
            act = ops.silu_mul(product(x, self.w_gate_up), x.dtype, block=self.block, **how)
        return product(act, self.w_down)


@dataclass(frozen=True)
class DenseMLPSpec:
    """The plain (ungated) feed-forward ``down(act(up(x)))``, no bias; ``activation``: "relu2" (the square of
    max(., 0)), "gelu_tanh" or "silu"."""

    hidden_size: int
    intermediate_size: int
    kind: str = "dense_mlp"
    activation: str = "relu2"
    names: Optional[Tuple[Tuple[str, str], ...]] = None     # names of the up and down weights under the part's prefix

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, f"{role}_proj.weight")


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    def __init__(self, spec: DenseMLPSpec, prefix: str, ctx: BuildContext):
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_up = self.w_down = None

    def tensors(self) -> Dict[str, TensorSpec]:
        h, i, p, n = self.spec.hidden_size, self.spec.intermediate_size, self.prefix, self.spec.name
        return {f"{p}.{n('up')}": TensorSpec((i, h)), f"{p}.{n('down')}": TensorSpec((h, i))}

    def load(self, get) -> None:
        self.w_up = get(f"{self.prefix}.{self.spec.name('up')}").contiguous()
        self.w_down = get(f"{self.prefix}.{self.spec.name('down')}").contiguous()

    def forward(self, x, batch):
        ops = self.ctx.ops
        # the product with the activation in its epilogue where a kernel of that form takes the shape; else the
        # product (whole, or float32 partial sums for a few tokens) and the activation as a pass of its own
        act = ops.linear_activation(x, self.w_up, self.spec.activation)
        return ops.linear_auto(act, self.w_down)
