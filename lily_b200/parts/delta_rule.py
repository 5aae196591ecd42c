"""A linear-attention mixer that writes by the gated delta rule, with its state in the request's slot.

One projection of the input gives ``[q | k | v | gate | beta | alpha]``: q and k with ``kv_heads`` heads of ``head_dim``,
v and the gate with ``heads`` heads of ``v_head_dim`` (value head h reads query/key head ``h // (heads / kv_heads)``),
beta and alpha one number a value head.  q, k and v pass a short causal convolution per channel (no bias) and SiLU;
q and k are then made unit vectors per head (``x / sqrt(sum x^2 + unit_eps)``; q also times ``head_dim^-0.5``).  Per
value head, with S a ``head_dim x v_head_dim`` matrix that is zero when the request starts,
``a_t = exp(-exp(A_log) softplus(alpha_t + dt_bias))`` and ``b_t = sigmoid(beta_t)``:

    S <- a_t S;    u = b_t (v_t - S^T k_t);    S <- S + k_t u^T;    o_t = S^T q_t       (read out after the write)

then each head's o is divided by its root mean square, multiplied by a gain that all heads share and by ``silu(gate)``,
and projected out.

What a request carries from step to step is one float32 row of its slot (``StateNeed``): the heads' matrices
``[heads, v_head_dim, head_dim]`` followed by the convolution's last ``taps - 1`` inputs ``[(taps - 1), channels]``.  The
kernels reach it through ``batch.slots`` on the device, so a step in which every request brings one token can be
captured in a CUDA graph (``graph_safe``); a portion of a prompt continues from the same row, whatever its length.
Decay, write strength, unit vectors, the state, the sums over it and the unit norm by head are float32 in both
precisions.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, Mixer, StateNeed, TensorSpec, register_part


@dataclass(frozen=True)
class DeltaRuleSpec:
    hidden_size: int
    heads: int
    kv_heads: int
    head_dim: int
    v_head_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    kind: str = "delta_rule"
    # names of the tensors under the part's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = (("q", "q"), ("k", "k"), ("v", "v"), ("q_conv", "q.conv"), ("k_conv", "k.conv"), ("v_conv", "v.conv"),
                 ("beta", "b"), ("alpha", "a"), ("A_log", "A_log"), ("dt_bias", "dt_bias"), ("norm", "norm"), ("gate", "g"),
                 ("o", "o"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def key_columns(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def inner(self) -> int:
        return self.heads * self.v_head_dim

    @property
    def channels(self) -> int:
        """Columns that pass the convolution: q, k and v."""
        return 2 * self.key_columns + self.inner

    @property
    def projected(self) -> int:
        return self.channels + self.inner + 2 * self.heads


@register_part("mixer", "delta_rule")
class DeltaRule(Mixer):
    graph_safe = True

    def __init__(self, spec: DeltaRuleSpec, prefix: str, ctx: BuildContext):
        if min(spec.heads, spec.kv_heads, spec.head_dim, spec.v_head_dim) < 1 or spec.heads % spec.kv_heads:
            raise ValueError(f"{spec.heads} value heads do not group over {spec.kv_heads} query/key heads")
        if spec.conv_taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_in = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.gain = None

    # ---- what it needs ----------------------------------------------------------

    @property
    def matrix_floats(self) -> int:
        return self.spec.heads * self.spec.head_dim * self.spec.v_head_dim

    def state_need(self) -> StateNeed:
        s = self.spec
        return StateNeed((self.matrix_floats + (s.conv_taps - 1) * s.channels,), torch.float32)

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        n = lambda role: f"{p}.{s.name(role)}"
        return {n("q"): TensorSpec((s.key_columns, s.hidden_size)), n("k"): TensorSpec((s.key_columns, s.hidden_size)),
                n("v"): TensorSpec((s.inner, s.hidden_size)),
                n("q_conv"): TensorSpec((s.key_columns, s.conv_taps), role="vector", init="normal"),
                n("k_conv"): TensorSpec((s.key_columns, s.conv_taps), role="vector", init="normal"),
                n("v_conv"): TensorSpec((s.inner, s.conv_taps), role="vector", init="normal"),
                n("beta"): TensorSpec((s.heads, s.hidden_size)), n("alpha"): TensorSpec((s.heads, s.hidden_size)),
                n("A_log"): TensorSpec((s.heads,), role="vector", init="normal"),
                n("dt_bias"): TensorSpec((s.heads,), role="vector", init="normal"),
                n("norm"): TensorSpec((s.v_head_dim,), role="vector", init="gain"),
                n("gate"): TensorSpec((s.inner, s.hidden_size)), n("o"): TensorSpec((s.hidden_size, s.inner))}

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        g = lambda role: get(f"{p}.{s.name(role)}")
        # one product for everything that reads the mixer's input: [q | k | v | gate | beta | alpha]
        self.w_in = torch.cat([g(r) for r in ("q", "k", "v", "gate", "beta", "alpha")]).contiguous()
        self.w_o = g("o").contiguous()
        # what enters the recurrence (or its short convolution) is held in float32
        self.conv_w = torch.cat([g(r).float() for r in ("q_conv", "k_conv", "v_conv")]).contiguous()
        self.a_log = g("A_log").float().contiguous()
        self.dt_bias = g("dt_bias").float().contiguous()
        self.gain = g("norm").float().repeat(s.heads).contiguous()            # one gain for all heads

    # ---- one step ----------------------------------------------------------------

    def forward(self, x, batch, cache, state, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        chunk = ops.SSM_CHUNK
        chunk_req, chunk_start = batch.plan(("token_chunks", chunk),
                                            lambda b: ops.token_chunks(b.h_new_lens, chunk, b.token_ids.device))
        proj = ops.linear(x, self.w_in)                                       # [tokens, q | k | v | gate | beta | alpha]
        qkv = ops.causal_conv_silu(proj, 0, s.channels, self.conv_w, None, state, self.matrix_floats, chunk_req,
                                   chunk_start, batch.cu_seqlens, batch.slots, chunk)
        y = ops.delta_rule(qkv, proj, s.channels + s.inner, s.channels + s.inner + s.heads, self.a_log, self.dt_bias, state,
                           batch.cu_seqlens, batch.slots, batch.num_requests, s.heads, s.kv_heads, s.head_dim, s.v_head_dim,
                           s.unit_eps, s.head_dim ** -0.5)
        gate = proj[:, s.channels:s.channels + s.inner]
        normed = ops.group_rmsnorm_gate(y, gate, self.gain, s.heads, s.norm_eps)
        return ops.linear_auto(normed, self.w_o)
