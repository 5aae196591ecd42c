"""A state-space mixer of the first Mamba kind (selective scan), with its state in the request's slot.

One projection of the input gives ``[x | z]`` (``inner`` columns each).  x passes a short causal convolution per
channel (with bias) and SiLU; a second projection of the result gives ``[dt | B | C]`` (``dt_rank``, ``state``,
``state`` columns), and ``dt`` is projected up to a step size per channel, ``softplus(W_dt dt + bias)``.  Per channel c
and state entry n, with ``A = -exp(A_log)`` of shape ``inner x state``,

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,        y_c = sum_n S[c, n] C_n + D_c x_c

then ``y * silu(z)`` is projected out.

What a request carries from step to step is one float32 row of its slot (``StateNeed``): the scan state
``[inner, state]`` followed by the convolution's last ``taps - 1`` inputs ``[(taps - 1), inner]``.  The kernels reach it
through ``batch.slots`` on the device, so a step in which every request brings one token can be captured in a CUDA
graph (``graph_safe``); a portion of a prompt continues from the same row, whatever its length.  The step size (from the
step projection's float32 result on), the decay, the state and the sums over it are float32 in both precisions.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, Mixer, StateNeed, TensorSpec, register_part


@dataclass(frozen=True)
class SelectiveScanSpec:
    hidden_size: int
    inner: int
    state: int
    dt_rank: int
    conv_taps: int
    kind: str = "selective_scan"
    # names of the tensors under the part's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("x", "x"), ("dt", "dt"), ("dt_bias", "dt.b"),
                 ("A_log", "A_log"), ("D", "D"), ("o", "o"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def low(self) -> int:
        """Columns of the second projection: dt, B and C."""
        return self.dt_rank + 2 * self.state


@register_part("mixer", "selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True

    def __init__(self, spec: SelectiveScanSpec, prefix: str, ctx: BuildContext):
        if min(spec.inner, spec.state, spec.dt_rank) < 1 or spec.conv_taps < 1:
            raise ValueError("inner, state, dt_rank and the taps are positive")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_in = self.w_x = self.w_dt = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a = self.d_skip = None

    # ---- what it needs ----------------------------------------------------------

    @property
    def scan_floats(self) -> int:
        return self.spec.inner * self.spec.state

    def state_need(self) -> StateNeed:
        s = self.spec
        return StateNeed((self.scan_floats + (s.conv_taps - 1) * s.inner,), torch.float32)

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        n = lambda role: f"{p}.{s.name(role)}"
        return {n("in"): TensorSpec((2 * s.inner, s.hidden_size)),
                n("conv"): TensorSpec((s.inner, s.conv_taps), role="vector", init="normal"),
                n("conv_bias"): TensorSpec((s.inner,), role="vector", init="zeros"),
                n("x"): TensorSpec((s.low, s.inner)), n("dt"): TensorSpec((s.inner, s.dt_rank)),
                n("dt_bias"): TensorSpec((s.inner,), role="vector", init="normal"),
                n("A_log"): TensorSpec((s.inner, s.state), role="vector", init="normal"),
                n("D"): TensorSpec((s.inner,), role="vector", init="gain"),
                n("o"): TensorSpec((s.hidden_size, s.inner))}

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        g = lambda role: get(f"{p}.{s.name(role)}")
        self.w_in = g("in").contiguous()
        self.w_x = g("x").contiguous()
        self.w_o = g("o").contiguous()
        # the step projection reads the first dt_rank columns of [dt | B | C]: its matrix is widened with zero columns
        # so that it takes the second projection's rows as they are (the sums are the same)
        w_dt = g("dt")
        self.w_dt = torch.zeros((s.inner, s.low), dtype=w_dt.dtype, device=w_dt.device)
        self.w_dt[:, :s.dt_rank].copy_(w_dt)
        # what enters the recurrence (or its short convolution) is held in float32
        self.conv_w = g("conv").float().contiguous()
        self.conv_b = g("conv_bias").float().contiguous()
        self.dt_bias = g("dt_bias").float().contiguous()
        self.a = (-torch.exp(g("A_log").float())).contiguous()
        self.d_skip = g("D").float().contiguous()

    # ---- one step ----------------------------------------------------------------

    def forward(self, x, batch, cache, state, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        chunk = ops.SSM_CHUNK
        chunk_req, chunk_start = batch.plan(("token_chunks", chunk),
                                            lambda b: ops.token_chunks(b.h_new_lens, chunk, b.token_ids.device))
        proj = ops.linear(x, self.w_in)                                       # [tokens, x | z]
        xc = ops.causal_conv_silu(proj, 0, s.inner, self.conv_w, self.conv_b, state, self.scan_floats, chunk_req,
                                  chunk_start, batch.cu_seqlens, batch.slots, chunk)
        low = ops.linear(xc, self.w_x)                                        # [tokens, dt | B | C]
        step = ops.linear(low, self.w_dt, self.dt_bias, out_dtype=torch.float32)
        # long portions run as chunks side by side; the cut is planned once a step for layers of one state size
        plan = batch.plan(("scan_plan", self.scan_floats),
                          lambda b: ops.scan_plan(b.h_new_lens, b.token_ids.device, self.scan_floats))
        need = ops.selective_workspace_floats(plan, s.inner, s.state)
        room = batch.workspace.floats("selective_chunks", need) if need and batch.workspace is not None else None
        if need and room is None:
            plan = None                                    # no scratch to be had: every portion runs whole
        gated = ops.selective_scan(xc, low, s.dt_rank, step, proj, s.inner, self.a, self.d_skip, state, batch.cu_seqlens,
                                   batch.slots, batch.num_requests, plan=plan, workspace=room)
        return ops.linear_auto(gated, self.w_o)
