"""Differential attention over the paged cache.

Every query head carries two softmax attention maps with queries and keys of their own over the same values; the head's
output is their difference ``a1 - lambda a2`` (one ``lambda`` for the layer), divided by its root mean square over the
value head's columns, times ``1 - lambda_init``, times ``sigmoid`` of one gate number per head that a projection of
the mixer's input gives.  Queries are multiplied by a temperature that grows with the logarithm of the position,
``1 + coef ln(floor((p + 1) / every) + 1)``; there is no rotation.  Scores may be soft-capped.

How it runs on the kernels the plain attention uses.  The rows of the q projection are ``[head][map][dim]`` and those
of the k projection ``[kv head][map][dim]``.  A kv head's cached key row is its two maps' keys side by side
(``2 dim`` columns); map m of head h becomes query head ``2 h + m`` of ``2 dim`` columns that are zero outside the
map's own half, so its scores over the whole key row are exactly the map's scores, and the grouping of query heads
over kv heads is the ordinary one.  ``diff_prepare`` scales the queries, lays them out that way and writes keys and
values to the token's page; the attention kernels (decode in key ranges, prefill in tiles) see an attention of
``2 heads`` query heads; ``diff_combine`` forms the difference, the unit norm and the gate.  One product gives q, k, v
and the gate numbers.  ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init`` is formed once, in float64, when the
four vectors are loaded.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.attention import AttentionPlan, LayerCache
from lily_b200.parts.base import BuildContext, CacheNeed, Mixer, TensorSpec, register_part

MAPS = 2          # attention maps a head combines


@dataclass(frozen=True)
class DiffAttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int                          # query / key size of one map
    v_head_dim: int
    scale: float
    lambda_init: float                     # added to the difference of the exponentials; the output is times 1 - this
    norm_eps: float
    softcap: Optional[float] = None
    q_temp_coef: float = 0.0               # 0: queries are not scaled by position
    q_temp_every: int = 1
    kind: str = "differential_attention"
    # names of the tensors under the part's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = (("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"), ("o", "o_proj.weight"),
                 ("g", "g_proj.weight"), ("lq1", "lambda_q1"), ("lk1", "lambda_k1"), ("lq2", "lambda_q2"), ("lk2", "lambda_k2"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def key_dim(self) -> int:
        """Columns of a kv head's cached key row: its maps' keys side by side."""
        return MAPS * self.head_dim


@register_part("mixer", "differential_attention")
class DifferentialAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: DiffAttentionSpec, prefix: str, ctx: BuildContext):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not group over {spec.num_kv_heads} kv heads")
        if spec.q_temp_coef and spec.q_temp_every < 1:
            raise ValueError("the query temperature steps every positive number of positions")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_in = self.w_o = None
        self.lam = 0.0

    # ---- what it needs ----------------------------------------------------------

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(s.num_kv_heads, s.key_dim, None, None if s.v_head_dim == s.key_dim else s.v_head_dim)

    @property
    def columns(self) -> Tuple[int, int, int, int]:
        """Widths of the q, k, v and gate parts of the stacked projection."""
        s = self.spec
        return s.num_heads * s.key_dim, s.num_kv_heads * s.key_dim, s.num_kv_heads * s.v_head_dim, s.num_heads

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        q, k, v, g = self.columns
        out = {f"{p}.{s.name('q')}": TensorSpec((q, s.hidden_size)), f"{p}.{s.name('k')}": TensorSpec((k, s.hidden_size)),
               f"{p}.{s.name('v')}": TensorSpec((v, s.hidden_size)), f"{p}.{s.name('g')}": TensorSpec((g, s.hidden_size)),
               f"{p}.{s.name('o')}": TensorSpec((s.hidden_size, s.num_heads * s.v_head_dim))}
        for role in ("lq1", "lk1", "lq2", "lk2"):
            out[f"{p}.{s.name(role)}"] = TensorSpec((s.head_dim,), role="vector", init="normal")
        return out

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        q, k, v, g = self.columns
        wq = get(f"{p}.{s.name('q')}")
        self.w_in = torch.empty((q + k + v + g, s.hidden_size), dtype=wq.dtype, device=wq.device)
        at = 0
        for role, rows in (("q", q), ("k", k), ("v", v), ("g", g)):
            self.w_in[at:at + rows].copy_(wq if role == "q" else get(f"{p}.{s.name(role)}"))
            at += rows
        del wq
        self.w_o = get(f"{p}.{s.name('o')}").contiguous()
        lq1, lk1, lq2, lk2 = (get(f"{p}.{s.name(r)}").double().cpu() for r in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + float(s.lambda_init)

    # ---- one step ----------------------------------------------------------------

    def _plan(self, batch, group: int, dtype, page: int):
        """As the plain attention's plan, for ``MAPS * heads`` query heads of ``key_dim`` columns."""
        s, ops = self.spec, self.ctx.ops
        nq, d, dv = MAPS * s.num_heads, s.key_dim, s.v_head_dim
        key = ("attention", group, nq, s.num_kv_heads, d, dtype, page, dv, bool(s.softcap), False, True)
        sized = {} if dv == d else {"dv": dv}
        capped = {"softcap": s.softcap} if s.softcap else {}

        def make(b):
            nd = b.num_decode
            decode = ops.plan_decode_attention(dtype, nd, nq, s.num_kv_heads, d, b.max_decode_len, even=b.decode_even,
                                               fusable=False, **sized)
            if decode != ops.plan_decode_attention(dtype, nd, nq, s.num_kv_heads, d, b.max_decode_len,
                                                   even=not b.decode_even, fusable=False, **sized):
                b.even_asked = True
            rows = tiles = None
            if b.num_requests > nd:
                rows = ops.prefill_tile_rows(dtype, d, page, b.num_tokens - nd, **capped, **sized)
                tiles = ops.prefill_tiles(b.h_prefix_lens, b.h_new_lens, nd, rows, b.token_ids.device)
            return AttentionPlan(decode, rows, tiles)
        return batch.plan(key, make)

    def forward(self, x, batch, cache: LayerCache, state=None, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        page = self.ctx.page_size
        nq, nkv, d, dv = MAPS * s.num_heads, s.num_kv_heads, s.key_dim, s.v_head_dim
        sized = {} if dv == d else {"dv": dv}
        capped = {"softcap": s.softcap} if s.softcap else {}
        table = batch.block_tables[cache.group]
        plan = self._plan(batch, cache.group, cache.data.dtype, page)
        proj = ops.linear(x, self.w_in)                                        # [tokens, q | k | v | gate]
        q = ops.diff_prepare(proj, batch.positions, batch.token_req, table, cache.data, s.num_heads, nkv, s.head_dim, dv,
                             MAPS, page, s.q_temp_coef, s.q_temp_every, write_kv=write_cache)
        maps_out = torch.empty((q.shape[0], nq * dv), dtype=q.dtype, device=q.device)
        nd, dec = batch.num_decode, plan.decode
        if nd:
            scratch = batch.workspace.floats("attention_decode", dec.scratch_floats) if dec.scratch_floats else None
            ops.attention_decode(q[:nd], cache.data, table, batch.seq_lens, maps_out[:nd], scratch, dec.splits, nq, nkv, d,
                                 page, s.scale, None, stages=dec.stages, **capped, **sized)
        if batch.num_requests > nd:
            tile_req, tile_start = plan.tiles
            ops.attention_prefill(q, cache.data, table, batch.cu_seqlens, batch.prefix_lens, tile_req, tile_start, maps_out,
                                  nq, nkv, d, page, s.scale, None, tile_rows=plan.tile_rows, **capped, **sized)
        q_cols, k_cols, v_cols, _ = self.columns
        out = ops.diff_combine(maps_out, proj, q_cols + k_cols + v_cols, s.num_heads, dv, MAPS, self.lam,
                               1.0 - s.lambda_init, s.norm_eps)
        return ops.linear_auto(out, self.w_o)
