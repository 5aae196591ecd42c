"""Grouped-query attention over the paged cache.

q, k and v come from one product with the stacked matrix ``[q rows | k rows | v rows]``; one fused
kernel then normalises each q and k head (when ``qk_norm``), rotates them by the position tables,
leaves q in a buffer and writes k and v into the token's page; attention runs over the cache
(split-key decode kernel for requests that bring one token, prefill kernel for portions); the
output projection closes the part.  Options of the spec: a value head size of its own (``v_head_dim``), scores soft-capped
to ``softcap * tanh(score / softcap)``, an output gate (the concatenated heads times ``sigmoid(W_g x)`` ahead of the
output projection, W_g reading the mixer's input), rotation of interleaved pairs (the rows of the q and k projections
are reordered once at load time, see ``rope.pairing_order``), and the checkpoint's own tensor names.  How a step's attention is cut (key ranges, kernel forms, tile
lists) is this part's own plan, made once a step from the batch's host fields by asking the kernels
(``ops.plan_decode_attention``, ``ops.prefill_tile_rows``, ``ops.prefill_tiles``); the step function
knows nothing of it.  Sizes, eps, scale, window and the position encoding are
parameters of the spec; nothing here knows which model it serves.

Formulas: lily/models/llama.py:50-90 (projections, scale = head_dim^-0.5 unless the spec gives
one), lily/models/qwen3.py:17-32 (per-head q/k RMSNorm before the rotation),
lily/layers/attention/triton_backend.py:110-141 (cache write before attention).
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, CacheNeed, Mixer, StateNeed, TensorSpec, build_part, register_part


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: bool = False
    norm_eps: float = 1e-6
    bias: bool = False
    window: Optional[int] = None          # None: all keys; n: the last n keys
    scale: Optional[float] = None         # None: head_dim ** -0.5
    position: Any = None                  # a position spec (e.g. RopeSpec) or None
    kind: str = "attention"
    v_head_dim: Optional[int] = None      # None: head_dim
    softcap: Optional[float] = None       # scores become softcap * tanh(score * scale / softcap)
    out_gate: bool = False                # heads * sigmoid(W_g x) before the output projection
    # names of the tensors under the part's prefix: q, k, v, o (and g) weights; None: "<x>_proj.weight"
    # (the convolution's weights: roles "q_conv", "k_conv", "v_conv", default "<x>_proj.conv")
    names: Optional[Tuple[Tuple[str, str], ...]] = None
    keep_first: int = 0                   # with a window: key j is also seen when j < keep_first
    conv_taps: int = 0                    # 0: none; n: y_t = sum_j w[:, j] u_(t - n + 1 + j) on each channel of q, k and v
    out_bias: bool = True                 # with ``bias``: the output projection has one too
    sink: bool = False                    # weights exp(s_j) / (1 + sum exp(s_j)): a key of score 0 that has no value
    talk: bool = False                    # weights_h <- sum_g T[h, g] weights_g with T the tensor of role "talk" [heads, heads]
    v_norm: bool = False                  # each value head divided by its root mean square (norm_eps, no gain), cached so
    # "first": this layer's (normed) values are kept for the step; "blend": the cached value is
    # (1 - lambda) v + lambda v_first with lambda the scalar tensor of role "v_blend" and v_first the kept values of
    # the same token; layers that share have one kv_heads x v_head_dim
    v_share: Optional[str] = None

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim

    def name(self, role: str) -> str:
        if role.endswith("_conv"):
            default = f"{role[0]}_proj.conv"
        elif role.endswith("_bias"):
            default = f"{role[0]}_proj.bias"
        elif role.endswith("_norm"):
            default = f"{role[0]}_norm.weight"
        else:
            default = f"{role}_proj.weight" if role in ("q", "k", "v", "o", "g") else role
        return dict(self.names or ()).get(role, default)

    @property
    def projected(self) -> int:
        """Columns of the stacked q, k and v projections."""
        return (self.num_heads + self.num_kv_heads) * self.head_dim + self.num_kv_heads * self.value_dim


@dataclass
class AttentionPlan:
    """One step's attention for one set of sizes: the decode rows' plan (``ops.plan_decode_attention``) and,
    when requests bring portions, the prefill kernel's tile height and its (request, offset) lists."""

    decode: Any
    tile_rows: Optional[int]
    tiles: Any


@dataclass
class LayerCache:
    """The cache one run of a mixer reads and writes: its group and its layer's pages."""

    group: int
    data: torch.Tensor            # [pages + 1, 2, kv_heads, page_size, head_dim], or flat pages when values have a
                                  # head size of their own (``ops.cache_layer_fits``)


@register_part("mixer", "attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: AttentionSpec, prefix: str, ctx: BuildContext):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not group over {spec.num_kv_heads} kv heads")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5
        self.position = build_part("position", spec.position, prefix, ctx) if spec.position is not None else None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_gain = self.k_gain = self.w_g = None
        if spec.v_share not in (None, "first", "blend"):
            raise ValueError(f"values are shared as 'first' or 'blend', not {spec.v_share!r}")
        if (spec.sink or spec.talk or spec.v_norm or spec.v_share) and (spec.conv_taps or spec.softcap or spec.window or spec.out_gate):
            raise ValueError("sink, mixed heads and normed or shared values come without convolution, cap, window and gate")
        self.talk = None
        self.v_blend = None
        if spec.keep_first and not spec.window:
            raise ValueError("first positions are kept in sight only beside a window")
        if spec.conv_taps < 0 or (spec.conv_taps and spec.bias):
            raise ValueError("the short convolution has at least one tap and comes without biases")
        self.conv_w = None

    # ---- what it needs ----------------------------------------------------------

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(s.num_kv_heads, s.head_dim, s.window, None if s.value_dim == s.head_dim else s.value_dim,
                         keep_first=int(s.keep_first) if s.window else 0)

    def state_need(self) -> Optional[StateNeed]:
        s = self.spec
        if s.conv_taps > 1:
            return StateNeed(((s.conv_taps - 1) * s.projected,), torch.float32)      # the last projected rows, oldest first
        return None

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        heads_out = s.num_heads * s.value_dim
        out = {f"{p}.{s.name('q')}": TensorSpec((q, s.hidden_size)),
               f"{p}.{s.name('k')}": TensorSpec((kv, s.hidden_size)),
               f"{p}.{s.name('v')}": TensorSpec((s.num_kv_heads * s.value_dim, s.hidden_size)),
               f"{p}.{s.name('o')}": TensorSpec((s.hidden_size, heads_out))}
        if s.out_gate:
            out[f"{p}.{s.name('g')}"] = TensorSpec((heads_out, s.hidden_size))
        if s.conv_taps:
            out.update({f"{p}.{s.name('q_conv')}": TensorSpec((q, s.conv_taps), role="vector", init="normal"),
                        f"{p}.{s.name('k_conv')}": TensorSpec((kv, s.conv_taps), role="vector", init="normal"),
                        f"{p}.{s.name('v_conv')}": TensorSpec((s.num_kv_heads * s.value_dim, s.conv_taps), role="vector", init="normal")})
        if s.bias:
            out.update({f"{p}.{s.name('q_bias')}": TensorSpec((q,), role="matrix"),
                        f"{p}.{s.name('k_bias')}": TensorSpec((kv,), role="matrix"),
                        f"{p}.{s.name('v_bias')}": TensorSpec((s.num_kv_heads * s.value_dim,), role="matrix")})
            if s.out_bias:
                out[f"{p}.{s.name('o_bias')}"] = TensorSpec((s.hidden_size,), role="matrix")
        if s.qk_norm:
            out.update({f"{p}.{s.name('q_norm')}": TensorSpec((s.head_dim,), role="vector", init="gain"),
                        f"{p}.{s.name('k_norm')}": TensorSpec((s.head_dim,), role="vector", init="gain")})
        if s.talk:
            out[f"{p}.{s.name('talk')}"] = TensorSpec((s.num_heads, s.num_heads), role="vector", init="mixing")
        if s.v_share:
            out[f"{p}.{s.name('v_blend')}"] = TensorSpec((), role="vector", init="half")
        return out

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        wq, wk = get(f"{p}.{s.name('q')}"), get(f"{p}.{s.name('k')}")
        if self.position is not None and getattr(self.position, "interleaved", False):
            # pairs (2i, 2i + 1) become (i, i + rotary_dim / 2) in every q and k head alike: the scores are the same
            from lily_b200.parts.rope import pairing_order
            order = pairing_order(s.head_dim, self.position.rotary_dim).to(wq.device)
            wq = wq.view(s.num_heads, s.head_dim, -1)[:, order].reshape(q, -1)
            wk = wk.view(s.num_kv_heads, s.head_dim, -1)[:, order].reshape(kv, -1)
        self.w_qkv = torch.empty((q + kv + s.num_kv_heads * s.value_dim, s.hidden_size), dtype=wq.dtype, device=wq.device)
        self.w_qkv[:q].copy_(wq)
        self.w_qkv[q:q + kv].copy_(wk)
        del wq, wk
        self.w_qkv[q + kv:].copy_(get(f"{p}.{s.name('v')}"))
        self.w_o = get(f"{p}.{s.name('o')}").contiguous()
        if s.out_gate:
            self.w_g = get(f"{p}.{s.name('g')}").contiguous()
        if s.conv_taps:
            wc = [get(f"{p}.{s.name(r)}").float() for r in ("q_conv", "k_conv", "v_conv")]
            if self.position is not None and getattr(self.position, "interleaved", False):
                wc[0] = wc[0].view(s.num_heads, s.head_dim, -1)[:, order].reshape(q, -1)
                wc[1] = wc[1].view(s.num_kv_heads, s.head_dim, -1)[:, order].reshape(kv, -1)
            self.conv_w = torch.cat(wc).contiguous()                       # [q | k | v channels, taps], float32
        if s.bias:
            self.b_qkv = torch.cat([get(f"{p}.{s.name(n + '_bias')}") for n in "qkv"]).contiguous()
            if s.out_bias:
                self.b_o = get(f"{p}.{s.name('o_bias')}").contiguous()
        if s.talk:
            self.talk = get(f"{p}.{s.name('talk')}").float().contiguous()        # the weights and their mixing are float32
        if s.v_share:
            blend = get(f"{p}.{s.name('v_blend')}")                              # the first layer's is loaded and not used
            self.v_blend = float(blend.float().item()) if s.v_share == "blend" else None
        if s.qk_norm:
            self.q_gain = get(f"{p}.{s.name('q_norm')}")
            self.k_gain = get(f"{p}.{s.name('k_norm')}")
            if self.q_gain.dtype != self.k_gain.dtype:
                self.q_gain, self.k_gain = self.q_gain.float(), self.k_gain.float()

    # ---- one step ----------------------------------------------------------------

    def _plan(self, batch, group: int, dtype, page: int):
        """How this step's attention runs for this mixer's sizes in cache group ``group``; made once a step and
        shared by every layer with the same sizes (``batch.plan``)."""
        s, ops = self.spec, self.ctx.ops
        key = ("attention", group, s.num_heads, s.num_kv_heads, s.head_dim, dtype, page, s.value_dim, bool(s.softcap),
               bool(s.keep_first), bool(s.conv_taps), s.sink, s.talk)
        sized = {} if s.value_dim == s.head_dim else {"dv": s.value_dim}      # options go to the kernels' faces only
        capped = {"softcap": s.softcap} if s.softcap else {}                  # where the spec sets them
        if s.keep_first:
            sized = dict(sized, keep_first=int(s.keep_first))
        tiled = dict(sized)
        if s.sink or s.talk:
            tiled = dict(tiled, sink=s.sink, all_values=s.talk)
            if not ops.sink_on_tensor_cores(dtype, s.head_dim, s.value_dim):
                # options of the CUDA-core kernels; with mixed heads a query head's output row spans all kv heads' values
                # (unless those come as a plane a kv head)
                wide = s.talk and not ops.all_values_in_planes(dtype, s.num_kv_heads, s.head_dim, s.value_dim)
                sized = dict(sized, cuda_cores=True, dv=s.num_kv_heads * s.value_dim if wide else s.value_dim)
            else:
                sized = dict(sized, fusable=False)      # one launch a kv head of the mma.sync kernel, queries prepared ahead

        def make(b):
            nd = b.num_decode
            # the rows the decode kernel sees (with mixed heads it may run every kv head's values in one launch)
            seen = ops.all_values_decode_rows(dtype, nd, s.num_kv_heads, s.head_dim, s.value_dim) if s.talk else nd
            decode = ops.plan_decode_attention(dtype, seen, s.num_heads, s.num_kv_heads, s.head_dim, b.max_decode_len,
                                               even=b.decode_even, **sized)
            if decode != ops.plan_decode_attention(dtype, seen, s.num_heads, s.num_kv_heads, s.head_dim, b.max_decode_len,
                                                   even=not b.decode_even, **sized):
                b.even_asked = True              # a captured step with this plan serves batches of this kind only
            if (s.conv_taps or s.v_norm or s.v_share) and decode.fused:
                # something stands between projection and rotation, or the values are not cached as projected
                decode = dataclasses.replace(decode, fused=False)
            rows = tiles = None
            if b.num_requests > nd:
                rows = ops.prefill_tile_rows(dtype, s.head_dim, page, b.num_tokens - nd, **capped, **tiled)
                tiles = ops.prefill_tiles(b.h_prefix_lens, b.h_new_lens, nd, rows, b.token_ids.device)
            return AttentionPlan(decode, rows, tiles)
        return batch.plan(key, make)

    def forward(self, x, batch, cache: LayerCache, state=None, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        page = self.ctx.page_size
        dv = s.value_dim
        sized = {} if dv == s.head_dim else {"dv": dv}
        capped = {"softcap": s.softcap} if s.softcap else {}
        kept = {"keep_first": int(s.keep_first)} if s.keep_first else {}
        if s.sink or s.talk:
            kept = dict(kept, sink=s.sink, all_values=s.talk)
        table = batch.block_tables[cache.group]
        plan = self._plan(batch, cache.group, cache.data.dtype, page)
        if s.conv_taps:
            chunk = ops.SSM_CHUNK
            chunk_req, chunk_start = batch.plan(("token_chunks", chunk),
                                                lambda b: ops.token_chunks(b.h_new_lens, chunk, b.token_ids.device))
            qkv = ops.causal_conv(ops.linear(x, self.w_qkv), 0, s.projected, self.conv_w, None, state, 0, chunk_req,
                                  chunk_start, batch.cu_seqlens, batch.slots, chunk, activation="none")
        else:
            qkv = ops.linear_auto(x, self.w_qkv, self.b_qkv)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        nd, dec = batch.num_decode, plan.decode
        scratch = batch.workspace.floats("attention_decode", dec.scratch_floats) if nd and dec.scratch_floats else None
        gate = ops.linear_auto(x, self.w_g) if s.out_gate else None
        if nd == batch.num_tokens and dec.fused:
            # every request brings one token: the decode attention kernel finishes q, k and v itself
            out = torch.empty((nd, s.num_heads * s.head_dim), dtype=cache.data.dtype, device=cache.data.device)
            ops.attention_decode_fused(qkv, self.q_gain, self.k_gain, s.norm_eps, cos, sin, cache.data, table, batch.seq_lens,
                                       out, scratch, dec.splits, s.num_heads, s.num_kv_heads, s.head_dim, rotary_dim, page,
                                       self.scale, s.window, write_kv=write_cache, stages=dec.stages, **capped)
            if gate is not None:
                ops.sigmoid_gate(out, gate)
            return ops.linear_auto(out, self.w_o, self.b_o)
        values = {}
        if s.v_norm or s.v_share:
            values = {"v_norm": s.v_norm}
            if s.v_share:
                # the first sharing layer's values of this step's tokens, float32; the layers behind it read them
                cols = s.num_kv_heads * dv
                values["v_keep"] = batch.plan(("first_values", cols), lambda b: torch.empty((b.num_tokens, cols), dtype=torch.float32,
                                                                                             device=x.device))
                if s.v_share == "blend":
                    values["v_blend"] = self.v_blend
        q = ops.qk_norm_rope_write(qkv, self.q_gain, self.k_gain, s.norm_eps, cos, sin, batch.positions,
                                   batch.token_req, table, cache.data, s.num_heads, s.num_kv_heads, s.head_dim,
                                   rotary_dim, page, write_kv=write_cache, **sized, **values)
        if s.talk:
            out = ops.all_values_sums(q.dtype, q.shape[0], s.num_heads, s.num_kv_heads, s.head_dim, dv, q.device)
        else:
            out = torch.empty((q.shape[0], s.num_heads * dv), dtype=q.dtype, device=q.device)
        planes = out.dim() == 3                          # a plane a kv head (the mma.sync kernels) instead of wider rows
        if nd:
            # (the one-token requests' rows are the first of every plane)
            ops.attention_decode(q[:nd], cache.data, table, batch.seq_lens, out if planes else out[:nd], scratch, dec.splits,
                                 s.num_heads, s.num_kv_heads, s.head_dim, page, self.scale, s.window, stages=dec.stages,
                                 **capped, **sized, **kept)
        if batch.num_requests > nd:
            tile_req, tile_start = plan.tiles
            ops.attention_prefill(q, cache.data, table, batch.cu_seqlens, batch.prefix_lens, tile_req, tile_start,
                                  out, s.num_heads, s.num_kv_heads, s.head_dim, page, self.scale, s.window,
                                  tile_rows=plan.tile_rows, **capped, **sized, **kept)
        if gate is not None:
            ops.sigmoid_gate(out, gate)
        if s.talk:
            out = ops.head_mix(out, self.talk, s.num_heads, s.num_kv_heads, dv, q.dtype)
        return ops.linear_auto(out, self.w_o, self.b_o)
