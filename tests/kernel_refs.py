"""Plain PyTorch statements of what each CUDA kernel computes, with the kernels' signatures.

Two uses, both in tests only: (1) each kernel is compared with its function here on the GPU, at
sizes other than the engine's; (2) handed to the engine as ``ops`` on the CPU they let the cache
manager, batch packing, step function, scheduler and replay be tested without a device.  They
compute in float32 and round once to the output dtype.  Nothing in ``lily_b200`` imports this.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

launches = {"count": 0}        # the kernels' Python faces count their launches here; these statements launch nothing
TC_MIN_ROWS = 65               # as the kernels: products of this many rows and more take the fused gate/up epilogue


def gate_up_fused_pays(rows, fused_rows):
    return rows >= TC_MIN_ROWS
FUSE_DECODE = True             # tests flip this to send all-decode steps through either form of the attention


def library():
    return None


def sm_count():
    return 148


def _sum(t):
    """Kernels that take a product take it whole or as float32 partial sums [splits, rows, cols]."""
    return t.sum(0) if t.dim() == 3 else t


def embed(table, ids, out=None, future=None, scale=1.0):
    ids = ids.long()
    if future is not None:
        ids = torch.where(ids < 0, future.long()[(-ids - 1).clamp(min=0)], ids)
    return table[ids].float() * scale


def logit_transform(logits, scale=1.0, softcap=None):
    logits.mul_(scale)
    if softcap:
        logits.copy_(softcap * torch.tanh(logits / softcap))
    return logits


def scatter_tokens(tokens, logit_rows, token_req, slots, future):
    n = tokens.numel()
    future[slots.long()[token_req.long()[logit_rows.long()[:n]]]] = tokens.to(future.dtype)


def add_rmsnorm(resid, delta, weight, eps, out_dtype, rows=None, write_residual=True, out=None):
    if delta is not None:
        delta = _sum(delta)
    if rows is not None:
        v = resid[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].float()
    else:
        if delta is not None:
            if write_residual:
                resid += delta.float()
                v = resid
            else:
                v = resid + delta.float()
        else:
            v = resid
    var = v.pow(2).mean(-1, keepdim=True)
    return ((v * torch.rsqrt(var + eps)) * weight.float()).to(out_dtype)


def add_rmsnorm_multi(resid, deltas, gains, eps, out_dtype, bias=None, write_residual=True):
    v = resid
    for d in deltas:
        if d is not None:
            v = v + _sum(d).float()
    if bias is not None:
        v = v + bias.float()
    if write_residual:
        resid.copy_(v)
    unit = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return tuple((unit * g.float()).to(out_dtype) for g in gains)


def silu_mul(gate_up, out_dtype=None, out=None, block=None, activation="silu", limit=0.0, alpha=1.0):
    out_dtype = out_dtype or gate_up.dtype
    gate_up = _sum(gate_up)
    i = gate_up.shape[1] // 2
    if block:
        runs = gate_up.view(gate_up.shape[0], i // block, 2, block)
        g, u = runs[:, :, 0].reshape(-1, i).float(), runs[:, :, 1].reshape(-1, i).float()
    else:
        g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    if activation == "gelu_tanh":
        return (0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u).to(out_dtype)
    if activation == "swish_clamped":
        g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
        return ((g / (1 + torch.exp(-alpha * g))) * (u + 1)).to(out_dtype)
    assert activation == "silu"
    return ((g / (1 + torch.exp(-g))) * u).to(out_dtype)


def _pages(kv_layer, nkv, page_size, d, dv, values_in_keys=False):
    """Views of a cache layer's keys [pages, nkv, page, d] and values [pages, nkv, page, dv] (all layouts)."""
    if kv_layer.dim() == 5:
        return kv_layer[:, 0], kv_layer[:, 1]
    if values_in_keys:
        keys = kv_layer.view(-1, nkv, page_size, d)
        return keys, keys[..., :dv]
    cut = nkv * page_size * d
    return kv_layer[:, :cut].view(-1, nkv, page_size, d), kv_layer[:, cut:].view(-1, nkv, page_size, dv)


def qk_norm_rope_write(qkv, q_gain, k_gain, eps, cos, sin, positions, token_req, block_table, kv_layer, nq, nkv, d,
                       rotary_dim, page_size, write_kv=True, q_out=None, dv=None, v_norm=False, v_keep=None, v_blend=None):
    qkv = _sum(qkv)
    n = qkv.shape[0]
    dv = dv or d
    x = qkv.float()
    q = x[:, :nq * d].view(n, nq, d)
    k = x[:, nq * d:(nq + nkv) * d].view(n, nkv, d)
    v = x[:, (nq + nkv) * d:].view(n, nkv, dv)

    def norm(t, gain):
        if gain is None:
            return t
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)) * gain.float()

    def rot(t):
        if cos is None:
            return t
        half = rotary_dim // 2
        c = cos[positions.long()].unsqueeze(1)
        s = sin[positions.long()].unsqueeze(1)
        x1, x2, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)

    q = rot(norm(q, q_gain))
    if write_kv:
        k = rot(norm(k, k_gain))
        if v_norm:
            v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        if v_keep is not None and v_blend is None:
            v_keep.copy_(v.reshape(n, nkv * dv))
        elif v_keep is not None:
            v = (1.0 - v_blend) * v + v_blend * v_keep.view(n, nkv, dv)
        pos = positions.long()
        page = block_table[token_req.long(), pos // page_size].long()
        within = pos % page_size
        keys, values = _pages(kv_layer, nkv, page_size, d, dv)
        keys[page, :, within] = k.to(kv_layer.dtype)
        values[page, :, within] = v.to(kv_layer.dtype)
    return q.reshape(n, nq * d).to(kv_layer.dtype)


def cast(x, dtype):
    return x.to(dtype)


def linear(x, weight, bias=None, out_dtype=None):
    out = x.float() @ weight.float().t()
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype or x.dtype)


def linear_split(x, weight, splits=None):
    """For a few tokens the product comes as float32 partial sums over slices of K (here: two halves)."""
    m, k = x.shape
    if m > 16 or k % 2 or (splits is not None and splits < 1):
        return None
    n = splits or 2
    if k % n:
        return None
    xs, ws = x.float().view(m, n, k // n), weight.float().view(-1, n, k // n)
    return torch.einsum("msk,nsk->smn", xs, ws).contiguous()


def linear_auto(x, weight, bias=None):
    if bias is None:
        parts = linear_split(x, weight)
        if parts is not None:
            return parts
    return linear(x, weight, bias)


def swiglu_skinny_need(tokens, intermediate, hidden, dtype, block=None, whenever_possible=False):
    return (16, 4) if dtype == torch.bfloat16 and tokens <= 8 and hidden % 64 == 0 else None


def swiglu_skinny(x, gate_up, block, scratch, counters, out=None, activation="silu", limit=0.0, alpha=1.0):
    assert int(counters.abs().sum()) == 0           # the kernel finds them zero and leaves them zero
    return silu_mul(linear(x, gate_up, out_dtype=torch.float32), x.dtype, block=block, activation=activation, limit=limit, alpha=alpha)


def logits(x, head):
    return linear(x, head, out_dtype=torch.float32)


def gate_up_interleave(dtype, intermediate):
    return 128 if dtype == torch.bfloat16 and intermediate % 128 == 0 else None


def gemm_tc_takes(x, weight):
    return x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0


def gemm_tc(x, weight, bias=None, silu_mul_block=False, activation="silu", plain_activation=None, limit=0.0, alpha=1.0):
    out = linear(x, weight, bias, out_dtype=torch.float32)
    if plain_activation:
        return _activate(out, plain_activation).to(x.dtype)
    return silu_mul(out, x.dtype, block=128, activation=activation, limit=limit, alpha=alpha) if silu_mul_block else out.to(x.dtype)


def uses_tensor_cores(dtype, d):
    return dtype == torch.bfloat16 and d in (64, 128, 192, 256)


def prefill_tile_rows(dtype=None, d=0, page_size=0, new_tokens=0, softcap=None, dv=None, values_in_keys=False, heads=0,
                      keep_first=0, sink=False, all_values=False):
    return 32


def prefill_tiles(prefix_lens, new_lens, first, rows, device):
    pairs = [(r, s) for r in range(first, len(new_lens)) for s in range(0, new_lens[r], rows)]
    both = torch.tensor([[r for r, _ in pairs], [s for _, s in pairs]], dtype=torch.int32).reshape(2, -1).to(device)
    return both[0].contiguous(), both[1].contiguous()


def decode_clusters(d, splits, group):
    return 0


@dataclass(frozen=True)
class DecodePlan:
    splits: int
    fused: bool
    scratch_floats: int
    arm: str
    stages: int = 0


def plan_decode_attention(dtype, requests, nq, nkv, d, max_seq_len, even=False, dv=None, values_in_keys=False,
                          keep_first=0, fusable=True, cuda_cores=False):
    if requests == 0:
        return DecodePlan(1, False, 0, "single")
    splits = 2 if max_seq_len >= 32 else 1
    fused = FUSE_DECODE and (dv or d) == d and fusable and not keep_first and not cuda_cores
    return DecodePlan(splits, fused, decode_scratch_floats(requests, nq, dv or d, splits), "wave" if splits > 1 else "single")


def decode_scratch_floats(requests, nq, d, splits):
    return requests * nq * splits * (d + 2) if splits > 1 else 0


def _gather_kv(kv_layer, table_row, length, page_size, nkv=None, d=None, dv=None, values_in_keys=False):
    pos = torch.arange(length, device=kv_layer.device)
    page = table_row[(pos // page_size)].long()
    keys, values = _pages(kv_layer, nkv, page_size, d, dv, values_in_keys)
    k = keys[page, :, pos % page_size]                 # [length, nkv, d]
    v = values[page, :, pos % page_size]
    return k.float(), v.float()


def _attend(q, k, v, q_pos, scale, window, softcap=None, keep_first=0, sink=False, all_values=False):
    """q [rows, nq, d] at positions q_pos [rows]; k [keys, nkv, d], v [keys, nkv, dv] at positions 0..keys-1.
    ``sink``: a key of score 0 without a value joins the softmax; ``all_values``: every query head's weights over the
    values of every kv head, [rows, nq, nkv * dv]."""
    rep = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    kpos = torch.arange(k.shape[0], device=q.device)
    seen = kpos[None, :] <= q_pos[:, None]
    if window:
        seen &= (kpos[None, :] > q_pos[:, None] - window) | (kpos[None, :] < keep_first)
    s = s.masked_fill(~seen[None], float("-inf"))
    if sink:
        p = torch.softmax(torch.cat([s, torch.zeros_like(s[..., :1])], -1), -1)[..., :-1]
    else:
        p = torch.softmax(s, -1)
    if all_values:
        return torch.einsum("hqk,kgd->qhgd", p, v).reshape(q.shape[0], q.shape[1], -1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def attention_prefill(q, kv_layer, block_table, cu_seqlens, prefix_lens, tile_req, tile_start, out, nq, nkv, d,
                      page_size, scale, window=None, tile_rows=None, heads_per_block=0, softcap=None, dv=None,
                      values_in_keys=False, keep_first=0, sink=False, all_values=False):
    dv = dv or d
    for r in sorted(set(tile_req.tolist())):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        prefix = int(prefix_lens[r])
        k, v = _gather_kv(kv_layer, block_table[r], prefix + t1 - t0, page_size, nkv, d, dv, values_in_keys)
        qpos = torch.arange(prefix, prefix + t1 - t0, device=q.device)
        o = _attend(q[t0:t1].float().view(-1, nq, d), k, v, qpos, scale, window, softcap, keep_first, sink, all_values)
        out[t0:t1] = o.reshape(t1 - t0, -1).to(out.dtype)


def attention_decode(q, kv_layer, block_table, seq_lens, out, scratch, splits, nq, nkv, d, page_size, scale,
                     window=None, stages=0, softcap=None, dv=None, values_in_keys=False, keep_first=0, sink=False,
                     all_values=False):
    dv = dv or d
    for r in range(q.shape[0]):
        n = int(seq_lens[r])
        k, v = _gather_kv(kv_layer, block_table[r], n, page_size, nkv, d, dv, values_in_keys)
        o = _attend(q[r:r + 1].float().view(1, nq, d), k, v, torch.tensor([n - 1], device=q.device), scale, window, softcap,
                    keep_first, sink, all_values)
        out[r] = o.reshape(-1).to(out.dtype)


def attention_decode_fused(qkv, q_gain, k_gain, eps, cos, sin, kv_layer, block_table, seq_lens, out, scratch, splits, nq, nkv,
                           d, rotary_dim, page_size, scale, window=None, write_kv=True, stages=0, softcap=None):
    """What the one kernel does, as the two statements it replaces: every request brings one token, at position
    seq_len - 1."""
    qkv = _sum(qkv)
    n = qkv.shape[0]
    q = qk_norm_rope_write(qkv, q_gain, k_gain, eps, cos, sin, (seq_lens - 1).to(torch.int32),
                           torch.arange(n, dtype=torch.int32, device=qkv.device), block_table, kv_layer, nq, nkv, d, rotary_dim,
                           page_size, write_kv=write_kv)
    attention_decode(q.to(out.dtype), kv_layer, block_table, seq_lens, out, scratch, splits, nq, nkv, d, page_size, scale, window,
                     softcap=softcap)


def sigmoid_gate(out, gate):
    out.copy_((out.float() * torch.sigmoid(_sum(gate).float())).to(out.dtype))
    return out


def normed_mean(inputs, gains, eps, add=None):
    total = 0
    for t, g in zip(inputs, gains):
        v = _sum(t).float()
        total = total + (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)) * g.float()
    total = total / len(inputs)
    if add is not None:
        total = total + _sum(add).float()
    return total.unsqueeze(0)


SSM_CHUNK = 64


def token_chunks(new_lens, chunk, device):
    pairs = [(r, s) for r, n in enumerate(new_lens) for s in range(0, n, chunk)]
    both = torch.tensor([[r for r, _ in pairs], [s for _, s in pairs]], dtype=torch.int32).reshape(2, -1).to(device)
    return both[0].contiguous(), both[1].contiguous()


def causal_conv_silu(proj, col0, channels, weight, bias, state, state_off, chunk_req, chunk_start, cu_seqlens, slots,
                     chunk=SSM_CHUNK):
    return causal_conv(proj, col0, channels, weight, bias, state, state_off, chunk_req, chunk_start, cu_seqlens, slots, chunk)


def causal_conv(proj, col0, channels, weight, bias, state, state_off, chunk_req, chunk_start, cu_seqlens, slots,
                chunk=SSM_CHUNK, activation="silu"):
    taps = weight.shape[1]
    out = torch.empty((proj.shape[0], channels), dtype=proj.dtype, device=proj.device)
    for r in range(cu_seqlens.numel() - 1):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        if t1 == t0:
            continue
        if taps > 1:
            held = state[int(slots[r]), state_off:state_off + (taps - 1) * channels].view(taps - 1, channels)
        else:
            held = torch.zeros((0, channels))                   # a single tap carries nothing from step to step
        seq = torch.cat([held, proj[t0:t1, col0:col0 + channels].float()])
        acc = (bias.float() if bias is not None else torch.zeros(channels))[None, :].expand(t1 - t0, channels).clone()
        for j in range(taps):
            acc = acc + seq[j:j + t1 - t0] * weight[:, j][None, :]
        out[t0:t1] = (acc * torch.sigmoid(acc) if activation == "silu" else acc).to(proj.dtype)
        if taps > 1:
            held.copy_(seq[-(taps - 1):])
    return out


def scan_plan(new_lens, device, state_floats=0):
    return None


def scan_workspace_floats(plan, heads, head_dim, n_state):
    return 0


def ssd_scan(xbc, proj, dt_col, dt_bias, a_log, d_skip, state, cu_seqlens, slots, requests, heads, head_dim, n_state, groups,
             plan=None, workspace=None):
    inner = heads * head_dim
    y = torch.empty((xbc.shape[0], inner), dtype=torch.float32, device=xbc.device)
    per = heads // groups
    a = -torch.exp(a_log.float())
    for r in range(requests):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        s = state[int(slots[r]), :inner * n_state].view(heads, head_dim, n_state)
        for t in range(t0, t1):
            x = xbc[t, :inner].float().view(heads, head_dim)
            b = xbc[t, inner:inner + groups * n_state].float().view(groups, n_state).repeat_interleave(per, 0)
            c = xbc[t, inner + groups * n_state:].float().view(groups, n_state).repeat_interleave(per, 0)
            dt = torch.nn.functional.softplus(proj[t, dt_col:dt_col + heads].float() + dt_bias.float())
            s.copy_(torch.exp(a * dt)[:, None, None] * s + (dt[:, None] * x)[:, :, None] * b[:, None, :])
            y[t] = (torch.einsum("hpn,hn->hp", s, c) + d_skip.float()[:, None] * x).reshape(inner)
    return y


def gated_group_rmsnorm(y, proj, gain, groups, eps):
    n, inner = y.shape
    z = proj[:, :inner].float()
    v = (y * (z * torch.sigmoid(z))).view(n, groups, inner // groups)
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return (v.view(n, inner) * gain.float()).to(proj.dtype)


def argmax(logits, out=None):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def apply_penalties(logits, entry_row, entry_token, entry_count, entry_bias, repetition, frequency, presence):
    for e in range(entry_row.numel()):
        r, t, c = int(entry_row[e]), int(entry_token[e]), int(entry_count[e])
        v = logits[r, t]
        if c > 0:
            rep = repetition[r]
            if rep != 1.0:
                v = v / rep if v > 0 else v * rep
            v = v - c * frequency[r] - presence[r]
        logits[r, t] = v + entry_bias[e]


def sample(logits, temperature, top_k, top_p, min_p, uniform, want_logprob=False):
    import plain_impl

    toks, lps = [], []
    for r in range(logits.shape[0]):
        t, k = float(temperature[r]), int(top_k[r])
        if t == 0 or k == 1:
            tok = int(torch.argmax(logits[r]))
            lp = float(torch.log_softmax(logits[r].float(), -1)[tok])
        else:
            probs = plain_impl.filtered_probs(logits[r].cpu(), t, k, float(top_p[r]), float(min_p[r]))
            tok = plain_impl.inverse_cdf_pick(probs, float(uniform[r]))
            lp = float(torch.log(probs[tok]))
        toks.append(tok)
        lps.append(lp)
    dev = logits.device
    return (torch.tensor(toks, dtype=torch.int32, device=dev),
            torch.tensor(lps, dtype=torch.float32, device=dev) if want_logprob else None)


def top_logprobs_cap():
    return 128


def top_logprobs(logits, k):
    rows, vocab = logits.shape
    cap = top_logprobs_cap()
    tokens = torch.zeros((rows, cap), dtype=torch.int32, device=logits.device)
    logprobs = torch.zeros((rows, cap), dtype=torch.float32, device=logits.device)
    counts = torch.zeros((rows,), dtype=torch.int32, device=logits.device)
    lp = torch.log_softmax(logits.float(), -1)
    for r in range(rows):
        kk = min(int(k[r]), cap, vocab)
        if kk <= 0:
            continue
        kth = torch.topk(lp[r], kk).values[-1]
        idx = torch.nonzero(lp[r] >= kth).flatten()[:cap]
        counts[r] = idx.numel()
        tokens[r, :idx.numel()] = idx.to(torch.int32)
        logprobs[r, :idx.numel()] = lp[r, idx]
    return tokens, logprobs, counts


# ---- per-head products, linear attention with a data-dependent decay, attention over a latent, routed experts

def head_linear(x, weight, out_dtype=None):
    """x [tokens, heads, k], weight [heads, n, k] -> [heads, tokens, n]."""
    out = torch.einsum("thk,hnk->htn", x.float(), weight.float())
    return out if (out_dtype == torch.float32 or x.dtype == torch.float32) else out.to(x.dtype)


def token_shift_mix(h, mu, state, state_off, cu_seqlens, token_req, slots):
    tokens, width = h.shape
    prev = torch.empty((tokens, width), dtype=torch.float32, device=h.device)
    for r in range(cu_seqlens.numel() - 1):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        if t1 == t0:
            continue
        held = state[int(slots[r]), state_off:state_off + width]
        prev[t0] = held
        prev[t0 + 1:t1] = h[t0:t1 - 1].float()
        held.copy_(h[t1 - 1].float())
    cur = h.float()
    return (cur[None] + (prev - cur)[None] * mu.float()[:, None, :]).to(h.dtype)


def wkv_decay(a, w2t, w0):
    return -torch.exp(torch.tanh(a.float()) @ w2t.float() + w0.float())


def wkv_max_head_dim():
    return 256


def wkv_plan(new_lens, device):
    return None


def wkv_workspace_floats(plan, heads, d):
    return 0


def wkv_scan(r, k, v, log_decay, u, state, cu_seqlens, slots, requests, heads, d, plan=None, workspace=None):
    y = torch.empty((r.shape[0], heads * d), dtype=torch.float32, device=r.device)
    for q in range(requests):
        t0, t1 = int(cu_seqlens[q]), int(cu_seqlens[q + 1])
        S = state[int(slots[q]), :heads * d * d].view(heads, d, d)
        for t in range(t0, t1):
            rt, kt, vt = (x[t].float().view(heads, d) for x in (r, k, v))
            kv = kt[:, :, None] * vt[:, None, :]
            y[t] = torch.einsum("hi,hij->hj", rt, S + u.float()[:, :, None] * kv).reshape(heads * d)
            S.copy_(torch.exp(log_decay[t].float().view(heads, d))[:, :, None] * S + kv)
    return y


def group_rmsnorm_gate(y, gate, gain, groups, eps):
    n, inner = y.shape
    v = y.float().view(n, groups, inner // groups)
    v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, inner)
    z = gate.float()
    return (v * gain.float() * (z * torch.sigmoid(z))).to(gate.dtype)


def _rotate_halves(t, cos, sin, positions, rotary_dim):
    if cos is None or not rotary_dim:
        return t
    half = rotary_dim // 2
    shape = [t.shape[0]] + [1] * (t.dim() - 2) + [half]
    c, s = cos[positions.long()].view(shape), sin[positions.long()].view(shape)
    x1, x2, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)


def latent_prepare(down, q0, q_rank, kv0, rank, rot, rotary_dim, q_gain, kv_gain, eps, cos, sin, positions, token_req,
                   block_table, layer, page_size, write_kv=True):
    x = down.float()
    unit = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)
    cq = (unit(x[:, q0:q0 + q_rank]) * q_gain.float()).to(layer.dtype)
    if write_kv:
        latent = unit(x[:, kv0:kv0 + rank]) * kv_gain.float()
        turned = _rotate_halves(x[:, kv0 + rank:kv0 + rank + rot], cos, sin, positions, rotary_dim)
        pos = positions.long()
        page = block_table[token_req.long(), pos // page_size].long()
        rows = layer.view(-1, page_size, rank + rot)
        rows[page, pos % page_size] = torch.cat([latent, turned], -1).to(layer.dtype)
    return cq


def latent_query(qa, q, heads, d, rank, rot, rotary_dim, cos, sin, positions):
    tokens = q.shape[0]
    turned = _rotate_halves(q.float().view(tokens, heads, d + rot)[..., d:], cos, sin, positions, rotary_dim)
    return torch.cat([qa.float().transpose(0, 1), turned], -1).reshape(tokens, heads * (rank + rot)).to(q.dtype)


def head_gate(ov, gate_rows, g0, out_dtype):
    heads, tokens, dv = ov.shape
    g = torch.sigmoid(gate_rows[:, g0:g0 + heads].float())                      # [tokens, heads]
    return (ov.float().transpose(0, 1) * g[:, :, None]).reshape(tokens, heads * dv).to(out_dtype)


@dataclass
class ExpertRouting:
    chosen: torch.Tensor
    weights: torch.Tensor
    top: int


def moe_route(h, router, correction, top, experts):
    s = torch.softmax(h.float() @ router.float().t(), -1)
    chosen = torch.topk(s + correction.float(), top, dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return ExpertRouting(chosen.to(torch.int32), picked / (picked.sum(-1, keepdim=True) + 1e-20), top)


def moe_experts(h, routing, w_gate_up, w_down, limit, alpha):
    tokens, width = h.shape
    experts = w_down.shape[0] if w_down.dim() == 3 else 0
    ff = w_down.shape[2] if experts else 0
    out = torch.zeros((tokens, width), dtype=torch.float32, device=h.device)
    x = h.float()
    for t in range(tokens):
        for e, a in zip(routing.chosen[t].tolist(), routing.weights[t].tolist()):
            if e < experts:
                gu = w_gate_up[e].float() @ x[t]
                g, u = gu[:ff].clamp(max=limit), gu[ff:].clamp(min=-limit, max=limit)
                act = (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(h.dtype).float()
                out[t] += a * (w_down[e].float() @ act)
            else:
                out[t] += a * x[t]
    return out


# ---------------------------------------------------------------------------- sandwich norms, plain feed-forward

def add_normed_rmsnorm(resid, delta, post_gain, post_eps, mult, weight, eps, out_dtype, rows=None, write_residual=True,
                       normalise=True):
    """resid += mult * (delta / rms(delta) * post_gain), or mult * (delta * post_gain) without ``normalise``; returns
    (the new rows) / rms * weight (None without ``weight``)."""
    d = _sum(delta).float()
    if normalise:
        d = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + post_eps)
    add = mult * (d * post_gain.float())
    if rows is not None:
        v = resid[rows.long()] + add[rows.long()]
    else:
        v = resid + add
        if write_residual:
            resid.copy_(v)
    if weight is None:
        return None
    return ((v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)) * weight.float()).to(out_dtype)


def _activate(z, activation):
    if activation == "relu2":
        return torch.clamp(z, min=0) ** 2
    if activation == "silu":
        return z * torch.sigmoid(z)
    assert activation == "gelu_tanh"
    return 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))


def activation(x, out_dtype, activation="relu2"):
    return _activate(_sum(x).float(), activation).to(out_dtype)


def linear_activation(x, weight, activation="relu2"):
    return _activate(_sum(linear_auto(x, weight)).float(), activation).to(x.dtype)


# ---------------------------------------------------------------------------- differential attention

def diff_prepare(proj, positions, token_req, block_table, kv_layer, heads, nkv, d, dv, maps, page_size, temp_coef, temp_every,
                 write_kv=True):
    """proj [tokens, heads*maps*d | nkv*maps*d | nkv*dv | ...]: queries times 1 + coef ln(floor((p + 1) / every) + 1), map m of
    head h laid out as query head h*maps + m of maps*d columns, zero outside columns [m*d, (m+1)*d); keys and values to the page."""
    n = proj.shape[0]
    x = proj.float()
    kd = maps * d
    q = x[:, :heads * kd].view(n, heads, maps, d)
    if temp_coef:
        p = positions.float()
        q = q * (1.0 + temp_coef * torch.log(torch.floor((p + 1.0) / float(temp_every)) + 1.0))[:, None, None, None]
    wide = torch.zeros((n, heads, maps, maps, d), dtype=torch.float32, device=proj.device)
    for m in range(maps):
        wide[:, :, m, m] = q[:, :, m]
    if write_kv:
        k = x[:, heads * kd:(heads + nkv) * kd].view(n, nkv, kd)
        v = x[:, (heads + nkv) * kd:(heads + nkv) * kd + nkv * dv].view(n, nkv, dv)
        pos = positions.long()
        page = block_table[token_req.long(), pos // page_size].long()
        keys, values = _pages(kv_layer, nkv, page_size, kd, dv)
        keys[page, :, pos % page_size] = k.to(kv_layer.dtype)
        values[page, :, pos % page_size] = v.to(kv_layer.dtype)
    return wide.reshape(n, heads * maps * kd).to(kv_layer.dtype)


def diff_combine(maps_out, proj, gate_col, heads, dv, maps, lam, out_scale, eps):
    """maps_out [tokens, heads*maps*dv]; o = a_0 - lam * a_1, divided by its root mean square over dv, times out_scale,
    times sigmoid(proj[:, gate_col + head])."""
    assert maps == 2
    n = maps_out.shape[0]
    a = maps_out.float().view(n, heads, maps, dv)
    o = a[:, :, 0] - lam * a[:, :, 1]
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_scale
    gate = torch.sigmoid(proj[:, gate_col:gate_col + heads].float())
    return (o * gate[:, :, None]).reshape(n, heads * dv).to(maps_out.dtype)


# ---------------------------------------------------------------------------- mixed heads, delta rule, selective scan

def sink_on_tensor_cores(dtype, d, dv=None, values_in_keys=False, softcap=None):
    return False


def all_values_decode_rows(dtype, requests, nkv, d, dv=None):
    return requests


def all_values_in_planes(dtype, nkv, d, dv=None):
    return False


def all_values_sums(dtype, tokens, nq, nkv, d, dv, device):
    return torch.empty((tokens, nq * nkv * (dv or d)), dtype=torch.float32, device=device)


def head_mix(sums, mix, nq, nkv, dv, out_dtype):
    """out[t, h] = sum_g mix[h, g] sums[t, g, kv(h)]; sums float32 [tokens, nq * nkv * dv]."""
    n = sums.shape[0]
    own = sums.view(n, nq, nkv, dv)[:, :, torch.arange(nq, device=sums.device) // (nq // nkv)]       # [n, g, h, dv]
    return torch.einsum("hg,nghd->nhd", mix.float(), own).reshape(n, nq * dv).to(out_dtype)


def delta_rule_max_head_dim():
    return 256


def delta_rule(qkv, proj, b_col, a_col, a_log, dt_bias, state, cu_seqlens, slots, requests, heads, kv_heads, d, dv, unit_eps,
               q_scale):
    n = qkv.shape[0]
    x = qkv.float()
    q = x[:, :kv_heads * d].view(n, kv_heads, d)
    k = x[:, kv_heads * d:2 * kv_heads * d].view(n, kv_heads, d)
    v = x[:, 2 * kv_heads * d:].view(n, heads, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * q_scale
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(proj[:, b_col:b_col + heads].float())
    decay = torch.exp(-torch.exp(a_log.float()) * torch.nn.functional.softplus(proj[:, a_col:a_col + heads].float() + dt_bias.float()))
    y = torch.zeros((n, heads * dv), dtype=torch.float32, device=qkv.device)
    for r in range(requests):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        row = state[int(slots[r])]
        S = row[:heads * dv * d].view(heads, dv, d).clone()                       # a head's matrix as [dv, d]
        for t in range(t0, t1):
            for h in range(heads):
                g = h // (heads // kv_heads)
                Sh = decay[t, h] * S[h]
                u = beta[t, h] * (v[t, h] - Sh @ k[t, g])
                S[h] = Sh + torch.outer(u, k[t, g])
                y[t, h * dv:(h + 1) * dv] = S[h] @ q[t, g]
        if t1 > t0:
            row[:heads * dv * d] = S.reshape(-1)
    return y


def selective_scan_max_state():
    return 256


def selective_workspace_floats(plan, inner, n_state):
    return 0


def selective_scan(x, low, b_col, step, proj, z_col, a, d_skip, state, cu_seqlens, slots, requests, plan=None, workspace=None):
    tokens, inner = x.shape
    n = a.shape[1]
    xf, dt = x.float(), torch.nn.functional.softplus(step.float())
    B, C = low[:, b_col:b_col + n].float(), low[:, b_col + n:b_col + 2 * n].float()
    z = proj[:, z_col:z_col + inner].float()
    out = torch.zeros((tokens, inner), dtype=torch.float32, device=x.device)
    for r in range(requests):
        t0, t1 = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        row = state[int(slots[r])]
        S = row[:inner * n].view(inner, n).clone()
        for t in range(t0, t1):
            S = torch.exp(dt[t][:, None] * a.float()) * S + (dt[t] * xf[t])[:, None] * B[t][None, :]
            out[t] = (S @ C[t] + d_skip.float() * xf[t]) * (z[t] / (1 + torch.exp(-z[t])))
        if t1 > t0:
            row[:inner * n] = S.reshape(-1)
    return out.to(x.dtype)
