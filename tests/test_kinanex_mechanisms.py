"""Each mechanism of the Kinanex decoder alone: the kernels' faces (CUDA on the GPU, their plain statements on the
CPU) against the functions of ``plain_kinanex``, with inputs made so that a fault shows: one key scaled to stand out
far back, at a page border and as the newest; queries that no key answers, so that the sink takes the weight; a
head-mixing matrix that swaps heads; states carried over portions of every length down to two tokens and over slots
that change hands; a value written by the first token and read hundreds of steps later; sizes that are no powers of two."""

import math

import pytest
import torch
import torch.nn.functional as F

import kernel_refs
import plain_kinanex as pk

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def ops_for(device):
    if device == "cpu":
        return kernel_refs
    from lily_b200.csrc import ops
    return ops


def i32(values, device):
    return torch.tensor(values, dtype=torch.int32, device=device)


def close(got, want, dtype, scale=1.0):
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-4
    torch.testing.assert_close(got.float().cpu(), want.float(), atol=tol * scale, rtol=tol)


def portions(total, sizes):
    """``total`` tokens cut into portions that cycle through ``sizes``."""
    out, k = [], 0
    while sum(out) < total:
        out.append(min(sizes[k % len(sizes)], total - sum(out)))
        k += 1
    return out


CUTS = {"whole": lambda t: [t], "mixed": lambda t: portions(t, [37, 1, 2, 64, 1, 1, 5, 130]), "decoded": lambda t: [t - 40] + [1] * 40}


# ------------------------------------------------------------------ attention: sink, mixed heads, values of their own size

def run_attention(ops, device, dtype, q, k, v, talk, scale, page, cuts, sink=True):
    """q [t, H, d], k [t, G, d], v [t, G, dv] through the cache write, the attention kernels (a portion of one token
    takes the decode kernel) and the head mix; pages come in a scrambled order."""
    t, heads, d = q.shape
    kvh, dv = k.shape[1], v.shape[2]
    pages = -(-t // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(1)) + 1
    table = i32(order.tolist(), device).view(1, pages)
    shape = (pages + 1, 2, kvh, page, d) if dv == d else (pages + 1, kvh * page * (d + dv))
    cache = torch.zeros(shape, dtype=dtype, device=device)
    out = torch.empty((t, heads * dv), dtype=dtype, device=device)
    qkv = torch.cat([q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)], 1).to(device=device, dtype=dtype)
    sized = {} if dv == d else {"dv": dv}
    how = {"sink": sink, "all_values": talk is not None}
    wide = kvh * dv if talk is not None else dv
    mix = None if talk is None else talk.to(device=device, dtype=torch.float32).contiguous()
    done = 0
    for n in cuts:
        rows = qkv[done:done + n].contiguous()
        pos = i32(list(range(done, done + n)), device)
        qq = ops.qk_norm_rope_write(rows, None, None, 1e-6, None, None, pos, i32([0] * n, device), table, cache, heads, kvh,
                                    d, 0, page, **sized)
        if talk is not None:
            o = ops.all_values_sums(dtype, n, heads, kvh, d, dv, device)     # wide float32 rows, or a plane a kv head
        else:
            o = torch.empty((n, heads * dv), dtype=dtype, device=device)
        if n == 1:
            if ops.sink_on_tensor_cores(dtype, d, dv):
                rows = ops.all_values_decode_rows(dtype, 1, kvh, d, dv) if talk is not None else 1
                plan = ops.plan_decode_attention(dtype, rows, heads, kvh, d, done + 1, fusable=False)
            else:
                plan = ops.plan_decode_attention(dtype, 1, heads, kvh, d, done + 1, dv=dv if o.dim() == 3 else wide, cuda_cores=True)
            scratch = torch.empty(max(1, plan.scratch_floats), dtype=torch.float32, device=device)
            ops.attention_decode(qq, cache, table, i32([done + 1], device), o, scratch, plan.splits, heads, kvh, d, page, scale,
                                 None, **sized, **how)
        else:
            tile = ops.prefill_tile_rows(dtype, d, page, n, **sized, **how)
            tr, ts = ops.prefill_tiles([done], [n], 0, tile, device)
            ops.attention_prefill(qq, cache, table, i32([0, n], device), i32([done], device), tr, ts, o, heads, kvh, d, page,
                                  scale, None, tile_rows=tile, **sized, **how)
        out[done:done + n] = o if talk is None else ops.head_mix(o, mix, heads, kvh, dv, dtype)
        done += n
    assert done == t
    return out.float().cpu().view(t, heads, dv)


def plain_attention(q, k, v, talk, scale, sink=True):
    t, heads, _ = q.shape
    kv_of = torch.arange(heads) // (heads // k.shape[1])
    pos = torch.arange(t)
    scores = torch.einsum("ihd,jhd->hij", q.double(), k.double()[:, kv_of]) * scale
    mask = (pos[None, :] <= pos[:, None])[None]
    w = pk.sink_softmax(scores, mask) if sink else torch.softmax(scores.masked_fill(~mask, float("-inf")), -1)
    if talk is not None:
        w = torch.einsum("hg,gij->hij", talk.double(), w)
    return torch.einsum("hij,jhe->ihe", w, v.double()[:, kv_of]).float()


ATTENTION_CASES = [  # heads, kv heads, d, dv, page, tokens
    (4, 2, 16, 24, 16, 230),
    (6, 3, 40, 10, 8, 150),
    (2, 1, 64, 64, 64, 300),            # head sizes the mma.sync kernels take in bfloat16: a launch a kv head
    (4, 2, 64, 64, 16, 330),
    (6, 3, 128, 128, 64, 280),
    (12, 4, 64, 40, 64, 700),
    (3, 3, 24, 20, 16, 120),            # every head its own kv head
    (4, 1, 128, 128, 32, 420),
    (8, 8, 16, 72, 16, 130),            # more value columns over all kv heads than a row of the CUDA-core kernel gathers
]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d,dv,page,t", ATTENTION_CASES)
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_sink_and_mixed_heads_with_keys_that_stand_out(device, dtype, heads, kvh, d, dv, page, t, cut):
    """Keys many times larger than the rest draw nearly all weight of every later query: the first position, one far
    back in the middle of a page, the last and the first of two neighbouring pages.  The queries of one stretch point
    away from every key: their scores are far below zero and the sink takes the weight, so their outputs are nearly
    zero (a softmax without the sink would give an average of values).  The mixing matrix is far from the identity."""
    if device == "cpu" and (dtype == torch.bfloat16 or t > 300):
        pytest.skip("the plain statements are checked in float32 on the short cases")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(d + dv + heads)
    q = torch.randn(t, heads, d, generator=g)
    k = torch.randn(t, kvh, d, generator=g) * 0.3
    k[:, :, 0] = k[:, :, 0].abs() + 1.0
    v = torch.randn(t, kvh, dv, generator=g)
    for m in sorted({0, page + page // 2, 2 * page - 1, 2 * page, t // 2}):
        k[m] = 0.0
        k[m, :, 0] = 4.0 * math.sqrt(d)
    q[:, :, 0] = q[:, :, 0].abs() + 0.5
    quiet = slice(t // 2 + 5, t // 2 + 12)
    q[quiet] = 0.0
    q[quiet, :, 0] = -12.0 * math.sqrt(d)                        # every key's first column is above one: scores below -12
    talk = 0.3 * torch.eye(heads) + 0.7 * torch.eye(heads).roll(1, 0) + 0.2 * torch.randn(heads, heads, generator=g)
    if dtype == torch.bfloat16:
        q, k, v = (x.bfloat16().float() for x in (q, k, v))
    scale = 1.0 / math.sqrt(d)
    want = plain_attention(q, k, v, talk, scale)
    assert float(want[quiet].abs().max()) < 0.05 * float(want.abs().max())                   # the sink took the weight there
    got = run_attention(ops, device, dtype, q, k, v, talk, scale, page, CUTS[cut](t))
    close(got, want, dtype, scale=float(want.abs().max()))
    # the sink alone (heads not mixed), on the same kernels
    got = run_attention(ops, device, dtype, q, k, v, None, scale, page, CUTS[cut](t))
    close(got, plain_attention(q, k, v, None, scale), dtype, scale=float(want.abs().max()))


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("dtype,d,dv", [(torch.float32, 32, 16), (torch.bfloat16, 64, 64), (torch.bfloat16, 64, 40)])
def test_the_sink_counts_once_however_the_keys_are_cut(device, splits, dtype, d, dv):
    """Decode over 1 to 5 key ranges (CUDA-core kernel, and the mma.sync kernel with its four warps a range, merged
    in a cluster or by the combine kernel): the extra unit of the denominator enters once."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    heads, kvh, page, t = 4, 2, 16, 200
    g = torch.Generator().manual_seed(splits)
    q, k, v = (torch.randn(t, n, w, generator=g).to(dtype).float() for n, w in ((heads, d), (kvh, d), (kvh, dv)))
    talk = torch.randn(heads, heads, generator=g)
    want = plain_attention(q, k, v, talk, 0.2)[-1]
    table = i32(list(range(1, t // page + 2)), device).view(1, -1)
    shape = (t // page + 2, 2, kvh, page, d) if dv == d else (t // page + 2, kvh * page * (d + dv))
    cache = torch.zeros(shape, dtype=dtype, device=device)
    qkv = torch.cat([q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)], 1).to(device=device, dtype=dtype)
    sized = {} if dv == d else {"dv": dv}
    qq = ops.qk_norm_rope_write(qkv, None, None, 1e-6, None, None, i32(list(range(t)), device), i32([0] * t, device), table, cache,
                                heads, kvh, d, 0, page, **sized)
    o = ops.all_values_sums(dtype, 1, heads, kvh, d, dv, device)
    scratch = torch.empty(heads * splits * kvh * (dv + 2), dtype=torch.float32, device=device)
    ops.attention_decode(qq[-1:].contiguous(), cache, table, i32([t], device), o, scratch, splits, heads, kvh, d, page, 0.2, None,
                         sink=True, all_values=True, **sized)
    got = ops.head_mix(o, talk.to(device), heads, kvh, dv, torch.float32)
    close(got.view(heads, dv), want, dtype, scale=float(want.abs().max()))


# ------------------------------------------------------------------ values: unit root mean square, kept and blended

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d,dv,rot", [(4, 2, 16, 12, 8), (2, 1, 64, 64, 64), (6, 3, 24, 7, 0), (12, 4, 64, 40, 32)])
def test_values_are_normed_kept_and_blended_on_their_way_to_the_cache(device, dtype, heads, kvh, d, dv, rot):
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    t, page, eps, lam = 37, 16, 1e-5, 0.3
    g = torch.Generator().manual_seed(dv)
    rows = lambda: (torch.randn(t, (heads + kvh) * d + kvh * dv, generator=g) * 3.0).to(dtype)
    first, second = rows(), rows()
    pos, req = i32(list(range(t)), device), i32([0] * t, device)
    table = i32([3, 1, 2], device).view(1, 3)
    gains = [(1.0 + 0.2 * torch.randn(d, generator=g)).to(device) for _ in range(2)]
    angle = torch.arange(t)[:, None] * (100.0 ** (-torch.arange(0, rot, 2) / max(rot, 1)))[None, :]
    cos, sin = (angle.cos().float().to(device), angle.sin().float().to(device)) if rot else (None, None)
    sized = {} if dv == d else {"dv": dv}

    def cached_values(cache):
        flat = cache.float().cpu()
        vals = flat[:, 1] if flat.dim() == 5 else flat[:, kvh * page * d:].view(-1, kvh, page, dv)
        return torch.stack([vals[[3, 1, 2][p // page], :, p % page] for p in range(t)])          # [t, kvh, dv]

    shape = (4, 2, kvh, page, d) if dv == d else (4, kvh * page * (d + dv))
    kept = torch.zeros((t, kvh * dv), dtype=torch.float32, device=device)
    cache1 = torch.zeros(shape, dtype=dtype, device=device)
    ops.qk_norm_rope_write(first.to(device), gains[0], gains[1], eps, cos, sin, pos, req, table, cache1, heads, kvh, d, rot, page,
                           v_norm=True, v_keep=kept, **sized)
    v1 = pk.rms(first.float()[:, (heads + kvh) * d:].view(t, kvh, dv), eps)
    close(kept.view(t, kvh, dv), v1, torch.float32)                       # kept in float32, before the cache's rounding
    close(cached_values(cache1), v1, dtype)
    cache2 = torch.zeros(shape, dtype=dtype, device=device)
    q2 = ops.qk_norm_rope_write(second.to(device), gains[0], gains[1], eps, cos, sin, pos, req, table, cache2, heads, kvh, d, rot,
                                page, v_norm=True, v_keep=kept, v_blend=lam, **sized)
    v2 = (1.0 - lam) * pk.rms(second.float()[:, (heads + kvh) * d:].view(t, kvh, dv), eps) + lam * v1
    close(cached_values(cache2), v2, dtype)
    # q and k go their usual way beside it
    rotd = {"dims": rot, "base": 100.0} if rot else None
    want_q = pk.rotate(pk.rms(second.float()[:, :heads * d].view(t, heads, d), eps) * gains[0].cpu(), rotd, torch.arange(t))
    close(q2.view(t, heads, d), want_q, dtype, scale=3.0)


# ------------------------------------------------------------------ the delta rule

def delta_inputs(t, heads, kvh, d, dv, seed, dtype, slow=False):
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn(t, 2 * kvh * d + heads * dv, generator=g)
    proj = torch.randn(t, 3 + 2 * heads, generator=g)
    a_log = torch.linspace(-2.0, 1.0, heads)
    if slow:
        a_log = torch.full((heads,), -9.0)
    dt_bias = 0.3 * torch.randn(heads, generator=g)
    return qkv.to(dtype), proj.to(dtype), a_log, dt_bias


def plain_delta(qkv, proj, a_log, dt_bias, heads, kvh, d, dv, eps=1e-6):
    t = qkv.shape[0]
    x, p = qkv.double(), proj.double()
    q = pk.unit(x[:, :kvh * d].view(t, kvh, d), eps) * d ** -0.5
    k = pk.unit(x[:, kvh * d:2 * kvh * d].view(t, kvh, d), eps)
    v = x[:, 2 * kvh * d:].view(t, heads, dv)
    beta = torch.sigmoid(p[:, 3:3 + heads])
    decay = torch.exp(-torch.exp(a_log.double()) * F.softplus(p[:, 3 + heads:] + dt_bias.double()))
    return torch.stack([pk.delta_rule(q[:, h // (heads // kvh)], k[:, h // (heads // kvh)], v[:, h], decay[:, h], beta[:, h])
                        for h in range(heads)], 1).float()


DELTA_CASES = [(4, 2, 16, 8), (3, 3, 20, 7), (2, 1, 64, 32), (4, 4, 12, 33), (2, 2, 128, 48), (1, 1, 200, 9)]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d,dv", DELTA_CASES)
def test_delta_rule_whole_in_portions_and_in_slots_that_change_hands(device, dtype, heads, kvh, d, dv):
    """Two requests side by side, cut into portions of other sizes each (down to two tokens and single tokens), their
    matrices carried in slots 2 and 1; then a third request takes slot 2 after it was zeroed."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    lens, cuts = [75, 41], [[20, 1, 2, 33, 1, 1, 17], [2, 2, 30, 1, 1, 5]]
    data = [delta_inputs(n, heads, kvh, d, dv, 5 + i, dtype) for i, n in enumerate(lens)]
    a_log, dt_bias = data[0][2], data[0][3]
    want = [plain_delta(x[0], x[1], a_log, dt_bias, heads, kvh, d, dv) for x in data]
    state = torch.zeros((4, heads * d * dv + 5), dtype=torch.float32, device=device)
    state[:, -5:] = 7.0                                            # what lies behind the matrices is not touched
    done, got = [0, 0], [[], []]
    for step in range(max(len(c) for c in cuts)):
        live = [r for r in range(2) if step < len(cuts[r])]
        ns = [cuts[r][step] for r in live]
        qkv = torch.cat([data[r][0][done[r]:done[r] + n] for r, n in zip(live, ns)]).to(device)
        proj = torch.cat([data[r][1][done[r]:done[r] + n] for r, n in zip(live, ns)]).to(device)
        cu = i32([0] + torch.tensor(ns).cumsum(0).tolist(), device)
        y = ops.delta_rule(qkv, proj, 3, 3 + heads, a_log.to(device), dt_bias.to(device), state, cu, i32([2 - r for r in live], device),
                           len(live), heads, kvh, d, dv, 1e-6, d ** -0.5)
        at = 0
        for r, n in zip(live, ns):
            got[r].append(y[at:at + n].float().cpu())
            at += n
            done[r] += n
    for r in range(2):
        close(torch.cat(got[r]).view(lens[r], heads, dv), want[r], dtype)
    assert float((state[:, -5:] - 7.0).abs().max()) == 0.0
    state[2].zero_()
    third = delta_inputs(30, heads, kvh, d, dv, 99, dtype)
    y = ops.delta_rule(third[0].to(device), third[1].to(device), 3, 3 + heads, a_log.to(device), dt_bias.to(device), state,
                       i32([0, 30], device), i32([2], device), 1, heads, kvh, d, dv, 1e-6, d ** -0.5)
    close(y.view(30, heads, dv), plain_delta(third[0], third[1], a_log, dt_bias, heads, kvh, d, dv), dtype)


@pytest.mark.parametrize("device", DEVICES)
def test_delta_rule_reads_after_hundreds_of_steps_what_the_first_token_wrote(device):
    """With nearly no decay, keys orthogonal to the first one and write strength one, the value of the first token
    stays in the matrix: a query along the first key, 400 decoded steps later, reads it back; and a second write
    with the same key replaces it (the delta rule erases what the key held)."""
    ops = ops_for(device)
    heads, d, dv, t = 2, 16, 8, 401
    qkv = torch.zeros(t, 2 * heads * d + heads * dv)
    q, k = qkv[:, :heads * d].view(t, heads, d), qkv[:, heads * d:2 * heads * d].view(t, heads, d)
    v = qkv[:, 2 * heads * d:].view(t, heads, dv)
    k[0, :, 0] = 1.0
    v[0] = torch.arange(1.0, dv + 1.0)
    for s in range(1, t):
        k[s, :, 1 + s % (d - 1)] = 1.0                           # orthogonal to the first key
        v[s] = 0.01 * s
    q[:, :, 0] = 1.0
    k[300, 1] = 0.0
    k[300, 1, 0] = 1.0                                           # head 1 writes again with the first key
    v[300, 1] = -5.0
    proj = torch.zeros(t, 2 * heads)
    proj[:, :heads] = 30.0                                       # sigmoid -> 1
    a_log, dt_bias = torch.full((heads,), -20.0), torch.zeros(heads)
    state = torch.zeros((2, heads * d * dv), dtype=torch.float32, device=device)
    outs = []
    for s in range(t):                                           # token by token, as in decoding
        outs.append(ops.delta_rule(qkv[s:s + 1].to(device), proj[s:s + 1].to(device), 0, heads, a_log.to(device), dt_bias.to(device),
                                   state, i32([0, 1], device), i32([1], device), 1, heads, heads, d, dv, 1e-6, d ** -0.5).cpu())
    last = outs[-1].view(heads, dv) * d ** 0.5
    close(last[0], torch.arange(1.0, dv + 1.0), torch.float32)
    close(last[1], torch.full((dv,), -5.0), torch.float32)
    close(torch.cat(outs).view(t, heads, dv), plain_delta(qkv, torch.cat([torch.zeros(t, 3), proj], 1), a_log, dt_bias, heads, heads, d, dv),
          torch.float32)


# ------------------------------------------------------------------ the selective scan

def plain_scan(x, low, rank, step, z, a_log, d_skip):
    n = a_log.shape[1]
    y = pk.selective_scan(x.double(), F.softplus(step.double()), -torch.exp(a_log.double()), low.double()[:, rank:rank + n],
                          low.double()[:, rank + n:rank + 2 * n], d_skip.double())
    return (y * F.silu(z.double())).float()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,state_n,rank", [(40, 6, 5), (24, 19, 1), (192, 16, 8), (33, 32, 3), (16, 70, 2)])
def test_selective_scan_whole_in_portions_and_in_slots_that_change_hands(device, dtype, inner, state_n, rank):
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(inner + state_n)
    lens, cuts = [90, 37], [[31, 1, 2, 40, 1, 1, 14], [2, 2, 25, 1, 1, 6]]
    a_log = torch.log(torch.linspace(0.2, 4.0, state_n)).expand(inner, state_n) + 0.3 * torch.randn(inner, state_n, generator=g)
    d_skip = 1.0 + 0.2 * torch.randn(inner, generator=g)
    data = []
    for n in lens:
        x, low = torch.randn(n, inner, generator=g).to(dtype), torch.randn(n, rank + 2 * state_n, generator=g).to(dtype)
        step, proj = torch.randn(n, inner, generator=g), torch.randn(n, 2 * inner + 3, generator=g).to(dtype)
        data.append((x, low, step, proj))
    want = [plain_scan(x, low, rank, step, proj[:, 3 + inner:], a_log, d_skip) for x, low, step, proj in data]
    a = (-torch.exp(a_log)).contiguous().to(device)
    state = torch.zeros((4, inner * state_n + 3), dtype=torch.float32, device=device)
    state[:, -3:] = 7.0
    done, got = [0, 0], [[], []]
    for s in range(max(len(c) for c in cuts)):
        live = [r for r in range(2) if s < len(cuts[r])]
        ns = [cuts[r][s] for r in live]
        cat = lambda j: torch.cat([data[r][j][done[r]:done[r] + n] for r, n in zip(live, ns)]).to(device)
        cu = i32([0] + torch.tensor(ns).cumsum(0).tolist(), device)
        y = ops.selective_scan(cat(0), cat(1), rank, cat(2), cat(3), 3 + inner, a, d_skip.to(device), state, cu,
                               i32([3 - 2 * r for r in live], device), len(live))
        at = 0
        for r, n in zip(live, ns):
            got[r].append(y[at:at + n].float().cpu())
            at += n
            done[r] += n
    for r in range(2):
        close(torch.cat(got[r]), want[r], dtype, scale=float(want[r].abs().max()))
    assert float((state[:, -3:] - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,state_n,rank", [(40, 6, 5), (192, 16, 8), (33, 32, 3)])
def test_selective_scan_long_portions_in_chunks_side_by_side(device, dtype, inner, state_n, rank):
    """One step with a portion of 700 tokens and one of 450 (both cut into chunks that run side by side and are joined
    in order), one of 50 and a single token (each in one piece), all continuing from states that an earlier step left."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(inner)
    before, lens = [30, 0, 7, 90], [700, 450, 50, 1]
    a_log = torch.log(torch.linspace(0.05, 2.0, state_n)).expand(inner, state_n) + 0.3 * torch.randn(inner, state_n, generator=g)
    d_skip = 1.0 + 0.2 * torch.randn(inner, generator=g)
    data = []
    for n in [b + m for b, m in zip(before, lens)]:
        x, low = torch.randn(n, inner, generator=g).to(dtype), torch.randn(n, rank + 2 * state_n, generator=g).to(dtype)
        step, proj = torch.randn(n, inner, generator=g) - 1.0, torch.randn(n, 2 * inner, generator=g).to(dtype)
        data.append((x, low, step, proj))
    want = [plain_scan(x, low, rank, step, proj[:, inner:], a_log, d_skip) for x, low, step, proj in data]
    a = (-torch.exp(a_log)).contiguous().to(device)
    state = torch.zeros((6, inner * state_n), dtype=torch.float32, device=device)
    slots = i32([5, 2, 1, 3], device)
    for part, (lo, ns) in enumerate((([0] * 4, before), (before, lens))):
        live = [r for r in range(4) if ns[r]]
        cat = lambda j: torch.cat([data[r][j][lo[r]:lo[r] + ns[r]] for r in live]).to(device)
        cu = i32([0] + torch.tensor([ns[r] for r in live]).cumsum(0).tolist(), device)
        plan = ops.scan_plan([ns[r] for r in live], device, inner * state_n)
        need = ops.selective_workspace_floats(plan, inner, state_n)
        if device == "cuda" and part == 1:
            assert plan.num_chunks == 6 + 4 and plan.num_direct == 2 and need > 0
        room = torch.empty(max(need, 1), dtype=torch.float32, device=device)
        y = ops.selective_scan(cat(0), cat(1), rank, cat(2), cat(3), inner, a, d_skip.to(device), state, cu,
                               slots[torch.tensor(live)].contiguous(), len(live), plan=plan, workspace=room)
        if part == 1:
            at = 0
            for r in live:
                close(y[at:at + ns[r]], want[r][lo[r]:], dtype, scale=float(want[r].abs().max()))
                at += ns[r]


# ------------------------------------------------------------------ feed-forward, layer scale, frequencies

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,ff,limit", [(5, 40, 0.7), (70, 56, 1.0), (3, 128, 50.0), (33, 7, 0.2)])
def test_clamped_gate_times_up_plus_one(device, dtype, tokens, ff, limit):
    """Gate and up values on both sides of the limit (the gate is clamped from above only)."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    gu = (torch.randn(tokens, 2 * ff, generator=torch.Generator().manual_seed(ff)) * 2.0 * min(limit, 3.0)).to(dtype)
    g, u = gu.float()[:, :ff], gu.float()[:, ff:]
    g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    close(ops.silu_mul(gu.to(device), dtype, activation="swish_clamped", limit=limit, alpha=1.702), want, dtype, scale=float(want.abs().max()))
    if dtype == torch.float32:
        halves = torch.stack([gu * 0.25, gu * 0.75]).to(device)            # a product that comes as partial sums
        close(ops.silu_mul(halves, dtype, activation="swish_clamped", limit=limit, alpha=1.702), want, dtype, scale=float(want.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [1, 5, 8, 40, 200, 700])
@pytest.mark.parametrize("width,ff,limit", [(256, 512, 0.8), (512, 1024, 3.0), (128, 384, 0.3)])
def test_the_feed_forward_part_in_every_form_of_its_gate_up_product(tokens, width, ff, limit):
    """bfloat16: a few tokens take the weight-streaming kernel, many the tcgen05 product with the clamped gate in its
    epilogue, the rest the product and the stand-alone kernel; all against the plain feed-forward."""
    from lily_b200.csrc import ops
    from lily_b200.engine.batch import Workspace
    from lily_b200.parts.base import BuildContext, build_part
    from lily_b200.parts.mlp import SwiGLUSpec

    g = torch.Generator().manual_seed(tokens + ff)
    w = {"f.gate": torch.randn(ff, width, generator=g) / math.sqrt(width) * 2.0, "f.up": torch.randn(ff, width, generator=g) / math.sqrt(width) * 2.0,
         "f.down": torch.randn(width, ff, generator=g) / math.sqrt(ff)}
    w = {k: v.bfloat16() for k, v in w.items()}
    x = torch.randn(tokens, width, generator=g).bfloat16()
    want = pk.feed_forward(x.float(), {"p.mlp." + k[2:]: v.float() for k, v in w.items()}, "p.mlp", limit)
    ctx = BuildContext(device=torch.device("cuda"), dtype=torch.bfloat16, ops=ops)
    part = build_part("feed_forward", SwiGLUSpec(width, ff, activation="swish_clamped", limit=limit, alpha=1.702,
                                                 names=(("gate", "gate"), ("up", "up"), ("down", "down"))), "f", ctx)
    part.load(lambda name: w[name].cuda())

    class Step:
        workspace = Workspace("cuda")
    out = part.forward(x.cuda(), Step())
    out = out.sum(0) if out.dim() == 3 else out              # a few tokens: the down product comes as partial sums
    close(out, want, torch.bfloat16, scale=float(want.abs().max()))
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width", [(3, 48), (70, 256), (2, 1024), (9, 4096), (130, 200), (5, 50)])
def test_a_gain_per_column_on_the_way_into_the_stream(device, dtype, tokens, width):
    """``x += s * delta`` in float32 and the norm of the new rows, in one pass (every form of the kernel: a cluster a
    row, rows in registers, rows in shared memory), with and without gathered rows."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("the plain statements are checked in float32")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(width)
    resid, delta = torch.randn(tokens, width, generator=g), (torch.randn(tokens, width, generator=g) * 3.0).to(dtype)
    scale, gain = 0.6 + 0.2 * torch.randn(width, generator=g), (1.0 + 0.2 * torch.randn(width, generator=g))
    want_x = resid + scale * delta.float()
    want = pk.rms(want_x, 1e-5) * gain
    x = resid.clone().to(device)
    out = ops.add_normed_rmsnorm(x, delta.to(device), scale.to(device), 1e-5, 1.0, gain.to(device), 1e-5, dtype, normalise=False)
    close(x, want_x, torch.float32)
    close(out, want, dtype, scale=float(want.abs().max()))
    rows = i32([tokens - 1, 0], device)
    x = resid.clone().to(device)
    out = ops.add_normed_rmsnorm(x, delta.to(device), scale.to(device), 1e-5, 1.0, gain.to(device), 1e-5, dtype, rows=rows,
                                 write_residual=False, normalise=False)
    close(out, want[[tokens - 1, 0]], dtype, scale=float(want.abs().max()))
    close(x, resid, torch.float32)


def test_rotation_frequencies_in_all_three_bands():
    """Short waves keep their frequency, long ones are slowed by the factor, those between are blended; the engine's
    tables against the closed form."""
    from lily_b200.config.model_config import RopeScaling
    from lily_b200.parts.rope import RopeSpec, inverse_frequencies

    rot = {"dims": 16, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}}
    f = pk.rotary_frequencies(rot)
    plain = 100.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    wavelength = 2 * math.pi / plain
    kept, slowed = wavelength < 48 / 3.0, wavelength > 48 / 1.0
    assert kept.any() and slowed.any() and (~kept & ~slowed).any()
    assert torch.equal(f[kept], plain[kept]) and torch.allclose(f[slowed], plain[slowed] / 4.0)
    between = ~kept & ~slowed
    assert bool(((f[between] < plain[between]) & (f[between] > plain[between] / 4.0)).all())
    spec = RopeSpec(16, 16, 100.0, RopeScaling("llama3", 4.0, 1.0, 3.0, 48), exact_frequencies=True)
    torch.testing.assert_close(inverse_frequencies(spec), f.float(), rtol=1e-6, atol=0)
