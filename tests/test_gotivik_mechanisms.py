"""Each mechanism of the Gotivik decoder alone: the kernels' faces (CUDA on the GPU, their plain statements on the
CPU) and the parts that use them against the functions of ``plain_gotivik``, with inputs made so that a fault shows:
one key scaled to stand out among the kept first positions, just behind them, at a page border and at both sides of
the window's edge; states carried over portions of every length down to two tokens; positions at both sides of a
step of the query temperature; sizes that take the tensor-core kernels and sizes that are not powers of two."""

import math

import pytest
import torch

import kernel_refs
import plain_gotivik as pg

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


# ------------------------------------------------------------------ window with kept first positions

def run_attention(ops, device, dtype, q, k, v, scale, window, keep, page, cuts, softcap=None):
    """q [t, H, d], k [t, G, d], v [t, G, dv] through the cache write and the attention kernels, the sequence cut into
    the portions ``cuts`` (a portion of one token takes the decode kernel); pages come in a scrambled order."""
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
    done = 0
    for n in cuts:
        rows = qkv[done:done + n].contiguous()
        pos = i32(list(range(done, done + n)), device)
        qq = ops.qk_norm_rope_write(rows, None, None, 1e-6, None, None, pos, i32([0] * n, device), table, cache, heads, kvh,
                                    d, 0, page, **sized)
        o = torch.empty((n, heads * dv), dtype=dtype, device=device)
        if n == 1:
            plan = ops.plan_decode_attention(dtype, 1, heads, kvh, d, done + 1, keep_first=keep, **sized)
            scratch = torch.empty(max(1, plan.scratch_floats), dtype=torch.float32, device=device)
            ops.attention_decode(qq, cache, table, i32([done + 1], device), o, scratch, plan.splits, heads, kvh, d, page, scale,
                                 window, softcap=softcap, keep_first=keep, **sized)
        else:
            tile = ops.prefill_tile_rows(dtype, d, page, n, softcap=softcap, keep_first=keep, **sized)
            tr, ts = ops.prefill_tiles([done], [n], 0, tile, device)
            ops.attention_prefill(qq, cache, table, i32([0, n], device), i32([done], device), tr, ts, o, heads, kvh, d, page,
                                  scale, window, tile_rows=tile, softcap=softcap, keep_first=keep, **sized)
        out[done:done + n] = o
        done += n
    assert done == t
    return out.float().cpu().view(t, heads, dv)


KEPT_CASES = [  # heads, kv heads, d, dv, page, window, kept first positions, tokens
    (4, 2, 16, 24, 16, 37, 5, 230),          # CUDA-core kernels, a value size of its own
    (3, 1, 40, 40, 8, 20, 19, 150),          # nearly as many kept as the window holds
    (2, 1, 24, 24, 16, 9, 40, 120),          # more kept than the window holds
    (4, 2, 64, 64, 64, 70, 3, 700),          # tensor-core kernels: prefill in tiles of 64 and 128 rows, decode
    (2, 1, 128, 128, 64, 130, 64, 700),      # kept positions fill a key tile of the decode kernel exactly
    (4, 1, 128, 128, 64, 200, 131, 900),     # ... and spill into a second tile of 128 keys
    (2, 2, 192, 192, 32, 100, 7, 420),
]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d,dv,page,window,keep,t", KEPT_CASES)
@pytest.mark.parametrize("cut", ["whole", "mixed", "decoded"])
def test_kept_first_positions_and_the_windows_edge(device, dtype, heads, kvh, d, dv, page, window, keep, t, cut):
    """Keys many times larger than the rest draw nearly all weight of every query that sees them.  They stand at the
    last kept position, at the first that is not kept, at a page border inside the window's reach and far back: a
    query sees the last kept one from any distance, the next one only from up to ``window - 1`` positions behind."""
    if device == "cpu" and (dtype == torch.bfloat16 or t > 300):
        pytest.skip("the plain statements are checked in float32 on the short cases")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(d + dv + keep)
    q = torch.randn(t, heads, d, generator=g)
    k = torch.randn(t, kvh, d, generator=g) * 0.3
    v = torch.randn(t, kvh, dv, generator=g)
    marks = sorted({0, keep - 1, keep, keep + 1, 2 * page - 1, 2 * page, t // 2})
    for m in marks:                               # every later query scores high against these keys
        k[m] = 0.0
        k[m, :, 0] = 5.0 * math.sqrt(d)
    q[:, :, 0] = q[:, :, 0].abs() + 1.0
    scale = d ** -0.5
    cuts = {"whole": [t], "mixed": portions(t, [129, 2, 1, 64, 200, 3, 1, 1, 77]),
            "decoded": [t - 40] + [1] * 40}[cut]
    got = run_attention(ops, device, dtype, q, k, v, scale, window, keep, page, cuts)
    as_stored = lambda x: x.to(dtype).float()
    want = pg.softmax_attention(as_stored(q), as_stored(k), as_stored(v), scale, pg.visible(t, window, keep))
    close(got, want, dtype)
    # the marked keys decide the outputs: without the kept positions the result is another one
    other = pg.softmax_attention(as_stored(q), as_stored(k), as_stored(v), scale, pg.visible(t, window, 0))
    assert (other - want).abs().max() > 0.5


@pytest.mark.parametrize("device", DEVICES)
def test_kept_positions_need_a_window(device):
    """Without a window every earlier key is seen and the number of kept positions changes nothing."""
    ops = ops_for(device)
    g = torch.Generator().manual_seed(3)
    t, heads, kvh, d, page = 90, 2, 1, 16, 16
    q, k, v = torch.randn(t, heads, d, generator=g), torch.randn(t, kvh, d, generator=g), torch.randn(t, kvh, d, generator=g)
    a = run_attention(ops, device, torch.float32, q, k, v, 0.25, None, 7, page, [50, 1, 39])
    b = run_attention(ops, device, torch.float32, q, k, v, 0.25, None, 0, page, [50, 1, 39])
    assert torch.equal(a, b)
    close(a, pg.softmax_attention(q, k, v, 0.25, pg.visible(t, None, 0)), torch.float32)


# ------------------------------------------------------------------ short convolution with its state

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,channels,extra", [(4, 40, 0), (2, 24, 8), (3, 200, 0), (1, 16, 4), (4, 1536, 0)])
def test_convolution_over_portions_and_slots(device, dtype, taps, channels, extra):
    """The convolution without activation over three requests whose tokens come in portions of every size (two
    tokens and single tokens among them), several requests a step, the state rows of a finished request given to the
    next one: equal to the convolution of each whole sequence with zeros ahead of its start."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("one precision on the CPU")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(taps * 100 + channels)
    lens = [97, 33, 150]
    col0 = 8
    width = col0 + channels + extra
    seqs = [torch.randn(n, width, generator=g).to(dtype) for n in lens]
    w = torch.randn(channels, taps, generator=g) * 0.6
    want = [pg.causal_conv(s[:, col0:col0 + channels].float(), w) for s in seqs]
    state = torch.full((3, (taps - 1) * channels + 5), 7.0, dtype=torch.float32, device=device)     # two slots (1, 2); stale numbers
    off = 5
    cuts = [portions(lens[0], [2, 1, 30, 1, 64, 3]), portions(lens[1], [1, 2, 5, 70]), portions(lens[2], [66, 2, 2, 1, 128])]
    got = [[] for _ in lens]
    # requests 0 and 1 run side by side in slots 1 and 2; request 2 then takes slot 1 again
    schedule = []
    a, b = list(cuts[0]), list(cuts[1])
    while a or b:
        step = []
        if a:
            step.append((0, 1, a.pop(0)))
        if b:
            step.append((1, 2, b.pop(0)))
        schedule.append(step)
    schedule += [[(2, 1, n)] for n in cuts[2]]
    done = [0, 0, 0]
    for step in schedule:
        for r, slot, _ in step:
            if done[r] == 0 and taps > 1:
                state[slot, off:off + (taps - 1) * channels] = 0.0           # a new request starts from zeros
        rows = torch.cat([seqs[r][done[r]:done[r] + n] for r, _, n in step]).to(device).contiguous()
        news = [n for _, _, n in step]
        cu = i32([0] + torch.tensor(news).cumsum(0).tolist(), device)
        slots = i32([slot for _, slot, _ in step], device)
        chunk_req, chunk_start = ops.token_chunks(news, ops.SSM_CHUNK, device)
        out = ops.causal_conv(rows, col0, channels, w.to(device), None, state, off, chunk_req, chunk_start, cu, slots,
                              ops.SSM_CHUNK, activation="none")
        at = 0
        for r, _, n in step:
            got[r].append(out[at:at + n].float().cpu())
            at += n
            done[r] += n
    for r in range(3):
        close(torch.cat(got[r]), want[r], dtype, scale=3.0)
    assert torch.all(state[:, :off] == 7.0) and torch.all(state[0] == 7.0)


# ------------------------------------------------------------------ rotation tables

@pytest.mark.parametrize("dims,head,base,scaling", [
    (8, 16, 100.0, {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 0.5}),
    (16, 48, 3000.0, {"factor": 2.5, "original": 512, "fast": 24.0, "slow": 2.0}),
    (64, 128, 1000000.0, {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}),
    (12, 12, 50.0, None),
    (6, 24, 10.0, {"factor": 3.0, "original": 8, "fast": 1.0, "slow": 1.0}),         # a ramp of no width
])
def test_rotation_tables_and_the_kernel_that_rotates(dims, head, base, scaling):
    """The tables the mixer hands to the kernel equal cos and sin of position x scaled frequency, stretched; and
    rotating by them pairs feature i with feature i + dims / 2 and leaves the features past ``dims`` alone."""
    from lily_b200.config.model_config import RopeScaling
    from lily_b200.parts.base import BuildContext, build_part
    from lily_b200.parts.rope import RopeSpec

    rot = {"dims": dims, "base": base}
    sc = RopeScaling()
    if scaling:
        rot["scaling"] = scaling
        sc = RopeScaling("yarn", factor=scaling["factor"], original_max_position_embeddings=scaling["original"],
                         fast_turns=scaling["fast"], slow_turns=scaling["slow"])
    ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32, ops=kernel_refs, page_size=16, max_position=3000)
    cos, sin = build_part("position", RopeSpec(head, dims, base, sc, exact_frequencies=True), "x", ctx).tables()
    f, stretch = pg.yarn_frequencies(rot)
    pos = torch.arange(3000)
    ang = pos.float()[:, None] * f[None, :]
    torch.testing.assert_close(cos, ang.cos() * stretch, atol=2e-6, rtol=0)
    torch.testing.assert_close(sin, ang.sin() * stretch, atol=2e-6, rtol=0)
    if scaling and scaling["fast"] != scaling["slow"]:
        plain, _ = pg.yarn_frequencies({"dims": dims, "base": base})
        assert not torch.equal(plain, f) and f[0] == plain[0]                # the fastest wave keeps its frequency
    # through the kernel's face: q and k rotated at positions far apart, the rest of the head untouched
    g = torch.Generator().manual_seed(dims)
    n, heads = 5, 2
    at = torch.tensor([0, 1, 17, 1500, 2999])
    x = torch.randn(n, heads + 1, head, generator=g)
    v = torch.randn(n, head, generator=g)
    qkv = torch.cat([x.reshape(n, -1), v], 1)
    cache = torch.zeros(3000 // 16 + 2, 2, 1, 16, head)
    table = (torch.arange(3000 // 16 + 1, dtype=torch.int32) + 1).view(1, -1)
    q = kernel_refs.qk_norm_rope_write(qkv, None, None, 1e-6, cos, sin, at.int(), torch.zeros(n, dtype=torch.int32), table, cache,
                                       heads, 1, head, dims, 16)
    want = pg.rotate_halves(x, at, f, stretch)
    torch.testing.assert_close(q.view(n, heads, head), want[:, :heads], atol=1e-5, rtol=1e-5)
    for j, p in enumerate(at.tolist()):
        torch.testing.assert_close(cache[int(table[0, p // 16]), 0, 0, p % 16], want[j, heads], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(cache[int(table[0, p // 16]), 1, 0, p % 16], v[j])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_kernel_with_stretched_tables(dtype):
    """The CUDA kernel with partial rotation and stretched tables against the plain rotation."""
    from lily_b200.csrc import ops
    dims, head, heads, n = 32, 64, 3, 6
    rot = {"dims": dims, "base": 5000.0, "scaling": {"factor": 2.0, "original": 256, "fast": 8.0, "slow": 1.0}}
    f, stretch = pg.yarn_frequencies(rot)
    at = torch.tensor([0, 3, 255, 256, 1000, 2047])
    ang = torch.arange(2048).float()[:, None] * f[None, :]
    cos, sin = (ang.cos() * stretch).cuda(), (ang.sin() * stretch).cuda()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n, heads + 1, head, generator=g).to(dtype)
    v = torch.randn(n, head, generator=g).to(dtype)
    qkv = torch.cat([x.reshape(n, -1), v], 1).cuda()
    cache = torch.zeros(2048 // 64 + 1, 2, 1, 64, head, dtype=dtype, device="cuda")
    table = (torch.arange(2048 // 64, dtype=torch.int32, device="cuda") + 1).view(1, -1)
    q = ops.qk_norm_rope_write(qkv, None, None, 1e-6, cos, sin, at.int().cuda(), torch.zeros(n, dtype=torch.int32, device="cuda"),
                               table, cache, heads, 1, head, dims, 64)
    want = pg.rotate_halves(x.float(), at, f, stretch)
    close(q.view(n, heads, head), want[:, :heads], dtype, scale=2.0)
    for j, p in enumerate(at.tolist()):
        close(cache[p // 64 + 1, 0, 0, p % 64], want[j, heads], dtype, scale=2.0)


# ------------------------------------------------------------------ differential attention: queries, difference, gate

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d,dv,every,extra", [(4, 2, 8, 12, 7, 4), (3, 1, 16, 16, 1, 3), (4, 2, 32, 64, 64, 4),
                                                        (8, 2, 64, 128, 256, 8), (2, 2, 12, 20, 1000, 2)])
def test_queries_of_the_maps_and_their_temperature(device, dtype, heads, kvh, d, dv, every, extra):
    """Positions on both sides of every step of the temperature (``every - 1`` is the last position of a step, since
    the count is of ``p + 1``), position 0, and far ones; each map's query lands in its own columns of its own query
    head with zeros beside it, keys and values at the token's place in its page."""
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("one precision on the CPU")
    ops = ops_for(device)
    coef, page = 0.4, 16
    at = sorted({0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 2 * every, 5 * every - 1, 5 * every + 3} - {-1})
    n = len(at)
    kd = 2 * d
    g = torch.Generator().manual_seed(heads + d)
    proj = torch.randn(n, (heads + kvh) * kd + kvh * dv + extra, generator=g).to(dtype)
    pages = at[-1] // page + 1
    table = (torch.randperm(pages, generator=g).int() + 1).view(1, pages)
    shape = (pages + 1, 2, kvh, page, kd) if dv == kd else (pages + 1, kvh * page * (kd + dv))
    cache = torch.zeros(shape, dtype=dtype, device=device)
    q = ops.diff_prepare(proj.to(device), i32(at, device), i32([0] * n, device), table.to(device), cache, heads, kvh, d, dv, 2, page,
                         coef, every)
    temp = pg.query_temperature(at[-1] + 1, {"coef": coef, "every": every})[at]
    assert temp[0] == (1.0 if every > 1 else 1.0 + coef * math.log(2.0))
    src = proj.float()[:, :heads * kd].view(n, heads, 2, d) * temp[:, None, None, None]
    got = q.float().cpu().view(n, heads, 2, 2, d)
    for m in range(2):
        close(got[:, :, m, m], src[:, :, m], dtype, scale=4.0)
        assert torch.all(got[:, :, m, 1 - m] == 0)
    keys, values = kernel_refs._pages(cache.cpu(), kvh, page, kd, dv)
    for j, p in enumerate(at):
        pgn = int(table[0, p // page])
        assert torch.equal(keys[pgn, :, p % page].reshape(-1), proj[j, heads * kd:(heads + kvh) * kd])
        assert torch.equal(values[pgn, :, p % page].reshape(-1), proj[j, (heads + kvh) * kd:(heads + kvh) * kd + kvh * dv])
    # with write_kv off the cache stays as it is
    before = cache.clone()
    ops.diff_prepare(proj.to(device) * 2, i32(at, device), i32([0] * n, device), table.to(device), cache, heads, kvh, d, dv, 2, page,
                     coef, every, write_kv=False)
    assert torch.equal(before, cache)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dv,extra", [(4, 12, 5), (3, 16, 0), (4, 64, 8), (8, 128, 8), (2, 256, 16), (2, 520, 8), (5, 20, 3)])
def test_difference_unit_norm_and_gate(device, dtype, heads, dv, extra):
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("one precision on the CPU")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(heads * dv)
    n, lam, diff, eps = 9, 0.73, 0.3, 1e-5
    maps_out = torch.randn(n, heads, 2, dv, generator=g).to(dtype)
    maps_out[0] = 0.0                                                       # a row of zeros: eps keeps the division finite
    maps_out[1, :, 1] = maps_out[1, :, 0] / lam                             # the maps cancel (up to rounding)
    proj = (torch.randn(n, extra + heads, generator=g) * 3).to(dtype)
    got = ops.diff_combine(maps_out.view(n, -1).to(device), proj.to(device), extra, heads, dv, 2, lam, 1.0 - diff, eps)
    a = maps_out.float()
    o = pg.rms(a[:, :, 0] - lam * a[:, :, 1], eps) * (1.0 - diff) * torch.sigmoid(proj.float()[:, extra:])[:, :, None]
    keep = torch.ones(n, dtype=torch.bool)
    keep[1] = False                                                         # a difference of rounding errors has no stable direction
    close(got.view(n, heads, dv)[keep], o[keep], dtype)
    assert torch.isfinite(got).all() and torch.all(got[0] == 0)


def test_lambda_of_a_layer():
    """The mixer's lambda from the four vectors, as the plain implementation forms it."""
    from lily_b200.parts.base import BuildContext, build_part
    from lily_b200.parts.diff_attention import DiffAttentionSpec
    g = torch.Generator().manual_seed(4)
    d, width = 8, 16
    spec = DiffAttentionSpec(width, 2, 1, d, 12, 0.3, 0.35, 1e-5, names=(("lq1", "lq1"), ("lk1", "lk1"), ("lq2", "lq2"), ("lk2", "lk2"),
                                                                         ("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g")))
    ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32, ops=kernel_refs, page_size=16)
    part = build_part("mixer", spec, "m", ctx)
    w = {name: torch.randn(t.shape, generator=g) * 0.5 for name, t in part.tensors().items()}
    part.load(lambda name: w[name])
    assert abs(part.lam - pg.differential_lambda(w, "m", 0.35)) < 1e-12
    assert abs(part.lam - 0.35) > 1e-3


# ------------------------------------------------------------------ norms on both sides of a sublayer, squared ReLU

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,tokens", [(48, 5), (136, 70), (128, 3), (256, 100), (1024, 65), (2048, 9), (2048, 130), (4096, 66),
                                          (8192, 3), (8192, 70), (3000, 67)])
def test_add_with_a_norm_on_both_sides(device, out_dtype, width, tokens):
    """``x + m * N_b(delta)`` in float32 and ``N(.)`` of the sum, for widths and row counts that take each form of
    the kernel (rows in registers, in shared memory, shared by a cluster), the delta in either precision or as float32
    partial sums, with the stream written back or only some rows' outputs formed."""
    if device == "cpu" and (out_dtype == torch.bfloat16 or width > 2048):
        pytest.skip("one precision and the smaller widths on the CPU")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(width + tokens)
    eps_b, eps, m = 1e-5, 1e-6, 0.7
    x = torch.randn(tokens, width, generator=g)
    post, gain = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
    for form in ("same dtype", "partial sums"):
        delta = torch.randn(tokens, width, generator=g) * 5
        delta = delta.to(out_dtype) if form == "same dtype" else torch.stack([delta * 0.25, delta * 0.5, delta * 0.25])
        summed = delta.float() if form == "same dtype" else delta.sum(0)
        new = x + m * (pg.rms(summed, eps_b) * post)
        want = pg.rms(new, eps) * gain
        stream = x.clone().to(device)
        got = ops.add_normed_rmsnorm(stream, delta.to(device), post.to(device), eps_b, m, gain.to(device).to(out_dtype), eps, out_dtype)
        close(got, want, out_dtype, scale=2.0)
        torch.testing.assert_close(stream.cpu(), new, atol=1e-5, rtol=1e-5)
        # only some rows' outputs, the stream left alone
        rows = i32([tokens - 1, 0, tokens // 2], device)
        stream = x.clone().to(device)
        some = ops.add_normed_rmsnorm(stream, delta.to(device), post.to(device), eps_b, m, gain.to(device).to(out_dtype), eps, out_dtype,
                                      rows=rows, write_residual=False)
        close(some, want[rows.long().cpu()], out_dtype, scale=2.0)
        assert torch.equal(stream.cpu(), x)
        # the add alone
        stream = x.clone().to(device)
        assert ops.add_normed_rmsnorm(stream, delta.to(device), post.to(device), eps_b, m, None, eps, out_dtype) is None
        torch.testing.assert_close(stream.cpu(), new, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,cols", [(3, 40), (70, 392), (5, 1000), (33, 4099)])
def test_squared_relu(device, dtype, tokens, cols):
    if device == "cpu" and dtype == torch.bfloat16:
        pytest.skip("one precision on the CPU")
    ops = ops_for(device)
    g = torch.Generator().manual_seed(cols)
    z = (torch.randn(tokens, cols, generator=g) * 3).to(dtype)
    z[0, :4] = torch.tensor([0.0, -0.0, -1e-3, 1e-3]).to(dtype)
    close(ops.activation(z.to(device), dtype, "relu2"), pg.relu_squared(z.float()), dtype, scale=4.0)
    parts = torch.stack([z.float() * 0.5, z.float() * 0.5])
    close(ops.activation(parts.to(device), dtype, "relu2"), pg.relu_squared(z.float()), dtype, scale=4.0)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("width,ff,tokens", [(48, 40, 7), (128, 392, 3), (256, 200, 70)])
def test_feed_forward_part(device, width, ff, tokens):
    """The feed-forward part (product, squared ReLU, product) against ``down(relu(up h)^2)``."""
    from lily_b200.parts.base import BuildContext, build_part
    from lily_b200.parts.mlp import DenseMLPSpec
    ctx = BuildContext(device=torch.device(device), dtype=torch.float32, ops=ops_for(device), page_size=16)
    part = build_part("feed_forward", DenseMLPSpec(width, ff, activation="relu2", names=(("up", "up"), ("down", "down"))), "l0.mlp", ctx)
    g = torch.Generator().manual_seed(ff)
    w = {name: torch.randn(t.shape, generator=g) / math.sqrt(t.shape[-1]) for name, t in part.tensors().items()}
    assert sorted(w) == ["l0.mlp.down", "l0.mlp.up"]
    part.load(lambda name: w[name].to(device))
    h = torch.randn(tokens, width, generator=g)
    got = part.forward(h.to(device), None)
    got = got.sum(0) if got.dim() == 3 else got                              # float32 partial sums for a few tokens
    close(got, pg.feed_forward(h, w, "l0.mlp"), torch.float32, scale=2.0)
