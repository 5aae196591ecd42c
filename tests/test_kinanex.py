"""The Kinanex decoder through the engine against its plain implementation (``plain_kinanex``), in every cutting:
whole prompts, token-by-token decoding, portions down to two tokens, mixed batches of unequal requests, pages and
slots that are freed and used again, long decoding, greedy generation through the entry point and
the scheduler.  The CPU variants run the engine's host side over the kernels' plain statements; the ``gpu`` variants
run the CUDA kernels in float32 and bfloat16."""

import copy
import tempfile

import pytest
import torch

import kinanex_models as km
import plain_kinanex
from harness import make_runner, run_mixed, run_portions, run_whole
from lily_b200.config.model_config import ConfigError
from lily_b200.engine.batch import StepEntry

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
CONFIGS = {"varied": km.VARIED, "sharp": km.SHARP, "wide": km.WIDE, "odd": km.ODD, "recurrent": km.RECURRENT}


def plain_logits(cfg, weights, ids, dtype="float32"):
    if dtype == "bfloat16":
        weights = {k: v.bfloat16().float() for k, v in weights.items()}
    with plain_kinanex.precision(torch.float64):
        return plain_kinanex.forward(cfg, weights, ids).float()


def close(got, want, dtype, what=""):
    err = (got - want).abs()
    if dtype == "float32":
        assert float(err.max()) < 2e-4 * max(1.0, float(want.abs().max())), f"{what}: max error {float(err.max()):.3e}"
    else:
        scale = float(want.abs().max())
        assert float(err.max()) < 0.04 * scale and float(err.mean()) < 0.006 * scale, \
            f"{what}: max error {float(err.max()):.3e}, mean {float(err.mean()):.3e} (logits up to {scale:.2f})"


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def setup(request):
    cfg = CONFIGS[request.param]
    with tempfile.TemporaryDirectory() as tmp:
        weights = km.make_weights(cfg, 11)
        yield cfg, weights, km.write_model_dir(tmp + "/m", cfg, weights)


def runner_for(path, device, dtype="float32", max_tokens=512, page_size=16, max_requests=4):
    return make_runner(path, dtype=dtype, device=device, max_tokens=max_tokens, page_size=page_size,
                       max_requests=max_requests, context_length=1024)


def dtypes(device, cfg=None):
    """bfloat16 on the GPU too, except for the configuration whose near one-hot attention turns a rounding of a score
    into another key (it is there for the exact comparison in float32)."""
    return ["float32"] if device == "cpu" or cfg is km.SHARP else ["float32", "bfloat16"]


@pytest.mark.parametrize("device", DEVICES)
def test_whole_decoded_and_in_portions(setup, device):
    """A prompt whole; its last 40 tokens one by one (over several page borders, the recurrences' states and the
    convolutions' last inputs carried from step to step); portions of changing sizes down to two tokens and single
    tokens between them; and from the first token on."""
    cfg, weights, path = setup
    ids = km.tokens(150, cfg["vocab"], 5)
    for dtype in dtypes(device, cfg):
        want = plain_logits(cfg, weights, ids, dtype)
        runner = runner_for(path, device, dtype)
        close(run_whole(runner, ids), want, dtype, "whole")
        close(run_portions(runner, ids, [110] + [1] * 40), want, dtype, "decoded")
        close(run_portions(runner, ids, [3, 2, 31, 2, 1, 1, 17, 2, 5, 1, 64, 2]), want, dtype, "portions")
        close(run_portions(runner, ids, [1] * 24 + [2] * 10), want, dtype, "from the first token on")
        assert runner.cache.held_pages() == [0] * len(runner.cache.groups) and runner.cache.slots.available == 4


@pytest.mark.parametrize("device", DEVICES)
def test_mixed_batches_with_pages_and_slots_used_again(setup, device):
    """Up to four live requests of unequal lengths, portions of some beside single tokens of others, in a pool that
    holds fewer tokens than all requests together and with four slots for six requests."""
    cfg, weights, path = setup
    lens = {"a": 90, "b": 41, "c": 70, "d": 33, "e": 58, "f": 20}
    reqs = {k: km.tokens(n, cfg["vocab"], 40 + i) for i, (k, n) in enumerate(lens.items())}
    plan = [{"a": 30, "b": 2, "c": 17}, {"a": 1, "b": 20, "c": 2, "d": 33}, {"a": 1, "b": 1, "c": 1},
            {"a": 28, "b": 18, "c": 50}, {"a": 1, "e": 16}, {"a": 1, "e": 1, "f": 3}, {"a": 28, "e": 41, "f": 17}]
    ends = {1: ["d"], 3: ["b", "c"]}
    for dtype in dtypes(device, cfg):
        runner = runner_for(path, device, dtype, max_tokens=16 * 16)
        got = run_mixed(runner, reqs, plan, ends)
        for k, ids in reqs.items():
            close(got[k], plain_logits(cfg, weights, ids, dtype), dtype, f"request {k}")
        assert runner.cache.held_pages() == [0] * len(runner.cache.groups) and runner.cache.slots.available == 4


@pytest.mark.parametrize("device", DEVICES)
def test_a_batch_changes_no_request(setup, device):
    """The logits of a request do not depend on what else is in the batch or on the slot and pages it got."""
    cfg, weights, path = setup
    reqs = {k: km.tokens(n, cfg["vocab"], 70 + i) for i, (k, n) in enumerate({"a": 37, "b": 64, "c": 9}.items())}
    runner = runner_for(path, device)
    alone = {k: run_portions(runner, ids, [len(ids) - 4, 1, 1, 1, 1]) for k, ids in reqs.items()}
    filler = runner.open_request()                       # the batch's requests get other slots and pages than alone
    runner.step([StepEntry(filler, km.tokens(21, cfg["vocab"], 1), [])])
    plan = [{k: len(ids) - 4 for k, ids in reqs.items()}] + [{k: 1 for k in reqs}] * 4
    together = run_mixed(runner, reqs, plan)
    runner.close_request(filler)
    for k in reqs:
        assert float((together[k] - alone[k]).abs().max()) < 1e-5 * max(1.0, float(alone[k].abs().max())), k


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_through_graphs(setup, device):
    """Three requests decode 70 tokens side by side (captured steps on the GPU): states in their slots, the first
    sharing layer's values handed to the later ones inside the captured step."""
    cfg, weights, path = setup
    reqs = {k: km.tokens(n, cfg["vocab"], 90 + i) for i, (k, n) in enumerate({"a": 100, "b": 81, "c": 75}.items())}
    plan = [{"a": 30, "b": 11, "c": 5}] + [{"a": 1, "b": 1, "c": 1}] * 70
    for dtype in dtypes(device, cfg):
        runner = runner_for(path, device, dtype)
        before = runner.graph_steps
        got = run_mixed(runner, reqs, plan)
        for k, ids in reqs.items():
            close(got[k], plain_logits(cfg, weights, ids, dtype), dtype, f"request {k}")
        if device == "cuda":
            assert runner.model.graph_safe and runner.graph_steps - before == 70


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_entry_point(device):
    """``Engine.generate`` (scheduler, sampler, cache manager) against greedy decoding with the plain implementation."""
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.sampling.params import SamplingParams

    cfg = km.VARIED
    with tempfile.TemporaryDirectory() as tmp:
        weights = km.make_weights(cfg, 12)
        path = km.write_model_dir(tmp + "/m", cfg, weights)
        runner = runner_for(path, device, max_tokens=640, max_requests=3)
        engine = Engine(EngineConfig(model_path=path, dtype="float32", device=device,
                                     server_args={"chunked_prefill_size": 32, "max_prefill_tokens": 48}), runner=runner)
        prompts = [km.tokens(n, cfg["vocab"], 200 + n) for n in (45, 7, 70, 1, 33)]
        out = engine.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
        for ids, res in zip(prompts, out):
            seq = list(ids)
            for tok in res["output_ids"]:
                logits = plain_logits(cfg, weights, seq)[-1]
                best = int(torch.argmax(logits))
                # a near-tie may fall either way: the chosen token must be (almost) the best one
                assert tok == best or float(logits[best] - logits[tok]) < 1e-3
                seq.append(tok)
            assert len(res["output_ids"]) == 12


def test_config_refuses_what_the_design_does_not_have():
    from lily_b200.config.kinanex_config import KinanexConfig

    KinanexConfig.from_dict(km.VARIED)
    for path, value in ((("layers", 0, "type"), "parallel"), (("layers", 1, "mlp", "kind"), "experts"),
                        (("layers", 2, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "heads"), 5),
                        (("layers", 1, "mixer", "heads"), 3), (("layers", 1, "mixer", "conv"), 0), (("layers", 3, "mixer", "state"), 0),
                        (("layers", 1, "mlp", "limit"), 0.0), (("layers", 4, "mixer", "vdim"), 16),
                        (("layers", 2, "mixer", "rot", "scaling", "factor"), 0.0)):
        cfg = copy.deepcopy(km.VARIED)
        node = cfg
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            KinanexConfig.from_dict(cfg)
    cfg = copy.deepcopy(km.VARIED)
    del cfg["layers"][3]["mixer"]["dt_rank"]
    with pytest.raises(ConfigError):
        KinanexConfig.from_dict(cfg)


def test_caches_and_states_follow_the_layers():
    """Attention layers of one shape share a cache group; every recurrent layer has a state row of its own: the
    matrices or state vectors, then the convolution's carried inputs."""
    with tempfile.TemporaryDirectory() as tmp:
        path = km.write_model_dir(tmp + "/m", km.VARIED, km.make_weights(km.VARIED, 3))
        runner = make_runner(path, max_tokens=64, page_size=8, max_requests=2, context_length=64)
        model = runner.model
        needs = {(n.kv_heads, n.head_dim, n.v_head_dim, n.window): layers for n, layers in model.cache_groups}
        assert needs == {(3, 12, 10, None): 1, (2, 16, 12, None): 1, (2, 24, 12, None): 1, (2, 8, 12, None): 1}
        assert [tuple(s.shape[1:]) for s in runner.cache.states] == [
            (4 * 12 * 20 + 1 * (24 + 24 + 80),), (40 * 6 + 3 * 40,), (3 * 20 * 7,), (24 * 19 + 1 * 24,), (2 * 8 * 16 + 3 * (8 + 8 + 32),)]
        # the first layer that shares its values keeps them; those behind it blend; the one that does not share does neither
        assert [b.mixer.spec.v_share for b in model.blocks if b.mixer.kind == "attention"] == [None, "first", "blend", "blend"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_tool_in_every_cutting(dtype):
    """``bin/trace_run`` as a subprocess: whole, last tokens one by one, portions, then four live requests with pages
    and state slots used again (six requests over four slots and a pool of five pages of 64)."""
    from test_trace_run_gpu import Trace, replay

    cfg = km.WIDE
    with tempfile.TemporaryDirectory() as tmp:
        weights = km.make_weights(cfg, 21)
        path = km.write_model_dir(tmp + "/m", cfg, weights)
        reqs = {k: km.tokens(n, cfg["vocab"], 300 + i) for i, (k, n) in enumerate(
            {"w": 150, "t": 140, "p": 131, "a": 100, "b": 70, "c": 64, "d": 90, "e": 40}.items())}
        t = Trace(reqs)
        t.step({"w": 150}, end=["w"])
        t.step({"t": 90})
        for i in range(50):
            t.step({"t": 1}, end=["t"] if i == 49 else [])
        for i, n in enumerate([8, 2, 30, 17, 2, 3, 40, 2, 5, 22]):
            t.step({"p": n}, end=["p"] if i == 9 else [])
        t.step({"a": 60})
        t.step({"a": 1, "b": 33})
        t.step({"a": 1, "b": 2, "c": 64}, want={"c": [63, 0]})
        t.step({"b": 35, "a": 1, "d": 5}, end=["c"])
        t.step({"a": 37, "d": 2}, end=["b"])
        t.step({"d": 83, "e": 3}, end=["a"])
        t.step({"e": 1}, end=["d"])
        t.step({"e": 36}, end=["e"])
        rows = replay(path, dtype, t.steps, 320, tmp, cfg["vocab"])
        plain = {k: plain_logits(cfg, weights, ids, dtype) for k, ids in reqs.items()}
        for i, expect in enumerate(t.expect):
            want = torch.stack([plain[k][pos] for k, pos in expect])
            close(rows[i], want, dtype, f"step {i}")


@pytest.mark.parametrize("device", DEVICES)
def test_a_long_prompt_whole_and_cut(device):
    """700 tokens: far keys among hundreds, recurrences over hundreds of steps, whole and cut at odd places, beside
    a short request in the same step."""
    cfg = km.WIDE
    with tempfile.TemporaryDirectory() as tmp:
        weights = km.make_weights(cfg, 14)
        path = km.write_model_dir(tmp + "/m", cfg, weights)
        ids, other = km.tokens(700, cfg["vocab"], 6), km.tokens(30, cfg["vocab"], 7)
        for dtype in dtypes(device, cfg):
            want, want_other = plain_logits(cfg, weights, ids, dtype), plain_logits(cfg, weights, other, dtype)
            runner = runner_for(path, device, dtype, max_tokens=1024, page_size=64)
            close(run_whole(runner, ids), want, dtype, "whole")
            close(run_portions(runner, ids, [333, 2, 1, 364]), want, dtype, "portions")
            got = run_mixed(runner, {"a": ids, "b": other}, [{"a": 450, "b": 29}, {"a": 250, "b": 1}])
            close(got["a"], want, dtype, "beside a short request")
            close(got["b"], want_other, dtype, "the short request")
