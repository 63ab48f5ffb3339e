"""Fomanex on the device against the plain implementation: each mechanism alone (fed in portions beside another
request), a far rotated key that dominates across pages, a sink that takes nearly everything, a recurrence that forgets
at the rate of its decay and whose bonus reaches the current token alone, the router's choices under a correction, the
copies of the residual stream, whole models under every way of cutting the work, slots and pages used again, long
decoding through captured graphs, and greedy generation through the entry point and its scheduler."""
import json
import math
import os

import numpy as np
import pytest
import torch

from tests.plain import fomanex_plain as plain
from tests.fomanex_configs import FOMANEX, plain_inputs, write_fomanex_dir
from tests.replay_helpers import (collect, max_live_tokens, trace_mixed, trace_portions,
                                  trace_tail_decode, trace_whole)
from tests.test_fadosun_gpu import _rel, _run_mixer, _weights
from tests.test_zufusun_gpu import _run_feed_forward, replay

pytestmark = pytest.mark.gpu

# A position's error is norm(got - want) / norm(want) over its logits.  The norms of this design are element-wise and
# saturate, the sublayers' results are scaled down on their way into the stream, and the logits pass a cap: rounding
# errors stay the arithmetic's (1e-6 in float32, 1e-2 in bfloat16) except where a router's close call falls the other
# way.  A fault of a mechanism (a key too many, a lost state, a sink or a bonus left out, copies mixed the wrong way
# round) is 1e-2 or more in float32 at every position it touches.
TOL = {"float32": dict(median=5e-6, worst=2e-4), "bfloat16": dict(median=3e-2, worst=None, over=0.06, above=0.12)}
MIX_TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def assert_close(got, want, dtype, what=""):
    errs = sorted((float(np.linalg.norm(rows[p] - want[r][p]) / max(np.linalg.norm(want[r][p]), 1e-30)), r, p)
                  for r, rows in got.items() for p in rows)
    assert errs and all(np.isfinite(e[0]) for e in errs), f"{what} {dtype}: no output or a NaN"
    t = TOL[dtype]
    median, worst = errs[len(errs) // 2][0], errs[-1]
    assert median < t["median"], f"{what} {dtype}: median error {median:.3g}"
    if t["worst"] is not None:
        assert worst[0] < t["worst"], f"{what} {dtype}: worst error {worst[0]:.3g} at {worst[1:]}"
    else:
        over = sum(e[0] > t["above"] for e in errs)
        assert over <= max(2, int(t["over"] * len(errs))), f"{what} {dtype}: {over} of {len(errs)} positions over {t['above']}, worst {worst}"


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {name: write_fomanex_dir(name, str(tmp_path_factory.mktemp("fomanex_" + name))) for name in FOMANEX}


@pytest.fixture(scope="module")
def plain_logits(dirs):
    cache, inputs = {}, {}

    def get(name, requests):
        if name not in inputs:
            inputs[name] = plain_inputs(dirs[name])
        out = {}
        for rid, toks in requests.items():
            key = (name, tuple(toks))
            if key not in cache:
                cache[key] = plain.forward(*inputs[name], toks).numpy()
            out[rid] = cache[key]
        return out

    return get


def make_requests(name, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, FOMANEX[name]["json"]["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


LENGTHS = {"p": (1, 2, 37, 130), "q": (3, 18, 65, 150), "r": (2, 70, 140), "s": (1, 5, 64, 97)}


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(FOMANEX))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes(name, dtype, mode, page, dirs, plain_logits):
    """Whole prompts, a decoded tail, portions down to two tokens (and single ones), and four live requests whose
    slots and pages are used again, against each request alone in the plain implementation."""
    requests = make_requests(name, LENGTHS[name], seed=5)
    if mode == "mixed":
        requests = make_requests(name, LENGTHS[name] + (40, 21, 66, 9), seed=6)
    steps = {"whole": trace_whole, "tail": lambda r: trace_tail_decode(r, tail=45),
             "portions": lambda r: trace_portions(r, sizes=(7, 2, 19, 1, 3, 33, 2, 16, 5, 64)),
             "mixed": lambda r: trace_mixed(r, live=4, seed=3)}[mode](requests)
    outputs, _ = replay(dirs[name], dtype, steps, max_live_tokens(steps, round_to=page), page_tokens=page)
    assert_close(collect(steps, outputs), plain_logits(name, requests), dtype, f"{name} {mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_equals_the_prompt(dtype, dirs, plain_logits):
    """300 tokens one by one (captured graphs after the second step; every pass of the looped layers, the router's
    grouping and the key splits all inside them) against the whole sequence."""
    requests = make_requests("p", (300,), seed=11)
    steps = trace_tail_decode(requests, tail=299)
    outputs, runner = replay(dirs["p"], dtype, steps, 320)
    assert runner.graph_replays > 250
    assert_close(collect(steps, outputs), plain_logits("p", requests), dtype, "long decoding")
    eager, _ = replay(dirs["p"], dtype, steps, 320, cuda_graphs=False)
    assert max(float(np.abs(outputs[k] - eager[k]).max()) for k in outputs) < (1e-5 if dtype == "float32" else 1e-1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding(dtype, dirs, plain_logits):
    """1,300 tokens at a real model's head sizes: latent rows more than a thousand positions back, a state that has seen
    as many tokens, every layer twice: as one prompt with a decoded tail and as portions of 500."""
    requests = make_requests("r", (1300,), seed=17)
    for steps in (trace_tail_decode(requests, tail=24), trace_portions(requests, sizes=(500, 37, 500, 2))):
        outputs, _ = replay(dirs["r"], dtype, steps, 1344, page_tokens=64, max_batch_tokens=2048)
        assert_close(collect(steps, outputs), plain_logits("r", requests), dtype, "long prompt")


@pytest.mark.parametrize("name", ["q", "r"])
def test_a_slot_used_again_starts_from_zero(name, dirs, plain_logits):
    """One slot only: the second request gets the state, the last input and the pages the first left, in every pass."""
    requests = make_requests(name, (90, 75, 33), seed=21)
    steps = trace_portions(requests, sizes=(40, 3, 1, 31))
    outputs, _ = replay(dirs[name], "float32", steps, 96, max_requests=1)
    assert_close(collect(steps, outputs), plain_logits(name, requests), "float32", "one slot")


def test_every_pass_of_a_looped_layer_has_pages_and_state_of_its_own(dirs):
    from ember_b200.engine.batch import StepEntry
    from ember_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_dir(dirs["p"], dtype="float32", capacity_tokens=128, max_batch_tokens=128, max_requests=2, page_tokens=16)
    runner.admit("a")
    assert runner.reserve("a", 40)
    runner.step([StepEntry("a", make_requests("p", (40,), seed=2)["r0"], ())])
    # layer 0 once and layer 2 three times: four latent caches of three pages each, however they are grouped
    assert sum(u * len(g.layers) for u, g in zip(runner.cache.used_pages(), runner.cache.groups)) == 4 * 3
    runner.release("a")
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
