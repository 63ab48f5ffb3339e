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


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layer orders, sizes, head counts, copies, loops and constants drawn from a seed: whole prompts, portions and a
    mixed batch in float32 (the sharper comparison), the mixed batch in bfloat16."""
    from tests.fomanex_configs import drawn_fomanex, write_drawn_dir
    d = write_drawn_dir(seed, str(tmp_path))
    inputs = plain_inputs(d)
    rng = np.random.default_rng(100 + seed)
    vocab = drawn_fomanex(seed)["vocab"]
    requests = {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate((1, 2, int(rng.integers(30, 90)), int(rng.integers(100, 200)), 47, 19))}
    want = {rid: plain.forward(*inputs, toks).numpy() for rid, toks in requests.items()}
    for dtype, modes in (("float32", ("whole", "portions", "mixed")), ("bfloat16", ("mixed",))):
        for mode in modes:
            steps = {"whole": trace_whole, "portions": lambda r: trace_portions(r, sizes=(7, 2, 19, 1, 3, 33, 2, 16, 5, 64)),
                     "mixed": lambda r: trace_mixed(r, live=4, seed=seed)}[mode](requests)
            page = (16, 64)[seed % 2]
            outputs, _ = replay(d, dtype, steps, max_live_tokens(steps, round_to=page), page_tokens=page)
            assert_close(collect(steps, outputs), want, dtype, f"drawn {seed} {mode}")


@pytest.mark.parametrize("name", ["p", "q"])
def test_weights_stored_in_float32_serve_a_bfloat16_run(name, tmp_path, plain_logits, dirs):
    """The same values stored as float32: products keep the stored precision where they have a form for it and round
    to bfloat16 where they do not; either way the run is the bfloat16 one to rounding."""
    from ember_b200.weights.safetensors_io import save_file
    from tests.plain.qwen3_plain import read_safetensors
    d = write_fomanex_dir(name, str(tmp_path))
    path = os.path.join(d, "model.safetensors")
    save_file({k: (v.float() if v.is_floating_point() else v) for k, v in read_safetensors(path).items()}, path)
    requests = make_requests(name, (2, 50, 90), seed=8)
    steps = trace_portions(requests, sizes=(33, 2, 1, 16))
    outputs, _ = replay(d, "bfloat16", steps, 192)
    assert_close(collect(steps, outputs), plain_logits(name, requests), "bfloat16", "float32 weights")


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


# ------------------------------------------------------------------------ the mechanisms, each alone
from tests.test_zufusun_gpu import attention_kernel  # noqa: E402,F401  (a fixture: tensor-core or general attention)


def _latent_spec(heads, dim, rot_dim, vdim, kv_rank, rot, hidden, scale=0.2, eps=1e-6):
    from ember_b200.config import LatentAttentionSpec, NoPositionSpec, RotarySpec
    pos = NoPositionSpec()
    if rot_dim:
        sc = rot.get("scaling")
        kw = dict(scaling_factor=sc["factor"], scaling_original=sc["original"], scaling_fast=sc["fast"], scaling_slow=sc["slow"]) if sc else {}
        pos = RotarySpec(head_dim=rot_dim, rotary_dim=rot["dims"], theta=rot["base"], frequency_precision="float64", layout="half", **kw)
    return LatentAttentionSpec(hidden_size=hidden, num_heads=heads, head_dim=dim, rot_dim=rot_dim, value_dim=vdim, q_rank=0,
                               kv_rank=kv_rank, scale=scale, norm_eps=eps, sink=True, gate=False, own_kv=True, position=pos)


def _m(heads, dim, rot_dim, vdim, kv_rank, rot, scale=0.2):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


def _scaling(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _latent_plain(x, w, m, eps=1e-6):
    return plain.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", m, eps)


LATENT_CASES = [
    (3, 24, 8, 20, 40, {"dims": 8, "base": 1e4, "scaling": _scaling(8.0, 64, 16.0, 2.0)}, 64),
    (2, 32, 16, 48, 72, {"dims": 16, "base": 500.0}, 100),                                       # no stretching
    (40, 8, 4, 6, 20, {"dims": 4, "base": 77.0, "scaling": _scaling(2.0, 16, 8.0, 0.5)}, 64),    # forty heads on one latent
    (4, 128, 64, 128, 256, {"dims": 64, "base": 1e6, "scaling": _scaling(4.0, 128, 32.0, 1.0)}, 128),
    (1, 16, 2, 16, 512, {"dims": 2, "base": 10.0, "scaling": _scaling(16.0, 32, 4.0, 1.0)}, 72),  # one pair, the widest latent
    (2, 16, 0, 24, 32, {}, 64),                                                                   # nothing rotated
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rot_dim,vdim,kv_rank,rot,hidden", LATENT_CASES)
def test_latent_attention_alone(dtype, heads, dim, rot_dim, vdim, kv_rank, rot, hidden, attention_kernel):
    """Queries straight from the input, the cached latent with the up-projections folded around the attention against
    keys and values built per head, rotate-half pairs with stretched and unstretched frequencies."""
    spec = _latent_spec(heads, dim, rot_dim, vdim, kv_rank, rot, hidden)
    w = _weights(spec, seed=heads, std=0.12)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(8)).bfloat16()
    assert _rel(_run_mixer(spec, w, x, dtype), _latent_plain(x, w, _m(heads, dim, rot_dim, vdim, kv_rank, rot))) < MIX_TOL[dtype]


@pytest.mark.parametrize("heads,dim,rot_dim,vdim,kv_rank,rot,hidden", [LATENT_CASES[3], (16, 16, 16, 16, 48, {"dims": 16, "base": 1e4}, 64),
                                                                      (3, 24, 16, 20, 64, {"dims": 16, "base": 500.0, "scaling": _scaling(4.0, 64, 32.0, 1.0)}, 72)])
def test_latent_attention_on_tensor_cores(heads, dim, rot_dim, vdim, kv_rank, rot, hidden):
    """bfloat16 portions of 65 tokens and more on the tensor-core kernel, decoded tokens beside them and after them."""
    spec = _latent_spec(heads, dim, rot_dim, vdim, kv_rank, rot, hidden)
    w = _weights(spec, seed=heads, std=0.12)
    x = torch.randn(200, hidden, generator=torch.Generator().manual_seed(8)).bfloat16()
    got = _run_mixer(spec, w, x, torch.bfloat16, portions=((100, 3), (30, 40), (68, 1), (1, 1), (1, 1)))
    assert _rel(got, _latent_plain(x, w, _m(heads, dim, rot_dim, vdim, kv_rank, rot))) < MIX_TOL[torch.bfloat16]


@pytest.mark.parametrize("portions", [((200, 3),), ((120, 3), (40, 30), (38, 1), (1, 1), (1, 1)), ((2, 1),) * 50 + ((100, 1),)])
def test_a_far_rotated_key_that_dominates_is_seen_across_pages_and_portions(portions):
    """Scores that rest on the rotated key part alone (the unrotated queries are zero): a far key whose rotated part is
    large, queries that match it only if both were turned by their own positions' stretched angles, pair i with pair
    i + dims / 2, and multiplied by the stretching's magnitude."""
    heads, dim, rot_dim, vdim, hidden, T, far = 2, 8, 16, 24, 64, 200, 5
    rot = {"dims": 16, "base": 30.0, "scaling": _scaling(6.0, 40, 4.0, 0.5)}
    spec = _latent_spec(heads, dim, rot_dim, vdim, 24, rot, hidden, scale=1.0)
    w = _weights(spec, seed=4, std=0.1)
    w["m.sink"] = torch.full((heads,), -30.0).bfloat16()
    q = w["m.q"].float().view(heads, dim + rot_dim, hidden)
    q[:, :dim] = 0.0                                         # no unrotated score
    w["m.q"] = q.reshape(-1, hidden).bfloat16()
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(6))
    x[far] *= 6.0                                            # (the shared key part is not normed: it grows with the input)
    x = x.bfloat16()
    m = _m(heads, dim, rot_dim, vdim, 24, rot, scale=1.0)
    want = _latent_plain(x, w, m)
    for other in ({"dims": 16, "base": 30.0}, {"dims": 16, "base": 1e30}):                       # unstretched; (nearly) unturned
        assert _rel(_latent_plain(x, w, {**m, "rot": other})[150:], want[150:]) > 0.05
    assert _rel(_run_mixer(spec, w, x, torch.float32, portions=portions), want) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_sink_that_takes_nearly_everything(dtype):
    """Sinks of +6 against scores near zero: the sink has most of the weight and no value, so the result is small; left
    out, or counted once per key or per split, it would not be."""
    rot = {"dims": 8, "base": 100.0}
    spec = _latent_spec(4, 32, 8, 32, 48, rot, 64, scale=0.05)
    w = _weights(spec, seed=9, std=0.1)
    w["m.sink"] = torch.tensor([6.0, 5.0, 7.0, -2.0]).bfloat16()
    x = torch.randn(150, 64, generator=torch.Generator().manual_seed(12)).bfloat16()
    m = _m(4, 32, 8, 32, 48, rot, scale=0.05)
    want = _latent_plain(x, w, m)
    none = _latent_plain(x, {**w, "m.sink": torch.full((4,), -60.0)}, m)
    assert _rel(want, none) > 0.3
    got = _run_mixer(spec, w, x, dtype, portions=((70, 3), (40, 1), (38, 2), (1, 1), (1, 1)))
    assert _rel(got, want) < MIX_TOL[dtype]


# ------------------------------------------------------------------------ time mixing
def _wkv_spec(heads, dim, rank, hidden, eps=1e-6):
    from ember_b200.config import TimeMixSpec
    return TimeMixSpec(hidden_size=hidden, num_heads=heads, head_dim=dim, decay_rank=rank, norm_eps=eps)


def _wkv_plain(x, w, heads, dim, eps=1e-6):
    return plain.wkv(x.double(), {k: v.double() for k, v in w.items()}, "m.", {"heads": heads, "dim": dim}, eps)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rank,hidden", [(3, 24, 8, 64), (1, 40, 5, 100), (2, 128, 16, 128), (1, 288, 32, 72), (6, 12, 3, 64),
                                                   (5, 4, 2, 64)])
def test_time_mixing_alone(dtype, heads, dim, rank, hidden):
    """The blends with the previous token's input, the decay's two exponentials, the read-out before the update and
    the bonus, the per-head unit norm and the gate, in portions beside another request (the previous input and the
    state come from the request's slot at every portion's start); heads of four channels, and of 288 channels, which the
    register-resident scan does not take."""
    spec = _wkv_spec(heads, dim, rank, hidden)
    w = _weights(spec, seed=heads, std=0.12)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(2)).bfloat16()
    assert _rel(_run_mixer(spec, w, x, dtype), _wkv_plain(x, w, heads, dim)) < MIX_TOL[dtype]


def test_a_blend_that_reads_the_previous_token_alone():
    """mu = 1 everywhere: every projection reads the previous token's input and nothing of its own, so a request's
    first token reads zeros and a portion's first token reads what the portion before it left in the slot."""
    spec = _wkv_spec(2, 16, 4, 64)
    w = _weights(spec, seed=3, std=0.12)
    for b in "rkvgw":
        w["m.mu." + b] = torch.ones(64).bfloat16()
    x = torch.randn(90, 64, generator=torch.Generator().manual_seed(5)).bfloat16()
    want = _wkv_plain(x, w, 2, 16)
    moved = x.clone()
    moved[89] = 0                                            # the last token's own input does not reach its result
    assert _rel(_wkv_plain(moved, w, 2, 16)[89], want[89]) < 1e-9
    got = _run_mixer(spec, w, x, torch.float32, portions=((1, 1), (1, 1), (2, 1), (40, 7), (3, 1), (1, 1), (42, 19)))
    assert _rel(got, want) < MIX_TOL[torch.float32]
    assert float(got[0].abs().max()) < 1e-6                  # zeros in, zero keys and values, zero read-out


def test_the_recurrence_forgets_at_the_rate_of_its_decay_and_the_bonus_reaches_the_current_token_alone():
    """Decay biases so high that w is about 0.07 a token: a token twenty back no longer counts, the last few do.  A large
    bonus: the current token's own key and value dominate its read-out, and no later token's."""
    heads, dim = 2, 16
    spec = _wkv_spec(heads, dim, 4, 64)
    w = _weights(spec, seed=5, std=0.1)
    w["m.w0"] = torch.full((heads * dim,), 1.0).bfloat16()
    x = torch.randn(90, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    want = _wkv_plain(x, w, heads, dim)
    far, near = x.clone(), x.clone()
    far[60] = 0
    near[86] = 0
    assert _rel(_wkv_plain(far, w, heads, dim)[89], want[89]) < 1e-6
    assert _rel(_wkv_plain(near, w, heads, dim)[89], want[89]) > 1e-2
    assert _rel(_run_mixer(spec, w, x, torch.float32), want) < MIX_TOL[torch.float32]
    slow = dict(w)
    slow["m.w0"] = torch.full((heads * dim,), -6.0).bfloat16()          # w about 0.9975: the state keeps everything
    slow["m.u"] = torch.full((heads, dim), 8.0).bfloat16()
    want = _wkv_plain(x, slow, heads, dim)
    assert _rel(_wkv_plain(x, {**slow, "m.u": torch.zeros(heads, dim)}, heads, dim), want) > 0.2
    assert _rel(_run_mixer(spec, slow, x, torch.float32), want) < MIX_TOL[torch.float32]


# ------------------------------------------------------------------------ feed-forwards
def _expert_weights(hidden, ff, experts, seed):
    g = torch.Generator().manual_seed(seed)
    w = {"f.router": (0.5 * torch.randn(experts, hidden, generator=g)).bfloat16(),
         "f.correction": (0.3 * torch.randn(experts, generator=g)).bfloat16()}
    for e in range(experts):
        w[f"f.e{e}.gate"] = (0.3 * torch.randn(ff, hidden, generator=g)).bfloat16()
        w[f"f.e{e}.up"] = (0.3 * torch.randn(ff, hidden, generator=g)).bfloat16()
        w[f"f.e{e}.down"] = (0.04 * torch.randn(hidden, ff, generator=g)).bfloat16()
    return w


def _routed_spec(hidden, ff, experts, top, scale):
    from ember_b200.config import RoutedMLPSpec
    return RoutedMLPSpec(hidden_size=hidden, intermediate_size=ff, experts=experts, top=top, limit=0.0, alpha=1.0, up_offset=0.0,
                         scoring="sigmoid", correction=True, route_scale=scale, renormalize=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,ff,experts,top,scale", [(64, 40, 5, 2, 1.5), (100, 30, 6, 1, 2.0), (96, 24, 3, 3, 0.7), (128, 256, 40, 4, 2.5),
                                                         (64, 50, 2, 2, 1.0)])
def test_routed_feed_forward_alone(dtype, hidden, ff, experts, top, scale):
    """Sigmoid scores, one choice, as many choices as experts, more experts than a warp has lanes; silu experts without
    clamps; weights that are the chosen scores times a constant and do not sum to one."""
    w = _expert_weights(hidden, ff, experts, seed=experts)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(4)).bfloat16()
    mlp = {"router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}
    want = plain.routed_ff(x.double(), {k: v.double() for k, v in w.items()}, "f.", mlp)
    got, _, _ = _run_feed_forward(_routed_spec(hidden, ff, experts, top, scale), w, x, dtype)
    assert _rel(got, want) < MIX_TOL[dtype]


def test_the_correction_moves_the_choice_and_not_the_weights():
    """A correction of +2 on an expert whose scores are near zero: every token chooses it first all the same, and it
    weighs next to nothing; a correction of -2 keeps the expert whose scores are near one out."""
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    T, E, top, K = 200, 9, 3, 72
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, K, generator=g)
    w = 0.2 * torch.randn(E, K, generator=g)
    corr = 0.05 * torch.randn(E, generator=g)
    x[:, 0], w[:, 0] = 1.0, 0.0
    w[2, 0], w[6, 0] = -12.0, 12.0                             # expert 2 scores near 0, expert 6 near 1
    corr[2], corr[6] = 2.0, -2.0
    sel = torch.zeros(T * top, dtype=torch.int32, device=dev)
    wgt = torch.zeros(T * top, dtype=torch.float32, device=dev)
    ops.moe_router(x.to(dev), w.to(dev), T, top, sel, wgt, rule=(corr.to(dev), 1.5, False))
    s = torch.sigmoid(x.double() @ w.double().T)
    _, idx = torch.sort(s + corr.double(), dim=-1, descending=True, stable=True)
    assert sel.view(T, top).cpu().tolist() == idx[:, :top].tolist()
    assert bool((sel.view(T, top)[:, 0] == 2).all()) and not bool((sel == 6).any())
    assert torch.allclose(wgt.view(T, top).cpu().double(), 1.5 * torch.gather(s, 1, idx[:, :top]), atol=1e-6)
    assert float(wgt.view(T, top)[:, 0].max()) < 0.2
    # renormalised weights (another design's rule through the same kernel) sum to the scale
    ops.moe_router(x.to(dev), w.to(dev), T, top, sel, wgt, rule=(corr.to(dev), 1.5, True))
    assert torch.allclose(wgt.view(T, top).sum(-1).cpu(), torch.full((T,), 1.5), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,ff", [(64, 40), (100, 36), (128, 512)])
def test_dense_feed_forward_with_the_tanh_form_of_gelu(dtype, hidden, ff):
    from ember_b200.config import GatedMLPSpec
    g = torch.Generator().manual_seed(ff)
    w = {"f.gate": (0.4 * torch.randn(ff, hidden, generator=g)).bfloat16(), "f.up": (0.3 * torch.randn(ff, hidden, generator=g)).bfloat16(),
         "f.down": (0.02 * torch.randn(hidden, ff, generator=g)).bfloat16()}
    x = (1.5 * torch.randn(90, hidden, generator=torch.Generator().manual_seed(4))).bfloat16()      # gate values on both tails
    want = plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}, "f.")
    spec = GatedMLPSpec(hidden_size=hidden, intermediate_size=ff, activation="gelu_tanh", names=("gate", "up", "down"))
    got, _, _ = _run_feed_forward(spec, w, x, dtype)
    assert _rel(got, want) < MIX_TOL[dtype]
    silu_want = plain.lin(plain.silu(plain.lin(x.double(), w["f.gate"].double())) * plain.lin(x.double(), w["f.up"].double()), w["f.down"].double())
    assert _rel(silu_want, want) > 5e-3                   # (the float32 bound is 2e-5: the other activation would show)


# ------------------------------------------------------------------------ norm and copies of the residual stream
@pytest.mark.parametrize("streams,width", [(1, 64), (2, 100), (3, 96), (5, 33), (16, 8)])
def test_copies_of_the_stream_are_read_and_written_like_the_equations(streams, width):
    """u = sum_s in[s] x_s through tanh(alpha u) w + b; every copy at once from the old ones with a mix matrix that is
    not symmetric (indexed [from, to]), the result scaled by a vector, a multiplier and out[to]."""
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    T = 70
    g = torch.Generator().manual_seed(streams)
    X = torch.randn(T, streams, width, generator=g)
    in_w, out_w, mix = torch.rand(streams, generator=g) + 0.2, torch.rand(streams, generator=g) + 0.5, torch.randn(streams, streams, generator=g)
    alpha, nw, nb = torch.tensor([0.7]), 1 + 0.1 * torch.randn(width, generator=g), 0.1 * torch.randn(width, generator=g)
    scale, y = torch.randn(width, generator=g), torch.randn(T, width, generator=g)
    u = torch.einsum("s,tsw->tw", in_w.double(), X.double())
    want_read = torch.tanh(0.7 * u) * nw.double() + nb.double()
    want_X = torch.einsum("sr,tsw->trw", mix.double(), X.double()) + 0.6 * out_w.double()[None, :, None] * (scale.double() * y.double())[:, None, :]
    d = lambda t: t.to(dev).contiguous()          # noqa: E731
    Xd = d(X.view(T, streams * width))
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        out = torch.zeros(T + 3, width, device=dev, dtype=dtype)
        ops.stream_read(Xd, streams, d(in_w), out, T, norm=(d(alpha), d(nw), d(nb)))
        assert _rel(out[:T].cpu(), want_read) < tol and float(out[T:].float().abs().max()) == 0.0
    # rows off a 16-byte boundary take the kernels' one-element form: the same bits as the four-element form
    shifted = torch.zeros(T * streams * width + 1, device=dev)[1:].view(T, streams * width)
    shifted.copy_(Xd)
    a, b = torch.zeros(T, width, device=dev), torch.zeros(T, width, device=dev)
    ops.stream_read(Xd, streams, d(in_w), a, T, norm=(d(alpha), d(nw), d(nb)))
    ops.stream_read(shifted, streams, d(in_w), b, T, norm=(d(alpha), d(nw), d(nb)))
    assert torch.equal(a, b)
    ops.stream_write(shifted, streams, d(mix), d(out_w), d(scale), 0.6, d(y), T)
    plain_sum = torch.zeros(T, width, device=dev)
    ops.stream_read(Xd, streams, d(in_w), plain_sum, T)
    assert _rel(plain_sum.cpu(), u) < 1e-6
    ops.stream_write(Xd, streams, d(mix), d(out_w), d(scale), 0.6, d(y), T)
    assert _rel(Xd.cpu().view(T, streams, width), want_X) < 1e-6
    assert torch.equal(Xd, shifted)
    if streams > 1:
        wrong = torch.einsum("rs,tsw->trw", mix.double(), X.double()) + (want_X - torch.einsum("sr,tsw->trw", mix.double(), X.double()))
        assert _rel(wrong, want_X) > 0.1
    # without learned tensors: the plain residual sum on every copy
    Xe = d(X.view(T, streams * width))
    ops.stream_write(Xe, streams, None, None, None, 0.5, d(y), T)
    assert _rel(Xe.cpu().view(T, streams, width), X.double() + 0.5 * y.double()[:, None, :]) < 1e-6
    total = torch.zeros(T, width, device=dev)
    ops.stream_sum(Xe, streams, total, T)
    assert _rel(total.cpu(), (X.double() + 0.5 * y.double()[:, None, :]).sum(1)) < 1e-6


def test_dynamic_tanh_saturates_and_takes_rows():
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(2)
    x = 30.0 * torch.randn(50, 100, generator=g)
    x[0, :4] = torch.tensor([0.0, 1e-4, -200.0, 200.0])
    w, b, alpha = torch.randn(100, generator=g), torch.randn(100, generator=g), torch.tensor([0.9])
    rows = torch.tensor([49, 0, 7, 7], dtype=torch.int32)
    want = torch.tanh(0.9 * x.double()) * w.double() + b.double()
    out = torch.zeros(50, 100, device=dev)
    ops.dynamic_tanh(x.to(dev), alpha.to(dev), w.to(dev), b.to(dev), out, 50)
    assert float((out.cpu().double() - want).abs().max()) < 1e-5
    picked = torch.zeros(4, 100, device=dev)
    ops.dynamic_tanh(x.to(dev), alpha.to(dev), w.to(dev), b.to(dev), picked, 4, rows=rows.to(dev))
    assert float((picked.cpu().double() - want[rows.long()]).abs().max()) < 1e-5


@pytest.mark.parametrize("n", [1, 7, 4096, 4099, 3 * 257])
def test_logits_are_scaled_then_capped(n):
    """cap tanh(scale z / cap) over counts that are and are not a multiple of four (the two forms of the kernel agree to
    the bit: a logit does not depend on how many rows the step asked for), far beyond the cap, and without a cap."""
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    z = 40.0 * torch.randn(n + 5, generator=torch.Generator().manual_seed(n))
    z[0] = 1e4
    for scale, cap in ((1.7, 9.0), (0.25, 30.0), (3.0, 0.0)):
        buf = z.to(dev)
        ops.logit_finish(buf, n, scale, cap)
        want = cap * torch.tanh(scale * z[:n].double() / cap) if cap else scale * z[:n].double()
        assert float((buf[:n].cpu().double() - want).abs().max()) < 2e-6 * max(cap, 1.0) + (1e-5 * float(z.abs().max()) if not cap else 0.0)
        assert torch.equal(buf[n:].cpu(), z[n:])                      # nothing behind the count is touched
        if n >= 4:
            odd = z.to(dev)[1:]                                       # a start that is not on a 16-byte boundary
            ops.logit_finish(odd, n - 1, scale, cap)
            assert torch.equal(odd[:n - 1].cpu(), buf[1:n].cpu())


# ------------------------------------------------------------------------ through the programs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, dirs, plain_logits, tmp_path):
    """bin/trace_run as a user runs it (config.json without the low-rank size, four state slots, steps on standard
    input): portions beside single tokens of up to four live requests, and a step larger than any one batch."""
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    requests = make_requests("p", (300, 41, 75, 2, 33, 64), seed=9)
    steps = trace_mixed(requests, live=4, seed=1, max_portion=70)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs["p"], "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = FOMANEX["p"]["json"]["vocab"]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    assert_close(collect(steps, outputs), plain_logits("p", requests), dtype, "trace_run")


# ------------------------------------------------------------------------ through the entry point
@pytest.mark.parametrize("name", ["p", "s"])
def test_greedy_generation_through_the_engine(name, dirs):
    """Greedy tokens from ``ember_b200.load(...).generate`` (scheduler, portions of 16, few pages, four prompts of
    unequal length, three slots) against greedy decoding with the plain implementation."""
    import ember_b200
    cfg, W = plain_inputs(dirs[name])
    prompts = list(make_requests(name, (5, 40, 1, 23), seed=31).values())
    llm = ember_b200.load(dirs[name], dtype="float32", kv_cache_tokens=256, max_batch_tokens=64, max_seqs=3, prefill_chunk=16,
                          page_tokens=16)
    got = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for p, ids in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            seq.append(int(plain.forward(cfg, W, seq)[-1].argmax()))
        assert list(ids) == seq[len(p):]
    assert llm.runner.cache.check() == ""
