"""Zufusun on the device against the plain implementation: each mechanism alone (fed in portions beside another
request), keys just inside and just outside a window and the kept first tokens, a sink that takes nearly everything,
a far key that dominates, the router's choices, whole models under every way of cutting the work, slots and pages
used again, long decoding through captured graphs, and greedy generation through the entry point and its scheduler."""
import json
import os

import numpy as np
import pytest
import torch

from tests.plain import zufusun_plain as plain
from tests.replay_helpers import (collect, max_live_tokens, trace_mixed, trace_portions,
                                  trace_tail_decode, trace_whole)
from tests.zufusun_configs import ZUFUSUN, plain_inputs, write_zufusun_dir

pytestmark = pytest.mark.gpu

# A position's error is norm(got - want) / norm(want) over its logits.  Every sublayer's result passes an RMS norm
# before it joins the stream, so a rounding error keeps its size relative to the sublayer's own result however small
# that is, and a router's close call falls the other way under the smallest change: at most positions of a random
# model the error is that of the arithmetic (1e-6 in float32, 1e-2 in bfloat16), at a few it is many times larger,
# in every way of cutting the work alike.  A fault of a mechanism (a key too many, a lost state, a sink left out) is
# 1e-2 or more in float32 at every position it touches.
TOL = {"float32": dict(median=5e-6, worst=2e-4, over=0.0), "bfloat16": dict(median=3e-2, worst=None, over=0.06, above=0.12)}


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
    return {name: write_zufusun_dir(name, str(tmp_path_factory.mktemp("zufusun_" + name))) for name in ZUFUSUN}


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
    return {f"r{i}": rng.integers(0, ZUFUSUN[name]["json"]["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


def replay(model_dir, dtype, steps, capacity, page_tokens=16, max_requests=4, max_batch_tokens=512, **kw):
    import tempfile
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_dir(model_dir, dtype=dtype, capacity_tokens=capacity, max_batch_tokens=max_batch_tokens,
                                  max_requests=max_requests, page_tokens=page_tokens, **kw)
    with tempfile.TemporaryDirectory() as out:
        rp = TraceReplayer(runner, out)
        outputs = {}
        for s in steps:
            got = rp.run_step(s)
            if got is not None:
                outputs[s["step"]] = got.copy()
            assert runner.cache.check() == ""
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
    return outputs, runner


LENGTHS = {"u": (1, 2, 37, 130), "v": (3, 18, 65, 150), "w": (2, 70, 140)}


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ZUFUSUN))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes(name, dtype, mode, page, dirs, plain_logits):
    """Whole prompts, a decoded tail (the windows pass over decoded tokens), portions down to two tokens (and single
    ones), and four live requests whose slots and pages are used again, against each request alone in the plain
    implementation."""
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
    """300 tokens one by one (captured graphs after the second step; the router's grouping, the windows' page release
    and the key splits all inside them) against the whole sequence."""
    requests = make_requests("u", (300,), seed=11)
    steps = trace_tail_decode(requests, tail=299)
    outputs, runner = replay(dirs["u"], dtype, steps, 320)
    assert runner.graph_replays > 250
    assert_close(collect(steps, outputs), plain_logits("u", requests), dtype, "long decoding")
    eager, _ = replay(dirs["u"], dtype, steps, 320, cuda_graphs=False)
    assert max(float(np.abs(outputs[k] - eager[k]).max()) for k in outputs) < (1e-5 if dtype == "float32" else 1e-1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding(dtype, dirs, plain_logits):
    """1,300 tokens at a real model's head sizes: latent rows more than a thousand positions back, a window that has
    long left the first pages behind (the kept ones stay), a state that has seen as many tokens: as one prompt with
    a decoded tail and as portions of 500."""
    requests = make_requests("w", (1300,), seed=17)
    for steps in (trace_tail_decode(requests, tail=24), trace_portions(requests, sizes=(500, 37, 500, 2))):
        outputs, _ = replay(dirs["w"], dtype, steps, 1344, page_tokens=64, max_batch_tokens=2048)
        assert_close(collect(steps, outputs), plain_logits("w", requests), dtype, "long prompt")


def test_a_slot_used_again_starts_from_zero(dirs, plain_logits):
    """One slot only: the second request gets the state and the pages the first left."""
    requests = make_requests("v", (90, 75, 33), seed=21)
    steps = trace_portions(requests, sizes=(40, 3, 1, 31))
    outputs, _ = replay(dirs["v"], "float32", steps, 96, max_requests=1)
    assert_close(collect(steps, outputs), plain_logits("v", requests), "float32", "one slot")


def test_window_pages_go_back_while_a_request_runs(dirs):
    """The windowed layers' group holds the window's pages and the kept first tokens', not the whole request."""
    from ember_b200.engine.batch import StepEntry
    from ember_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_dir(dirs["u"], dtype="float32", capacity_tokens=512, max_batch_tokens=256, max_requests=2, page_tokens=16)
    toks = make_requests("u", (400,), seed=2)["r0"]
    runner.admit("a")
    for at in range(0, 400, 100):
        assert runner.reserve("a", 100)
        runner.step([StepEntry("a", toks[at:at + 100], ())])
    kinds = [(g.need.kind, g.need.window, g.need.keep_first) for g in runner.cache.groups]
    used = dict(zip(kinds, runner.cache.used_pages()))
    assert used[("window", 20, 3)] == 1 + 2           # the page of the three kept tokens, and the window's last two
    assert used[("window", 33, 0)] == 2
    assert used[("full", 0, 0)] == 25
    runner.release("a")


# ------------------------------------------------------------------------------ each mechanism alone
from tests.test_fadosun_gpu import _rel, _run_mixer, _weights      # noqa: E402  (the bench that feeds a mixer in portions)

MIX_TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _sink_spec(heads, kv, dim, vdim, window, keep, hidden, scale=0.2, bias=True, norm="whole"):
    from ember_b200.config import SinkAttentionSpec
    return SinkAttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=dim, value_dim=vdim, scale=scale,
                             bias=bias, qk_norm=norm, qk_norm_eps=1e-6, window=window, keep_first=keep, sink=True)


def _sink_m(heads, kv, dim, vdim, window, keep, scale=0.2):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    return m


@pytest.fixture(params=[1, 1 << 30], ids=["tensor-core attention", "general attention"])
def attention_kernel(request, monkeypatch):
    """bfloat16 steps take the tensor-core attention where the sizes allow; the second run keeps them on the general one."""
    from ember_b200.parts.sink_attention import _SinkSoftmax
    monkeypatch.setattr(_SinkSoftmax, "TC_MIN_TOKENS", request.param)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,window,keep,hidden", [(6, 2, 16, 24, 20, 3, 64), (4, 1, 20, 12, 7, 9, 100),
                                                                  (2, 2, 128, 128, 64, 1, 128), (3, 3, 18, 300, 1, 0, 72),
                                                                  (40, 1, 8, 8, 16, 16, 64), (2, 1, 32, 32, 0, 0, 64)])
def test_sink_attention_alone(dtype, heads, kv, dim, vdim, window, keep, hidden, attention_kernel):
    """Biases, the norm over the whole projections, windows of one key up to none at all, more kept tokens than the
    window is long, values wider and narrower than keys, forty query heads on one key head."""
    spec = _sink_spec(heads, kv, dim, vdim, window, keep, hidden)
    w = _weights(spec, seed=heads)
    for n in "qkv":
        w[f"m.{n}.b"] = (0.3 * torch.randn(w[f"m.{n}.b"].shape, generator=torch.Generator().manual_seed(7))).bfloat16()
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    want = plain.windowed_sink_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", _sink_m(heads, kv, dim, vdim, window, keep), 1e-6)
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


@pytest.mark.parametrize("heads,kv,dim,vdim,window,keep,hidden", [(4, 2, 128, 128, 64, 4, 128), (6, 2, 16, 32, 20, 3, 64),
                                                                  (3, 1, 48, 16, 33, 40, 72), (40, 1, 16, 16, 7, 0, 64)])
def test_sink_attention_on_tensor_cores(heads, kv, dim, vdim, window, keep, hidden):
    """bfloat16 portions of 65 tokens and more of the windowed layers (head sizes that are multiples of 16): keys and
    values from pools of their own, windows whose edges fall inside 32-key tiles, kept first tokens."""
    spec = _sink_spec(heads, kv, dim, vdim, window, keep, hidden)
    w = _weights(spec, seed=heads)
    x = torch.randn(200, hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    want = plain.windowed_sink_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", _sink_m(heads, kv, dim, vdim, window, keep), 1e-6)
    got = _run_mixer(spec, w, x, torch.bfloat16, portions=((100, 3), (30, 40), (68, 1), (1, 1), (1, 1)))
    assert _rel(got, want) < MIX_TOL[torch.bfloat16]


@pytest.mark.parametrize("kind", ["latent", "windowed", "whole"])
def test_tensor_core_attention_with_key_splits(kind, monkeypatch):
    """Small bfloat16 steps through the tensor-core kernel with their key ranges cut into splits of 32 keys that a
    second kernel merges (the sink joins there): latent rows, a windowed layer whose early splits are empty but for the
    kept tokens, and a layer that sees everything."""
    from ember_b200.parts.sink_attention import _SinkSoftmax
    monkeypatch.setattr(_SinkSoftmax, "TC_MIN_TOKENS", 1)
    monkeypatch.setattr(_SinkSoftmax, "SPLIT_KEYS", 32)
    x = torch.randn(200, 64, generator=torch.Generator().manual_seed(5)).bfloat16()
    portions = ((150, 3), (20, 10), (28, 1), (1, 1), (1, 1))
    if kind == "latent":
        spec = _latent_spec(4, 16, 16, 16, 32, 48, 16, 1e4, 64)
        w = _weights(spec, seed=4, std=0.12)
        want = _latent_plain(x, w, {"heads": 4, "dim": 16, "rot_dim": 16, "vdim": 16, "q_rank": 32, "kv_rank": 48, "scale": 0.2,
                                    "rot": {"dims": 16, "base": 1e4}})
    else:
        window, keep = (40, 5) if kind == "windowed" else (0, 0)
        spec = _sink_spec(4, 2, 32, 16, window, keep, 64)
        w = _weights(spec, seed=4)
        want = plain.windowed_sink_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", _sink_m(4, 2, 32, 16, window, keep), 1e-6)
    assert _rel(_run_mixer(spec, w, x, torch.bfloat16, portions=portions), want) < MIX_TOL[torch.bfloat16]


def _one_hot_attention(window, keep, hidden=64, dim=32, vdim=48, heads=2):
    """A layer whose queries copy the first half of the input and whose keys copy the second (zero biases, norm
    weights of one) and whose sink is far below every score, so that a key that points one way takes a query's
    weight if and only if it is visible."""
    spec = _sink_spec(heads, 1, dim, vdim, window, keep, hidden, scale=1.5)
    w = _weights(spec, seed=3, std=0.05)
    for n in ("q.b", "k.b", "v.b"):
        w["m." + n] = torch.zeros_like(w["m." + n])
    for n in ("q.norm", "k.norm"):
        w["m." + n] = torch.ones_like(w["m." + n])
    eye_q, eye_k = torch.zeros(dim, hidden), torch.zeros(dim, hidden)
    eye_q[:, :dim] = torch.eye(dim)
    eye_k[:, dim:2 * dim] = torch.eye(dim)
    w["m.q"], w["m.k"] = torch.cat([eye_q] * heads).bfloat16(), eye_k.bfloat16()
    w["m.sink"] = torch.full((heads,), -30.0).bfloat16()
    return spec, w


@pytest.mark.parametrize("portions", [((200, 3),), ((120, 3), (30, 30), (48, 1), (1, 1), (1, 1)),
                                      ((2, 1),) + ((1, 1),) * 60 + ((138, 2),)])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_tokens(portions):
    """Keys scaled so that each would take a late query's whole weight, placed at the last kept position, the first
    position that is not kept, just outside and just inside the window: the read-out equals the plain implementation's,
    and that one changes by much exactly when a visible one of those keys is taken out.  Run as one prompt, as
    portions with single tokens at the end, and with the first tokens decoded one by one."""
    window, keep, hidden, dim, T = 50, 4, 64, 32, 200
    spec, w = _one_hot_attention(window, keep)
    x = 0.1 * torch.randn(T, hidden, generator=torch.Generator().manual_seed(6))
    query = 199
    spots = {"kept": keep - 1, "not kept": keep, "outside": query - window, "inside": query - window + 1}
    for i, t in enumerate(spots.values()):
        x[t, dim:] = 0.0
        x[t, dim + i] = 4.0                                 # each marked key points its own way
    x[query, :dim] = 0.0
    x[query, :4] = 4.0                                      # after the norms the query scores 24 on each of them
    x = x.bfloat16()
    W = {k: v.double() for k, v in w.items()}
    m = _sink_m(2, 1, dim, 48, window, keep, scale=1.5)
    want = plain.windowed_sink_attention(x.double(), W, "m.", m, 1e-6)
    for name, t in spots.items():
        gone = x.clone()
        gone[t] = 0
        change = _rel(plain.windowed_sink_attention(gone.double(), W, "m.", m, 1e-6)[query], want[query])
        assert (change > 0.2) == (name in ("kept", "inside")), (name, change)
    got = _run_mixer(spec, w, x, torch.float32, portions=portions)
    assert _rel(got[query], want[query]) < 1e-4
    assert _rel(got, want) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_sink_that_takes_nearly_everything(dtype):
    """Sinks of +6 against scores near zero: the sink has most of the weight and no value, so the mixer's result is
    a small fraction of what it is without the sink; a kernel that forgot the sink would be off by that factor."""
    spec = _sink_spec(4, 2, 32, 32, 0, 0, 64, scale=0.05)
    w = _weights(spec, seed=9)
    w["m.sink"] = torch.tensor([6.0, -6.0, 5.0, 0.0]).bfloat16()
    x = torch.randn(90, 64, generator=torch.Generator().manual_seed(5)).bfloat16()
    W = {k: v.double() for k, v in w.items()}
    want = plain.windowed_sink_attention(x.double(), W, "m.", _sink_m(4, 2, 32, 32, 0, 0, 0.05), 1e-6)
    none = plain.windowed_sink_attention(x.double(), {**W, "m.sink": torch.full((4,), -60.0, dtype=torch.float64)}, "m.",
                                         _sink_m(4, 2, 32, 32, 0, 0, 0.05), 1e-6)
    assert _rel(want, none) > 0.3
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


def _latent_spec(heads, dim, rot_dim, vdim, q_rank, kv_rank, dims, base, hidden, own=True, scale=0.2):
    from ember_b200.config import LatentAttentionSpec, NoPositionSpec, RotarySpec
    pos = RotarySpec(head_dim=rot_dim, rotary_dim=dims, theta=base, frequency_precision="float64", layout="interleaved") if rot_dim else NoPositionSpec()
    return LatentAttentionSpec(hidden_size=hidden, num_heads=heads, head_dim=dim, rot_dim=rot_dim, value_dim=vdim, q_rank=q_rank,
                               kv_rank=kv_rank, scale=scale, norm_eps=1e-6, sink=True, gate=True, own_kv=own, position=pos)


def _latent_plain(x, w, m):
    W = {k: v.double() for k, v in w.items()}
    c, kr = plain.latent_kv(x.double(), W, "m.", m, 1e-6)
    return plain.latent_attention(x.double(), W, "m.", m, 1e-6, c, kr)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rot_dim,vdim,q_rank,kv_rank,dims,base,hidden", [
    (3, 24, 8, 20, 48, 40, 8, 1e4, 64), (2, 32, 16, 48, 24, 72, 8, 500.0, 100), (40, 8, 4, 6, 16, 20, 4, 77.0, 64),
    (4, 128, 64, 128, 192, 256, 64, 1e6, 128), (1, 16, 2, 16, 8, 512, 2, 10.0, 72)])
def test_latent_attention_alone(dtype, heads, dim, rot_dim, vdim, q_rank, kv_rank, dims, base, hidden, attention_kernel):
    """The cached latent with the up-projections folded around the attention against keys and values built per head:
    a rotation over a part of the rotated part, forty heads on one latent, the widest latent, a single head."""
    spec = _latent_spec(heads, dim, rot_dim, vdim, q_rank, kv_rank, dims, base, hidden)
    w = _weights(spec, seed=heads, std=0.12)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(8)).bfloat16()
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": 0.2,
         "rot": {"dims": dims, "base": base}}
    assert _rel(_run_mixer(spec, w, x, dtype), _latent_plain(x, w, m)) < MIX_TOL[dtype]


@pytest.mark.parametrize("heads,dim,rot_dim,vdim,q_rank,kv_rank,dims,base,hidden", [
    (4, 128, 64, 128, 192, 256, 64, 1e6, 128), (16, 16, 16, 16, 32, 48, 16, 1e4, 64), (40, 8, 16, 8, 16, 32, 8, 77.0, 64),
    (3, 24, 16, 20, 48, 64, 16, 500.0, 72)])
def test_latent_attention_on_tensor_cores(heads, dim, rot_dim, vdim, q_rank, kv_rank, dims, base, hidden):
    """bfloat16 portions of 65 tokens and more take the tensor-core kernel (rows and latents that are multiples of 16):
    tiles of 64 (token, head) rows that are full, ragged (three heads: 63 rows) or one token of forty heads; a latent
    whose halves are no multiple of 16 columns; decoded tokens beside the portions and after them."""
    spec = _latent_spec(heads, dim, rot_dim, vdim, q_rank, kv_rank, dims, base, hidden)
    w = _weights(spec, seed=heads, std=0.12)
    x = torch.randn(200, hidden, generator=torch.Generator().manual_seed(8)).bfloat16()
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": 0.2,
         "rot": {"dims": dims, "base": base}}
    got = _run_mixer(spec, w, x, torch.bfloat16, portions=((100, 3), (30, 40), (68, 1), (1, 1), (1, 1)))
    assert _rel(got, _latent_plain(x, w, m)) < MIX_TOL[torch.bfloat16]


def test_a_far_rotated_key_that_dominates_is_seen_across_pages_and_portions():
    """Scores that rest on the rotated key part alone (the unrotated queries are zero): a far key whose rotated part
    is large, queries that match it only if both were turned by their own positions' angles."""
    heads, dim, rot_dim, vdim, hidden, T, far = 2, 8, 16, 24, 64, 200, 5
    spec = _latent_spec(heads, dim, rot_dim, vdim, 32, 24, 16, 30.0, hidden, scale=1.0)
    w = _weights(spec, seed=4, std=0.1)
    w["m.sink"] = torch.full((heads,), -30.0).bfloat16()
    uq = w["m.uq"].float().view(heads, dim + rot_dim, 32)
    uq[:, :dim] = 0.0                                        # no unrotated score
    w["m.uq"] = uq.reshape(-1, 32).bfloat16()
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(6))
    x[far] *= 6.0                                            # (the shared key part is not normed: it grows with the input)
    x = x.bfloat16()
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": 32, "kv_rank": 24, "scale": 1.0,
         "rot": {"dims": 16, "base": 30.0}}
    want = _latent_plain(x, w, m)
    unturned = _latent_plain(x, w, {**m, "rot": {"dims": 16, "base": 1e30}})        # (all angles but the first pair's vanish)
    assert _rel(unturned[150:], want[150:]) > 0.2
    got = _run_mixer(spec, w, x, torch.float32, portions=((120, 3), (40, 30), (38, 1), (1, 1), (1, 1)))
    assert _rel(got, want) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,tau,rank,hidden", [(3, 24, 40, 8.0, 8, 64), (1, 40, 72, 4.0, 5, 100), (2, 128, 128, 16.0, 16, 128),
                                                            (1, 288, 64, 16.0, 32, 72), (2, 16, 33, 1.0, 3, 64)])
def test_gated_linear_attention_alone(dtype, heads, dim, vdim, tau, rank, hidden):
    """The recurrence in portions beside another request (register-resident scan, and the general one from 288 key
    channels), tau = 1, a value size that is no multiple of a block of columns."""
    from ember_b200.config import GatedLinearAttentionSpec
    spec = GatedLinearAttentionSpec(hidden_size=hidden, num_heads=heads, head_dim=dim, value_dim=vdim, tau=tau, decay_rank=rank, norm_eps=1e-6)
    w = _weights(spec, seed=heads, std=0.12)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(2)).bfloat16()
    want = plain.gated_linear_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.",
                                        {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, 1e-6)
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


def test_the_recurrence_forgets_at_the_rate_of_its_decay():
    """Decay biases so low that alpha is about 0.35 a token (tau 1): a token twenty back no longer counts, the last
    few do; a state that was not decayed (or not carried) would show at once."""
    from ember_b200.config import GatedLinearAttentionSpec
    spec = GatedLinearAttentionSpec(hidden_size=64, num_heads=2, head_dim=16, value_dim=24, tau=1.0, decay_rank=4, norm_eps=1e-6)
    w = _weights(spec, seed=5, std=0.1)
    w["m.a2.b"] = torch.full((32,), -0.6).bfloat16()
    x = torch.randn(90, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    m = {"heads": 2, "dim": 16, "vdim": 24, "tau": 1.0}
    W = {k: v.double() for k, v in w.items()}
    want = plain.gated_linear_attention(x.double(), W, "m.", m, 1e-6)
    far, near = x.clone(), x.clone()
    far[60] = 0
    near[86] = 0
    assert _rel(plain.gated_linear_attention(far.double(), W, "m.", m, 1e-6)[89], want[89]) < 1e-6
    assert _rel(plain.gated_linear_attention(near.double(), W, "m.", m, 1e-6)[89], want[89]) > 1e-2
    assert _rel(_run_mixer(spec, w, x, torch.float32), want) < MIX_TOL[torch.float32]


def _run_feed_forward(spec, weights, x_all, dtype, portions=(40, 3, 1, 2, 44)):
    from ember_b200.parts import build_part
    from tests.test_parts_gpu import Bench, store_of
    part = build_part("feed_forward", spec, "f.")
    b = Bench({}, dtype, capacity=512)
    part.load(store_of(weights), b.rt)
    hidden = x_all.shape[1]
    got, at = torch.zeros(x_all.shape[0], hidden), 0
    for n in portions:
        ctx = b.ctx([("x", n)])
        x = torch.zeros(256, hidden, device=b.dev, dtype=dtype)
        x[:n] = x_all[at:at + n].to(dtype)
        out = torch.full((256, hidden), 7.0, device=b.dev)
        part.forward(ctx, x, out, accumulate=False)
        added = torch.ones(256, hidden, device=b.dev)
        part.forward(ctx, x, added, accumulate=True)
        assert float((added[:n] - 1.0 - out[:n]).abs().max()) < 1e-6 * (10.0 + float(out[:n].abs().max()))    # a few float32 roundings of the sum
        got[at:at + n] = out[:n].cpu()
        at += n
    return got, part, b


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,ff,experts,top,limit", [(64, 40, 5, 2, 1.5), (100, 30, 6, 1, 2.0), (96, 24, 3, 3, 0.3),
                                                         (128, 256, 40, 4, 7.0), (64, 50, 2, 2, 1.0)])
def test_routed_feed_forward_alone(dtype, hidden, ff, experts, top, limit):
    """One choice, as many choices as experts, more experts than a warp has lanes, a limit that clamps most values."""
    from ember_b200.config import RoutedMLPSpec
    spec = RoutedMLPSpec(hidden_size=hidden, intermediate_size=ff, experts=experts, top=top, limit=limit)
    g = torch.Generator().manual_seed(experts)
    w = {"f.router": (0.5 * torch.randn(experts, hidden, generator=g)).bfloat16()}
    for e in range(experts):
        w[f"f.e{e}.gate"] = (0.3 * torch.randn(ff, hidden, generator=g)).bfloat16()
        w[f"f.e{e}.up"] = (0.3 * torch.randn(ff, hidden, generator=g)).bfloat16()
        w[f"f.e{e}.down"] = (0.2 * torch.randn(hidden, ff, generator=g)).bfloat16()
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(4)).bfloat16()
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    want = plain.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, "f.", mlp)
    got, _, _ = _run_feed_forward(spec, w, x, dtype)
    assert _rel(got, want) < MIX_TOL[dtype]


def test_the_router_chooses_and_weighs_like_the_plain_implementation():
    """Choices in descending order of logit with ties to the lower index, weights over the chosen alone; and the
    grouping puts every (token, choice) pair into its expert's range once."""
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    T, E, top = 300, 37, 5
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(1))
    logits[7, 3] = logits[7, 20] = logits[7].max() + 1.0                  # a tie for the first place
    logits[8] = 0.25                                                     # all equal: the first `top` experts
    sel = torch.zeros(T * top, dtype=torch.int32, device=dev)
    wgt = torch.zeros(T * top, dtype=torch.float32, device=dev)
    ops.moe_route(logits.to(dev), T, top, sel, wgt)
    val, idx = torch.sort(logits.double(), dim=-1, descending=True, stable=True)
    assert sel.view(T, top).cpu().tolist() == idx[:, :top].tolist()
    assert torch.allclose(wgt.view(T, top).cpu().double(), torch.softmax(val[:, :top], -1), atol=1e-6)
    assert sel.view(T, top)[7, :2].tolist() == [3, 20] and sel.view(T, top)[8].tolist() == list(range(top))
    # the kernel that makes the logits itself (fp32 weights and sums) chooses the same way
    for xdt in (torch.float32, torch.bfloat16):
        x = torch.randn(T, 72, generator=torch.Generator().manual_seed(2)).to(xdt)
        w = torch.randn(E, 72, generator=torch.Generator().manual_seed(3))
        sel2, wgt2 = torch.zeros_like(sel), torch.zeros_like(wgt)
        lg = torch.zeros(T, E, device=dev)
        ops.moe_router(x.to(dev), w.to(dev), T, top, sel2, wgt2, logits=lg)
        assert torch.allclose(lg.cpu().double(), x.double() @ w.double().T, atol=1e-4)
        v2, i2 = torch.sort(lg.cpu().double(), dim=-1, descending=True, stable=True)
        assert sel2.view(T, top).cpu().tolist() == i2[:, :top].tolist()
        assert torch.allclose(wgt2.view(T, top).cpu().double(), torch.softmax(v2[:, :top], -1), atol=1e-6)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    pair_of_slot = torch.zeros(T * top, dtype=torch.int32, device=dev)
    slot_of_pair = torch.zeros(T * top, dtype=torch.int32, device=dev)
    tiles = torch.zeros(1 + 2 * ops.moe_max_tiles(T * top, E), dtype=torch.int32, device=dev)
    mt = ops.moe_group(sel, T * top, E, offsets, pair_of_slot, slot_of_pair, tiles)
    off, pos, sop, s = offsets.cpu(), pair_of_slot.cpu(), slot_of_pair.cpu(), sel.cpu()
    assert off[0] == 0 and off[E] == T * top and sorted(pos.tolist()) == list(range(T * top))
    for e in range(E):
        assert all(int(s[p]) == e for p in pos[off[e]:off[e + 1]].tolist())
    assert all(int(pos[sop[i]]) == i for i in range(T * top))
    n = int(tiles[0])
    te, tr = tiles[1:1 + n].cpu().tolist(), tiles[1 + mt:1 + mt + n].cpu().tolist()
    assert n == sum((int(off[e + 1] - off[e]) + ops.MOE_TILE_ROWS - 1) // ops.MOE_TILE_ROWS for e in range(E))
    assert all(off[e] <= r < off[e + 1] for e, r in zip(te, tr))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_gate_and_rounding_kernels(dtype):
    """The silu gate after the per-head norm, and the fused norm + add that also leaves the rounded stream."""
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(8)
    T, groups, V = 9, 3, 44
    o, gate = torch.randn(T, groups * V + 5, generator=g).to(dev), torch.randn(T, 7 + groups * V, generator=g).to(dev)
    w = (1 + 0.1 * torch.randn(V, generator=g)).to(dev)
    out = torch.empty(T, groups * V, device=dev, dtype=dtype)
    ops.group_norm_gate(o, 5, gate, 7, w, False, 1e-6, ops.GATE_SILU_AFTER, out, T, groups, V)
    v, z = o[:, 5:].cpu().double().view(T, groups, V), gate[:, 7:].cpu().double().view(T, groups, V)
    want = plain.rms_norm(v, w.cpu(), 1e-6) * z * torch.sigmoid(z)
    assert _rel(out.float().cpu().view(T, groups, V), want) < (5e-3 if dtype == torch.bfloat16 else 1e-6)
    H = 100
    x, y = torch.randn(11, H, generator=g).to(dev), torch.randn(11, H, generator=g).to(dev)
    wn = (1 + 0.1 * torch.randn(H, generator=g)).to(dev)
    res, rounded = x.clone(), torch.zeros(11, H, device=dev, dtype=torch.bfloat16)
    ops.gated_norm_add(y, None, wn, None, 1e-6, False, res, 11, rounded=rounded)
    want = x.cpu().double() + plain.rms_norm(y.cpu().double(), wn.cpu(), 1e-6)
    assert _rel(res.cpu(), want) < 1e-6 and torch.equal(rounded, res.bfloat16())
    again = torch.zeros_like(rounded)
    ops.round_rows(res, again, 11 * H)
    assert torch.equal(again, rounded)


# ------------------------------------------------------------------------ through the programs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, dirs, plain_logits, tmp_path):
    """bin/trace_run as a user runs it (config.json without the low-rank size, four state slots, steps on standard
    input): portions beside single tokens of up to four live requests, and a step larger than any one batch."""
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    requests = make_requests("v", (300, 41, 75, 2, 33, 64), seed=9)
    steps = trace_mixed(requests, live=4, seed=1, max_portion=70)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs["v"], "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = ZUFUSUN["v"]["json"]["vocab"]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    assert_close(collect(steps, outputs), plain_logits("v", requests), dtype, "trace_run")


# ------------------------------------------------------------------------ through the entry point
def test_greedy_generation_through_the_engine(dirs):
    """Greedy tokens from ``ember_b200.load(...).generate`` (scheduler, portions of 16, few pages, four prompts of
    unequal length) against greedy decoding with the plain implementation."""
    import ember_b200
    cfg, W = plain_inputs(dirs["u"])
    prompts = list(make_requests("u", (5, 40, 1, 23), seed=31).values())
    llm = ember_b200.load(dirs["u"], dtype="float32", kv_cache_tokens=256, max_batch_tokens=64, max_seqs=3, prefill_chunk=16,
                          page_tokens=16)
    got = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for p, ids in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            seq.append(int(plain.forward(cfg, W, seq)[-1].argmax()))
        assert list(ids) == seq[len(p):]
    assert llm.runner.cache.check() == ""
