"""Pepapel on the device against the plain implementation: each mechanism alone (fed in portions beside another
request), keys just inside and just outside a chunk in prompts and in decoding, a far key that dominates across pages,
a score cap that binds, a temperature that changes from one position to the next, convolution inputs carried from one
portion to the next, a delta rule that forgets at the rate of its decay, the router's groups and identity experts,
whole models under every way of cutting the work, slots and pages used again, long decoding through captured graphs,
and greedy generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

from tests.plain import pepapel_plain as plain
from tests.pepapel_configs import PEPAPEL, drawn_pepapel, plain_inputs, write_pepapel_dir
from tests.replay_helpers import (collect, max_live_tokens, trace_mixed, trace_portions,
                                  trace_tail_decode, trace_whole)
from tests.test_fadosun_gpu import _rel, _weights
from tests.test_zufusun_gpu import _run_feed_forward, attention_kernel, replay  # noqa: F401  (attention_kernel: a fixture)

pytestmark = pytest.mark.gpu

# A position's error is norm(got - want) / norm(want) over its logits.  Every sublayer's sum passes a layer norm, so
# rounding keeps its relative size from layer to layer (1e-6 in float32, 1e-2 in bfloat16) except where a router's
# close call falls the other way.  A fault of a mechanism (a key too many, a lost state, a gate or a bias left out, a
# chunk's edge one off) is 1e-2 or more in float32 at every position it touches.
TOL = {"float32": dict(median=5e-6, worst=3e-4), "bfloat16": dict(median=3e-2, worst=None, over=0.06, above=0.12)}
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
    return {name: write_pepapel_dir(name, str(tmp_path_factory.mktemp("pepapel_" + name))) for name in PEPAPEL}


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
    return {f"r{i}": rng.integers(0, PEPAPEL[name]["json"]["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


LENGTHS = {"a": (1, 2, 37, 130), "b": (3, 18, 65, 150), "c": (2, 70, 140)}


# ------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(PEPAPEL))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes(name, dtype, mode, page, dirs, plain_logits):
    """Whole prompts, a decoded tail (chunk edges and temperature steps pass under decoded tokens), portions down to
    two tokens (and single ones), and four live requests whose slots and pages are used again, against each request
    alone in the plain implementation."""
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
    """Layer orders, sizes, head counts, taps, chunks, groups and constants drawn from a seed: whole prompts, portions and a
    mixed batch in float32 (the sharper comparison), the mixed batch in bfloat16."""
    cfg = drawn_pepapel(seed)
    d = write_pepapel_dir(cfg, str(tmp_path), seed=seed)
    inputs = plain_inputs(d)
    rng = np.random.default_rng(100 + seed)
    requests = {f"r{i}": rng.integers(0, cfg["vocab"], size=n).tolist()
                for i, n in enumerate((1, 2, int(rng.integers(30, 90)), int(rng.integers(100, 200)), 47, 19))}
    want = {rid: plain.forward(*inputs, toks).numpy() for rid, toks in requests.items()}
    for dtype, modes in (("float32", ("whole", "portions", "mixed")), ("bfloat16", ("mixed",))):
        for mode in modes:
            steps = {"whole": trace_whole, "portions": lambda r: trace_portions(r, sizes=(7, 2, 19, 1, 3, 33, 2, 16, 5, 64)),
                     "mixed": lambda r: trace_mixed(r, live=4, seed=seed)}[mode](requests)
            page = (16, 64)[seed % 2]
            outputs, _ = replay(d, dtype, steps, max_live_tokens(steps, round_to=page), page_tokens=page)
            assert_close(collect(steps, outputs), want, dtype, f"drawn {seed} {mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_equals_the_prompt(dtype, dirs, plain_logits):
    """300 tokens one by one (captured graphs after the second step; the convolutions' carried rows, the delta rule's
    state, the router's grouping and the key splits all inside them) against the whole sequence."""
    requests = make_requests("a", (300,), seed=11)
    steps = trace_tail_decode(requests, tail=299)
    outputs, runner = replay(dirs["a"], dtype, steps, 320)
    assert runner.graph_replays > 250
    assert_close(collect(steps, outputs), plain_logits("a", requests), dtype, "long decoding")
    eager, _ = replay(dirs["a"], dtype, steps, 320, cuda_graphs=False)
    assert max(float(np.abs(outputs[k] - eager[k]).max()) for k in outputs) < (1e-5 if dtype == "float32" else 1e-1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding(dtype, dirs, plain_logits):
    """900 tokens at a real model's head sizes: keys nearly a thousand positions back under a temperature that has
    stepped three times, chunks of 256 and of 100 that end inside portions, a state that has seen as many tokens: as
    one prompt with a decoded tail and as portions of 400."""
    requests = make_requests("c", (900,), seed=17)
    for steps in (trace_tail_decode(requests, tail=24), trace_portions(requests, sizes=(400, 37, 400, 2))):
        outputs, _ = replay(dirs["c"], dtype, steps, 960, page_tokens=64, max_batch_tokens=1024)
        assert_close(collect(steps, outputs), plain_logits("c", requests), dtype, "long prompt")


@pytest.mark.parametrize("name", ["a", "b"])
def test_a_slot_used_again_starts_from_zero(name, dirs, plain_logits):
    """One slot only: the second request gets the matrices, the convolution inputs and the pages the first left."""
    requests = make_requests(name, (90, 75, 33), seed=21)
    steps = trace_portions(requests, sizes=(40, 3, 1, 31))
    outputs, _ = replay(dirs[name], "float32", steps, 96, max_requests=1)
    assert_close(collect(steps, outputs), plain_logits(name, requests), "float32", "one slot")


@pytest.mark.parametrize("name", ["a", "b"])
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


# ------------------------------------------------------------------------ the mechanisms, each alone
def _run_mixer(spec, weights, x_all, dtype, portions=((40, 7), (3, 1), (1, 1), (2, 2), (44, 19)), prefix="m."):
    """The mixer fed in portions next to another request's portions; returns its stored output [T, hidden].  A mixer
    with several caches (pages and a state, or two mixers' caches) gets them by its own names."""
    from ember_b200.parts import build_part
    from tests.test_parts_gpu import Bench, store_of
    part = build_part("mixer", spec, prefix)
    keys = list(part.cache_needs())
    ident = lambda k: (0, k) if k else 0                                      # noqa: E731
    b = Bench({ident(k): v for k, v in part.cache_needs().items()}, dtype, capacity=512)
    part.load(store_of(weights), b.rt)
    hidden = x_all.shape[1]
    other = torch.randn(64, hidden, generator=torch.Generator().manual_seed(1)).bfloat16()
    got, at, oat = torch.zeros(x_all.shape[0], hidden), 0, 0
    for n, m in portions:
        ctx = b.ctx([("x", n), ("o", m)], tile_sizes=getattr(part, "tile_requests", lambda: ())())
        x = torch.zeros(256, hidden, device=b.dev, dtype=dtype)
        x[:n] = x_all[at:at + n].to(dtype)
        x[n:n + m] = other[oat:oat + m].to(dtype)
        out = torch.full((256, hidden), 7.0, device=b.dev)
        cache = b.storage.layer(0) if keys == [""] else {k: b.storage.layer(ident(k)) for k in keys}
        part.forward(ctx, x, out, cache, accumulate=False)
        got[at:at + n] = out[:n].cpu()
        at, oat = at + n, oat + m
    assert at == x_all.shape[0] and int(b.err.item()) == 0
    return got


def _attention_spec(heads, kv, dim, vdim, hidden, scale=0.2, softcap=0.0, q_temp=None, eps=1e-6):
    from ember_b200.config import SinkAttentionSpec
    return SinkAttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=dim, value_dim=vdim, scale=scale,
                             qk_norm="head", qk_norm_eps=eps, sink=False, softcap=softcap,
                             q_temp_coef=q_temp[0] if q_temp else 0.0, q_temp_every=q_temp[1] if q_temp else 0)


def _attention_m(heads, kv, dim, vdim, scale=0.2, softcap=0.0, q_temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _plain_mixer(fn, x, w, m, eps=1e-6):
    return fn(x.double(), {k: v.double() for k, v in w.items()}, "m.", m, eps)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,hidden,softcap,q_temp", [
    (6, 2, 16, 24, 64, 4.0, (0.5, 8)), (4, 1, 20, 12, 100, 0.0, (2.0, 1)), (2, 2, 128, 128, 128, 30.0, None),
    (3, 3, 18, 300, 72, 1.0, (0.3, 33)), (40, 1, 8, 8, 64, 0.0, None), (4, 1, 64, 32, 64, 40.0, (0.7, 64))])
def test_attention_alone(dtype, heads, kv, dim, vdim, hidden, softcap, q_temp, attention_kernel):
    """A norm per head with one weight for all heads, no rotation, a temperature with periods of 1 to 64 positions, caps
    from one that flattens most scores to none, values wider and narrower than keys, forty query heads on one key head."""
    spec = _attention_spec(heads, kv, dim, vdim, hidden, 0.5, softcap, q_temp)
    w = _weights(spec, seed=heads)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(2)).bfloat16()
    want = _plain_mixer(plain.attention_mixer, x, w, _attention_m(heads, kv, dim, vdim, 0.5, softcap, q_temp))
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


@pytest.mark.parametrize("dense", [True, False], ids=["TMA-fed kernels", "shared-row kernels"])
@pytest.mark.parametrize("heads,kv,dim,softcap,q_temp", [(8, 1, 128, 25.0, (0.4, 30)), (4, 2, 64, 0.0, (1.0, 9)), (16, 1, 64, 3.0, None),
                                                         (2, 2, 128, 0.7, None)])
def test_plain_causal_layers_on_the_engines_dense_attention_kernels(dense, heads, kv, dim, softcap, q_temp, monkeypatch):
    """Keys and values of one size, 64 or 128, without window, chunk or gate: bfloat16 steps go to the kernels Qwen3's
    attention uses (tcgen05 for prompt portions of 128-wide heads, the TMA-fed kernel with key splits for single tokens),
    which take the cap as a parameter; switched off, the same layer runs on the shared-row kernels.  Portions of 130 and
    60 tokens, then single tokens beside another request."""
    from ember_b200.parts.sink_attention import SinkAttention
    monkeypatch.setattr(SinkAttention, "DENSE_KERNELS", dense)
    spec = _attention_spec(heads, kv, dim, dim, 128, 0.6, softcap, q_temp)
    w = _weights(spec, seed=heads)
    x = torch.randn(200, 128, generator=torch.Generator().manual_seed(2)).bfloat16()
    want = _plain_mixer(plain.attention_mixer, x, w, _attention_m(heads, kv, dim, dim, 0.6, softcap, q_temp))
    got = _run_mixer(spec, w, x, torch.bfloat16, portions=((130, 3), (60, 20), (1, 1), (1, 1), (1, 0 + 1), (7, 2)))
    assert _rel(got, want) < MIX_TOL[torch.bfloat16]


@pytest.mark.parametrize("dense", [True, False], ids=["TMA-fed kernels", "shared-row kernels"])
@pytest.mark.parametrize("heads,kv,dim,taps,chunk,rot", [(8, 1, 128, 4, 50, {"dims": 64, "base": 1e4, "scaling": {"factor": 4.0}}),
                                                        (4, 2, 64, 2, 64, {"dims": 64, "base": 500.0}),
                                                        (2, 2, 128, 3, 7, {"dims": 16, "base": 1e6}),
                                                        (4, 4, 64, 1, 300, {"dims": 32, "base": 1e4})])
def test_chunked_layers_on_the_engines_dense_attention_kernels(dense, heads, kv, dim, taps, chunk, rot, monkeypatch):
    """Left halves whose keys and values are one size, 64 or 128: the same kernels take the chunk as a second lower bound
    on the visible keys, the gate per head follows as a pass of its own.  Chunks that end inside a 130-token portion, at
    a key tile's edge (64), every seven positions, and never (300); then single tokens across an edge."""
    from ember_b200.parts.sink_attention import SinkAttention
    monkeypatch.setattr(SinkAttention, "DENSE_KERNELS", dense)
    spec = _left_spec(heads, kv, dim, dim, 128, taps, chunk, rot, scale=0.5)
    w = _weights(spec, seed=heads, std=0.15)
    x = torch.randn(200, 128, generator=torch.Generator().manual_seed(8)).bfloat16()
    want = _plain_mixer(plain.chunked_attention_mixer, x, w, _left_m(heads, kv, dim, dim, taps, chunk, rot, 0.5))
    got = _run_mixer(spec, w, x, torch.bfloat16, portions=((130, 3), (60, 20), (1, 1), (1, 1), (1, 1), (7, 2)))
    assert _rel(got, want) < MIX_TOL[torch.bfloat16]
    for t in (49, 50, 51, 63, 64, 65, 127, 128, 129, 130, 189, 190, 191, 192, 193, 199):
        assert _rel(got[t], want[t]) < 3 * MIX_TOL[torch.bfloat16], t


def test_the_cap_and_the_temperature_are_there():
    """Scores of about +-12 under a cap of 3: without the cap the softmax is nearly one-hot, with it nearly flat among the
    larger scores.  A temperature period of 50: positions 48 and 49 differ by the factor 1 + ln 2."""
    spec = _attention_spec(2, 1, 32, 32, 64, scale=2.0, softcap=3.0, q_temp=(1.0, 50))
    w = _weights(spec, seed=3, std=0.3)
    x = torch.randn(120, 64, generator=torch.Generator().manual_seed(4)).bfloat16()
    m = _attention_m(2, 1, 32, 32, 2.0, 3.0, (1.0, 50))
    want = _plain_mixer(plain.attention_mixer, x, w, m)
    assert _rel(_plain_mixer(plain.attention_mixer, x, w, {**m, "softcap": 0.0}), want) > 0.2
    no_temp = _plain_mixer(plain.attention_mixer, x, w, {k: v for k, v in m.items() if k != "q_temp"})
    assert _rel(no_temp[:49], want[:49]) < 1e-12 and _rel(no_temp[49:], want[49:]) > 1e-3
    for portions in (((120, 3),), ((47, 1), (1, 1), (1, 1), (1, 1), (2, 1), (68, 30))):
        assert _rel(_run_mixer(spec, w, x, torch.float32, portions=portions), want) < MIX_TOL[torch.float32]


def _left_spec(heads, kv, dim, vdim, hidden, taps, chunk, rot, scale=0.2, eps=1e-6):
    from ember_b200.config import NoPositionSpec, RotarySpec, SinkAttentionSpec
    pos = NoPositionSpec()
    if rot:
        pos = RotarySpec(head_dim=dim, rotary_dim=rot["dims"], theta=rot["base"], frequency_precision="float64", layout="half",
                         linear_factor=(rot.get("scaling") or {}).get("factor", 1.0))
    return SinkAttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=dim, value_dim=vdim, scale=scale,
                             qk_norm="whole", qk_norm_eps=eps, sink=False, conv_taps=taps, position=pos, chunk=chunk, head_gate=True)


def _left_m(heads, kv, dim, vdim, taps, chunk, rot, scale=0.2):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "conv": taps, "mask": {"size": chunk}, "rot": rot}


LEFT_CASES = [
    (4, 2, 16, 24, 64, 4, 20, {"dims": 16, "base": 1e4, "scaling": {"factor": 8.0}}),
    (3, 1, 20, 12, 100, 1, 16, {"dims": 8, "base": 77.0}),                               # one tap: nothing carried
    (2, 2, 128, 128, 128, 3, 64, {"dims": 64, "base": 1e6, "scaling": {"factor": 2.0}}),
    (6, 3, 32, 48, 72, 5, 7, {"dims": 2, "base": 10.0, "scaling": {"factor": 1.0}}),     # one pair turns, chunks of seven
    (1, 1, 48, 16, 64, 2, 1, {"dims": 48, "base": 500.0}),                               # chunks of one: every token sees itself alone
    (6, 2, 40, 56, 64, 3, 120, {"dims": 40, "base": 2e4, "scaling": {"factor": 3.0}}),   # a chunk longer than the sequence
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,hidden,taps,chunk,rot", LEFT_CASES)
def test_chunked_attention_alone(dtype, heads, kv, dim, vdim, hidden, taps, chunk, rot, attention_kernel):
    """Convolutions of one to five taps whose inputs are carried from portion to portion, the norm over the whole
    projections, whole and partial rotations under a linear scaling, chunks from one position to longer than the
    sequence, and the gate per head."""
    spec = _left_spec(heads, kv, dim, vdim, hidden, taps, chunk, rot, scale=0.5)
    w = _weights(spec, seed=heads, std=0.15)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(8)).bfloat16()
    want = _plain_mixer(plain.chunked_attention_mixer, x, w, _left_m(heads, kv, dim, vdim, taps, chunk, rot, 0.5))
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


@pytest.mark.parametrize("portions", [((150, 3),), ((40, 3), (1, 1), (1, 1), (1, 1), (37, 30), (2, 1), (68, 1)), ((38, 1),) + ((1, 1),) * 5 + ((35, 1),) + ((1, 1),) * 5 + ((35, 1),) + ((1, 1),) * 5 + ((27, 1),),
                                      ((39, 1), (1, 1), (40, 1), (40, 1), (30, 1))])
def test_keys_just_inside_and_just_outside_a_chunk(portions):
    """Chunks of 40 with pages of 16.  The query at 40 sees itself alone and the one at 79 sees 40 .. 79: with a chunk's
    edge one off, position 40 (or 39) would see one key more or fewer, which changes its result by a large part.  Checked
    row by row around every edge, in a prompt's portion, at a portion's first token and for single tokens."""
    heads, kv, dim, vdim, hidden, taps, chunk = 2, 1, 16, 16, 64, 1, 40
    rot = {"dims": 4, "base": 100.0}
    spec = _left_spec(heads, kv, dim, vdim, hidden, taps, chunk, rot, scale=1.0)
    w = _weights(spec, seed=4, std=0.1)
    x = torch.randn(150, hidden, generator=torch.Generator().manual_seed(6)).bfloat16()
    m = _left_m(heads, kv, dim, vdim, taps, chunk, rot, 1.0)
    want = _plain_mixer(plain.chunked_attention_mixer, x, w, m)
    for off in (39, 41):
        moved = _plain_mixer(plain.chunked_attention_mixer, x, w, {**m, "mask": {"size": off}})
        assert min(_rel(moved[t], want[t]) for t in (40, 80, 120)) > 0.02
    got = _run_mixer(spec, w, x, torch.float32, portions=portions)
    for t in (0, 1, 38, 39, 40, 41, 78, 79, 80, 81, 118, 119, 120, 121, 149):
        assert _rel(got[t], want[t]) < 1e-4, t
    assert _rel(got, want) < 1e-4


@pytest.mark.parametrize("portions", [((200, 3),), ((120, 3), (40, 30), (38, 1), (1, 1), (1, 1)), ((2, 1),) * 50 + ((100, 1),)])
def test_a_far_key_that_dominates_is_seen_across_pages_and_portions(portions):
    """Attention over all earlier positions: key 5 is made large along the direction the late queries point in, so that
    among two hundred keys it has most of the weight; lost (a page too few, a split left out) the result changes wholly."""
    spec = _attention_spec(2, 1, 16, 24, 64, scale=1.5)
    w = _weights(spec, seed=4, std=0.1)
    x = torch.randn(200, 64, generator=torch.Generator().manual_seed(6))
    x[150:] = x[5] + 0.3 * x[150:]                           # late queries and key 5 come from nearly the same input
    x = x.bfloat16()
    w["m.q"] = w["m.k"].repeat(2, 1)                         # q and k projections alike: q_t . k_5 is large for t >= 150
    m = _attention_m(2, 1, 16, 24, 1.5)
    want = _plain_mixer(plain.attention_mixer, x, w, m)
    gone = x.clone()
    gone[5] = 0
    assert _rel(_plain_mixer(plain.attention_mixer, gone, w, m)[150:153], want[150:153]) > 0.05
    assert _rel(_run_mixer(spec, w, x, torch.float32, portions=portions), want) < 1e-4


def _delta_spec(heads, kv, dim, vdim, taps, hidden, eps=1e-6):
    from ember_b200.config import GatedDeltaSpec
    return GatedDeltaSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=dim, value_dim=vdim, conv_taps=taps,
                          norm_eps=eps, decay="head", gate="silu")


def _delta_m(heads, kv, dim, vdim, taps):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps,hidden", [(4, 2, 24, 40, 3, 64), (2, 2, 70, 130, 4, 100), (3, 1, 128, 64, 2, 128),
                                                           (6, 3, 32, 64, 4, 64), (1, 1, 288, 16, 4, 72), (5, 5, 4, 8, 1, 64)])
def test_delta_rule_with_one_decay_per_head_alone(dtype, heads, kv, dim, vdim, taps, hidden):
    """One decay and one step-size bias per head, a full-rank silu gate after the norm; heads of four channels, and of 288,
    which the register-resident scan does not take; fed in portions, so state and convolution inputs come from the slot."""
    spec = _delta_spec(heads, kv, dim, vdim, taps, hidden)
    w = _weights(spec, seed=heads)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(2)).bfloat16()
    want = _plain_mixer(plain.delta_rule_mixer, x, w, _delta_m(heads, kv, dim, vdim, taps))
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


def test_the_delta_rule_forgets_at_the_rate_of_its_decay():
    """A_log of 2 with step sizes near 1: a head's state shrinks about a thousandfold a token, so a token twenty back no
    longer counts; with A_log of -8 it keeps everything.  Heads differ: the decay is per head, not shared."""
    heads, kv, dim, vdim, taps = 2, 1, 16, 16, 2
    spec = _delta_spec(heads, kv, dim, vdim, taps, 64)
    w = _weights(spec, seed=5, std=0.1)
    w["m.A_log"] = torch.tensor([2.0, -8.0]).bfloat16()
    w["m.dt_bias"] = torch.tensor([1.0, 1.0]).bfloat16()
    w["m.o"] = torch.zeros_like(w["m.o"])
    w["m.o"][:32, :32] = torch.eye(32).bfloat16()            # the heads' results side by side in the output
    x = torch.randn(90, 64, generator=torch.Generator().manual_seed(3)).bfloat16()
    m = _delta_m(heads, kv, dim, vdim, taps)
    want = _plain_mixer(plain.delta_rule_mixer, x, w, m)
    far = x.clone()
    far[60] = 0
    moved = _plain_mixer(plain.delta_rule_mixer, far, w, m)
    assert _rel(moved[89, :16], want[89, :16]) < 1e-6 and _rel(moved[89, 16:32], want[89, 16:32]) > 1e-3
    assert _rel(_run_mixer(spec, w, x, torch.float32), want) < MIX_TOL[torch.float32]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parallel_halves_are_normed_and_averaged(dtype):
    """Left attention inside chunks, right the delta rule, each result divided by its root mean square over the width
    and weighed, then half the sum.  The left half is made a hundred times larger than the right: without the norms it
    alone would be left."""
    from ember_b200.config import ParallelMixerSpec
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0}}
    left, right = _left_spec(4, 2, 16, 24, 64, 3, 20, rot, scale=0.4), _delta_spec(4, 2, 16, 32, 4, 64)
    spec = ParallelMixerSpec(hidden_size=64, left=left, right=right, left_scale=0.5, right_scale=0.5, branch_norm=True, norm_eps=1e-6)
    w = _weights(spec, seed=2, std=0.12)
    w["m.left.o"] = (w["m.left.o"].float() * 100).bfloat16()
    x = torch.randn(90, 64, generator=torch.Generator().manual_seed(9)).bfloat16()
    m = {"left": _left_m(4, 2, 16, 24, 3, 20, rot, 0.4), "right": _delta_m(4, 2, 16, 32, 4)}
    W = {k: v.double() for k, v in w.items()}
    want = plain.parallel_mixer(x.double(), W, "m.", m, 1e-6)
    plain_sum = 0.5 * (plain.chunked_attention_mixer(x.double(), W, "m.left.", m["left"], 1e-6)
                       + plain.delta_rule_mixer(x.double(), W, "m.right.", m["right"], 1e-6))
    assert _rel(plain_sum, want) > 0.5
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


# ------------------------------------------------------------------------------------------ feed-forwards
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,ff,limit", [(64, 40, 1.5), (100, 30, 0.3), (128, 256, 7.0)])
def test_dense_feed_forward_with_biases_alone(dtype, hidden, ff, limit):
    """Biases on all three projections, a limit that clamps most values and one that clamps none."""
    from ember_b200.config import GatedMLPSpec
    spec = GatedMLPSpec(hidden_size=hidden, intermediate_size=ff, activation="clamped_swish", names=("gate", "up", "down"),
                        limit=limit, bias=True)
    g = torch.Generator().manual_seed(ff)
    w = {f"f.{n}": (0.3 * torch.randn(s, generator=g)).bfloat16()
         for n, s in (("gate", (ff, hidden)), ("up", (ff, hidden)), ("down", (hidden, ff)), ("gate.b", (ff,)), ("up.b", (ff,)), ("down.b", (hidden,)))}
    x = torch.randn(90, hidden, generator=g).bfloat16()
    want = plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}, "f.", {"limit": limit})
    no_bias = plain.dense_ff(x.double(), {k: (v.double() * (0.0 if k.endswith(".b") else 1.0)) for k, v in w.items()}, "f.", {"limit": limit})
    assert _rel(no_bias, want) > 0.05
    from ember_b200.parts import build_part
    from tests.test_parts_gpu import Bench, store_of
    part = build_part("feed_forward", spec, "f.")
    b = Bench({}, dtype, capacity=512)
    part.load(store_of(w), b.rt)
    ctx = b.ctx([("x", 90)])
    xd = torch.zeros(256, hidden, device=b.dev, dtype=dtype)
    xd[:90] = x.to(dtype)
    out = torch.full((256, hidden), 7.0, device=b.dev)
    part.forward(ctx, xd, out, accumulate=False)             # the part adds its last bias itself
    assert _rel(out[:90].cpu(), want) < MIX_TOL[dtype]
    part.forward(ctx, xd, out, accumulate=False, fold_bias=True)      # or leaves it to the caller
    assert _rel(out[:90].cpu() + part.result_bias.cpu(), want) < MIX_TOL[dtype]


ROUTED_CASES = [
    # hidden, ff, experts, identity, top, groups
    (64, 40, 4, 2, 2, (3, 2)), (100, 30, 2, 1, 3, None), (96, 24, 5, 0, 1, (5, 5)), (128, 256, 40, 8, 4, (8, 3)),
    (64, 50, 3, 5, 2, (4, 3)), (64, 32, 6, 0, 3, (2, 1)), (64, 16, 1, 7, 4, (1, 1)),
]


def _routed(hidden, ff, experts, identity, top, groups, seed, spread=4.0):
    from ember_b200.config import RoutedMLPSpec
    spec = RoutedMLPSpec(hidden_size=hidden, intermediate_size=ff, experts=experts, top=top, limit=0.0, scoring="softmax",
                         correction=True, groups=groups[0] if groups else 0, keep_groups=groups[1] if groups else 0,
                         identity=identity, expert="square_relu")
    g = torch.Generator().manual_seed(seed)
    n = experts + identity
    w = {"f.router": (spread * 0.1 * torch.randn(n, hidden, generator=g)).bfloat16(),
         "f.correction": (0.3 * torch.randn(n, generator=g)).bfloat16()}
    for e in range(experts):
        w[f"f.e{e}.up"] = (0.3 * torch.randn(ff, hidden, generator=g)).bfloat16()
        w[f"f.e{e}.down"] = (0.3 * torch.randn(hidden, ff, generator=g)).bfloat16()
    router = {"experts": experts, "top": top, "identity": identity}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return spec, w, {"kind": "moe", "expert": {"ff": ff}, "router": router}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,ff,experts,identity,top,groups", ROUTED_CASES)
def test_routed_feed_forward_alone(dtype, hidden, ff, experts, identity, top, groups):
    """Softmax over all router outputs, the correction for the choice alone (it is large enough to change it), groups
    kept and dropped, identity experts chosen and not, as many choices as outputs, forty-eight outputs (more than a warp
    has lanes), one expert among seven identities."""
    spec, w, mlp = _routed(hidden, ff, experts, identity, top, groups, seed=experts + top)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    W = {k: v.double() for k, v in w.items()}
    want = plain.moe_ff(x.double(), W, "f.", mlp)
    chosen, _ = plain.route(x.double(), W, "f.", mlp["router"])
    uncorrected, _ = plain.route(x.double(), {**W, "f.correction": torch.zeros_like(W["f.correction"])}, "f.", mlp["router"])
    if top < experts + identity:
        assert (chosen.sort(-1).values != uncorrected.sort(-1).values).any()
    if identity:
        assert (chosen >= experts).any()
    got, _, _ = _run_feed_forward(spec, w, x, dtype)
    errs = sorted(_rel(got[t], want[t]) for t in range(90))
    # a token whose choice is a close call may fall the other way in bfloat16 (the router reads the rounded input)
    assert errs[len(errs) // 2] < MIX_TOL[dtype] and errs[-3 if dtype == torch.bfloat16 else -1] < 10 * MIX_TOL[dtype]


def test_the_router_on_the_device_chooses_what_the_plain_one_does():
    """The choices themselves, from given logits: groups of neighbours, negative choice scores, ties to the lower index."""
    from ember_b200 import ops
    T, E, top = 64, 12, 3
    g = torch.Generator().manual_seed(1)
    logits = (2.0 * torch.randn(T, E, generator=g)).float()
    correction = torch.tensor([-9.0, -9.0, -9.5, -1.0, -1.0, -1.5, -9.5, -9.5, -9.5, 0.2, -0.3, 0.1])
    router = {"experts": 8, "identity": 4, "top": top, "groups": {"count": 4, "keep": 2}}
    W = {"r.router": torch.eye(E, dtype=torch.float64), "r.correction": correction.double()}
    chosen, weights = plain.route(logits.double(), W, "r.", router)
    sel = torch.zeros(T * top, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(T * top, dtype=torch.float32, device="cuda")
    ops.moe_route(logits.cuda(), T, top, sel, wgt, rule=(correction.cuda(), 1.0, False, "softmax", 4, 2))
    torch.cuda.synchronize()
    assert sel.view(T, top).cpu().tolist() == chosen.tolist()
    assert float((wgt.view(T, top).cpu().double() - weights).abs().max()) < 1e-6
    assert set(chosen.flatten().tolist()) <= {3, 4, 5, 9, 10, 11}            # the two kept groups


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_experts_of_prompt_portions_on_tensor_cores(dtype, tmp_path):
    """A portion of more than 256 tokens takes the per-expert product on the tensor cores in bfloat16 (gathered rows, the
    squared relu as a kernel of its own); identity experts' pairs have slots there and no rows to multiply."""
    cfg = {"architecture": "Pepapel", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0}, "postln_alpha": 2.0,
           "layers": [{"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.18},
                       "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 6, "top": 3, "identity": 2, "groups": {"count": 4, "keep": 3}}}}] * 2}
    d = write_pepapel_dir(cfg, str(tmp_path), seed=5)
    inputs = plain_inputs(d)
    toks = np.random.default_rng(3).integers(0, 300, size=420).tolist()
    requests = {"r0": toks}
    want = {"r0": plain.forward(*inputs, toks).numpy()}
    steps = trace_portions(requests, sizes=(300, 2, 118))
    outputs, _ = replay(d, dtype, steps, 448, max_batch_tokens=512)
    assert_close(collect(steps, outputs), want, dtype, "experts on tensor cores")


# ------------------------------------------------------------------------------------ the norm after the sum
@pytest.mark.parametrize("centred", [True, False], ids=["layer norm", "rms norm"])
@pytest.mark.parametrize("hidden,alpha,bias", [(64, 2.5, False), (100, 0.7, True), (2048, 1.0, True), (13000, 3.0, False)])
def test_scale_add_norm_in_one_kernel(hidden, alpha, bias, centred):
    """x <- norm(alpha x + y + b) in place, with the bfloat16 copy of the new rows; rows with a large mean, so that a
    variance taken as E[x^2] - mean^2 or a missing centring would show."""
    from ember_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    x = (torch.randn(37, hidden, generator=g) + 30.0).cuda()
    y = torch.randn(37, hidden, generator=g).cuda()
    w = (1 + 0.2 * torch.randn(hidden, generator=g)).cuda()
    b = torch.randn(hidden, generator=g).cuda() if bias else None
    z = alpha * x.double() + y.double() + (b.double() if bias else 0.0)
    if centred:
        z = z - z.mean(-1, keepdim=True)
    want = z / torch.sqrt((z * z).mean(-1, keepdim=True) + 1e-5) * w.double()
    rounded = torch.zeros(40, hidden, dtype=torch.bfloat16, device="cuda")
    keep = x[30:].clone()
    ops.scaled_add_norm(y, b, alpha, w, None, 1e-5, centred, x, 30, rounded=rounded)
    torch.cuda.synchronize()
    assert float((x[:30].double() - want[:30]).abs().max()) < 2e-5 * float(want.abs().max())
    assert torch.equal(rounded[:30], x[:30].bfloat16()) and torch.equal(x[30:], keep) and float(rounded[30:].abs().max()) == 0.0


@pytest.mark.parametrize("hidden", [64, 100, 2048])
def test_two_rows_normed_weighed_and_summed_in_one_kernel(hidden):
    from ember_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    a, b = (100.0 * torch.randn(20, hidden, generator=g)).cuda(), (0.01 * torch.randn(20, hidden, generator=g)).cuda()
    wa, wb = (1 + 0.2 * torch.randn(hidden, generator=g)).cuda(), torch.randn(hidden, generator=g).cuda()
    rms = lambda t: t.double() / torch.sqrt((t.double() ** 2).mean(-1, keepdim=True) + 1e-6)      # noqa: E731
    want = rms(a) * wa.double() + rms(b) * wb.double()
    out = torch.full((20, hidden), 3.0, device="cuda")
    ops.pair_norm_sum(a, wa, b, wb, 1e-6, out, 16)
    ops.pair_norm_sum(a, wa, b, wb, 1e-6, out, 16, accumulate=True)
    torch.cuda.synchronize()
    assert float((out[:16].double() - 2 * want[:16]).abs().max()) < 1e-5 * float(want.abs().max())
    assert float((out[16:] - 3.0).abs().max()) == 0.0
