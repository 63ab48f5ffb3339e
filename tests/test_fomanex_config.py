"""Fomanex without a device: reading config.json, the tensors a model declares, a cache or state for every pass of a
looped layer, the run order, the random-weights folder, and the plain implementation's own mechanisms on cases whose
answer is known."""
import json
import math

import pytest
import torch

from tests.fomanex_configs import FOMANEX, fomanex_config, plain_inputs, write_fomanex_dir


def test_registered_and_resolved_by_the_architecture_key():
    from ember_b200.config import FomanexConfig, config_from_dict, registered_architectures
    assert "Fomanex" in registered_architectures()
    cfg = config_from_dict(FOMANEX["p"]["json"])
    assert isinstance(cfg, FomanexConfig) and cfg.width == 96 and len(cfg.layers) == 4 and cfg.streams == 3
    assert config_from_dict(cfg.to_json()) == cfg
    bare = config_from_dict(FOMANEX["s"]["json"])
    assert (bare.streams, bare.loop, bare.logit_softcap, bare.embedding_scale, bare.residual_mult) == (0, None, 0.0, 1.0, 1.0)
    assert "streams" not in bare.to_json() and "loop" not in bare.to_json()


@pytest.mark.parametrize("name", sorted(FOMANEX))
def test_spec_layers_cache_needs_and_run_order(name):
    """Every run of a layer has a cache or a state of its own: the first pass under the layer's number, later passes
    under (layer, "", pass)."""
    from ember_b200.model.causal_lm import CausalLM
    from tests.plain.fomanex_plain import layer_order
    cfg = fomanex_config(name)
    j = FOMANEX[name]["json"]
    spec = cfg.to_model_spec()
    needs = CausalLM(spec).cache_needs()
    assert spec.tie_embeddings and spec.residual_streams == max(j.get("streams", 1), 1)
    assert [e.layer for e in spec.schedule] == layer_order(j)
    runs = {}
    for e in spec.schedule:
        assert e.instance == runs.get(e.layer, 0)
        runs[e.layer] = e.instance + 1
    assert len(needs) == len(spec.schedule)
    for i, l in enumerate(j["layers"]):
        m, roles = l["mixer"], spec.layers[i].roles()
        assert ("feed_forward" in roles) == (l["mlp"] is not None) == ("feed_forward_connection" in roles)
        for t in range(runs[i]):
            n = needs[i if t == 0 else (i, "", t)]
            if l["type"] == "latent_attention":
                assert (n.kind, n.num_kv_heads, n.head_dim, n.keys_only) == ("full", 1, m["kv_rank"] + m["rot_dim"], True)
            else:
                assert n.kind == "state" and n.state_shape == (m["heads"] * m["dim"] * m["dim"] + j["width"],)
    latent_rows = sum((l["mixer"]["kv_rank"] + l["mixer"]["rot_dim"]) * runs[i] for i, l in enumerate(j["layers"])
                      if l["type"] == "latent_attention")
    assert cfg.kv_bytes_per_token(2) == 2 * latent_rows


def test_bad_configurations_are_refused_when_read():
    from ember_b200.config import ConfigError, config_from_dict
    good = FOMANEX["p"]["json"]
    for edit in (lambda c: c.pop("width"), lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(type="gla"),
                 lambda c: c["layers"][0]["mixer"].pop("kv_rank"), lambda c: c["layers"][0]["mlp"].update(kind="glu"),
                 lambda c: c.update(layers=[]), lambda c: c["loop"].update(stop=5), lambda c: c["loop"].update(times=0),
                 lambda c: c["loop"].update(start=3, stop=2), lambda c: c["layers"][1]["mlp"]["router"].update(top=6),
                 lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), lambda c: c.update(logit_softcap=-1.0),
                 lambda c: c.update(streams=99), lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"),
                 lambda c: c["layers"][1]["mixer"].update(heads=0)):
        c = json.loads(json.dumps(good))
        edit(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)


def test_random_folder_declares_what_the_plain_implementation_reads(tmp_path):
    from tests.plain import fomanex_plain as plain
    d = write_fomanex_dir("p", str(tmp_path), drop_ranks=True)
    cfg, W = plain_inputs(d)
    assert "decay_rank" not in json.dumps(cfg)
    layers = []
    logits = plain.forward(cfg, W, [5, 17, 3, 200, 41, 7, 7, 250], layers_out=layers)
    assert logits.shape == (8, 300) and bool(torch.isfinite(logits).all()) and len(layers) == 1 + 2 * 3 + 1
    assert float(logits.abs().max()) < 12.0                                  # the cap
    from ember_b200.config import load_config
    from ember_b200.model.causal_lm import CausalLM
    from ember_b200.weights import WeightStore
    store = WeightStore.from_dir(d)
    model = CausalLM(load_config(d).to_model_spec())
    wkv = model.blocks[1].parts["mixer"]
    assert wkv.decay_rank == 0 and store.shape("l1.mix.w1") == (8, 96)      # the rank is the stored tensor's
    assert store.shape("l1.hc2.mix") == (3, 3) and store.shape("l0.norm1.alpha") == ()
    assert store.shape("l2.norm2") is None and store.shape("l2.hc2.in") is None      # a layer without feed-forward


def test_a_model_without_copies_of_the_stream_stores_no_connection_tensors(tmp_path):
    from ember_b200.weights import WeightStore
    d = write_fomanex_dir("s", str(tmp_path))
    store = WeightStore.from_dir(d)
    assert store.shape("l0.hc1.in") is None and store.shape("l0.ls1") == (64,)
    from tests.plain import fomanex_plain as plain
    cfg, W = plain_inputs(d)
    assert bool(torch.isfinite(plain.forward(cfg, W, [1, 2, 3])).all())


# ------------------------------------------------------------- the plain implementation on known answers
def test_plain_dynamic_tanh():
    from tests.plain.fomanex_plain import dynamic_tanh
    W = {"n": torch.tensor([2.0, 3.0]), "n.b": torch.tensor([0.5, -1.0]), "n.alpha": torch.tensor(0.5)}
    x = torch.tensor([[2.0, -4.0]], dtype=torch.float64)
    want = torch.tensor([[math.tanh(1.0) * 2 + 0.5, math.tanh(-2.0) * 3 - 1.0]], dtype=torch.float64)
    assert torch.allclose(dynamic_tanh(x, W, "n"), want)


def test_plain_halves_rotate_by_position_times_frequency():
    from tests.plain.fomanex_plain import rotate_half, scaled_frequencies
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0                                  # pair 0 is (element 0, element 2), pair 1 is (1, 3)
    x[:, 0, 1] = 1.0
    x[:, 0, 5] = 7.0
    y = rotate_half(x, {"dims": 4, "base": 100.0})
    for p in range(3):
        assert torch.allclose(y[p, 0, [0, 2]], torch.tensor([math.cos(p), math.sin(p)], dtype=torch.float64))
        assert torch.allclose(y[p, 0, [1, 3]], torch.tensor([math.cos(p * 0.1), math.sin(p * 0.1)], dtype=torch.float64))
        assert y[p, 0, 5] == 7.0 and y[p, 0, 4] == 0.0
    assert torch.equal(rotate_half(x[1:], {"dims": 4, "base": 100.0}, first_position=1), y[1:])
    # stretched: fast pairs keep their frequency, slow ones are divided by the factor, the ramp lies between; cos and
    # sin grow by 0.1 ln(factor) + 1
    rot = {"dims": 16, "base": 10000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}
    f, mult = scaled_frequencies(rot)
    plain_f = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    turn = lambda t: 16 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(10000.0))          # noqa: E731
    lo, hi = max(math.floor(turn(16.0)), 0), min(math.ceil(turn(2.0)), 15)
    assert (lo, hi) == (0, 2) and abs(mult - (0.1 * math.log(8.0) + 1)) < 1e-12
    assert torch.allclose(f[0], plain_f[0]) and torch.allclose(f[1], plain_f[1] * (0.5 / 8 + 0.5))
    assert torch.allclose(f[2:], plain_f[2:] / 8.0)
    one = torch.zeros(2, 16, dtype=torch.float64)
    one[:, 0] = 1.0
    assert abs(float(rotate_half(one, rot)[1].norm()) - mult) < 1e-12


def test_plain_router_scores_choice_and_weights():
    """The correction moves the choice and not the weight; the weights are scores times the constant, not renormalised."""
    from tests.plain.fomanex_plain import routed_ff, silu
    W = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5]], dtype=torch.float64),
         "r.correction": torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64)}
    for e in range(3):
        W[f"r.e{e}.gate"] = torch.eye(2, dtype=torch.float64) * (e + 1)
        W[f"r.e{e}.up"] = torch.eye(2, dtype=torch.float64)
        W[f"r.e{e}.down"] = torch.eye(2, dtype=torch.float64)
    mlp = {"router": {"experts": 3, "top": 1, "scale": 2.5}}
    h = torch.tensor([[3.0, 1.0]], dtype=torch.float64)             # scores sigmoid(3, 1, 2): without correction expert 0
    out = routed_ff(h, W, "r.", mlp)
    s2 = 1 / (1 + math.exp(-2.0))
    assert torch.allclose(out, s2 * 2.5 * silu(3.0 * h) * h)
    W["r.correction"] = torch.zeros(3, dtype=torch.float64)
    s0 = 1 / (1 + math.exp(-3.0))
    assert torch.allclose(routed_ff(h, W, "r.", mlp), s0 * 2.5 * silu(h) * h)


def test_plain_time_mixing_on_a_known_case():
    """One head of one channel, identity projections, mu = 0 (each projection reads the token itself): with decay w
    and bonus u, o_t = r_t (S_(t-1) + u k_t v_t) and S_t = w S_(t-1) + k_t v_t; the read-out's unit norm leaves its sign."""
    from tests.plain.fomanex_plain import wkv
    one = torch.ones(1, 1, dtype=torch.float64)
    W = {"m.mu." + n: torch.zeros(1, dtype=torch.float64) for n in "rkvgw"}
    W.update({"m." + n: one for n in ("r", "k", "v", "g", "w1", "w2", "o")})
    W.update({"m.w0": torch.tensor([-1.0], dtype=torch.float64), "m.u": torch.tensor([[-3.0]], dtype=torch.float64),
              "m.norm": torch.ones(1, dtype=torch.float64)})
    h = torch.tensor([[1.0], [2.0], [0.5]], dtype=torch.float64)
    got = wkv(h, W, "m.", {"heads": 1, "dim": 1}, 0.0)
    S, want = 0.0, []
    for x in h[:, 0].tolist():
        o = x * (S + -3.0 * x * x)
        S = math.exp(-math.exp(math.tanh(x) - 1.0)) * S + x * x
        want.append(math.copysign(1.0, o) * x / (1 + math.exp(-x)))
    assert torch.allclose(got[:, 0], torch.tensor(want, dtype=torch.float64))
    # mu = 1: every projection reads the token before (zeros before the first)
    W.update({"m.mu." + n: torch.ones(1, dtype=torch.float64) for n in "rkvgw"})
    assert torch.allclose(wkv(h, W, "m.", {"heads": 1, "dim": 1}, 0.0)[1:, 0], torch.tensor(want[:2], dtype=torch.float64))


def test_plain_hyper_connections_on_a_known_case(tmp_path):
    """Copies that start equal, are read as a weighted sum and written all at once from the old ones."""
    from tests.plain import fomanex_plain as plain
    d = write_fomanex_dir("p", str(tmp_path))
    cfg, W = plain_inputs(d)
    cfg = dict(cfg, layers=cfg["layers"][:1], loop=None)
    cfg["layers"][0]["mlp"] = None
    toks = [4, 9, 2]
    layers = []
    plain.forward(cfg, W, toks, layers_out=layers)
    x0 = plain.dynamic_tanh(W["embed"][toks] * 9.8, W, "embed.norm")
    u = x0 * W["l0.hc1.in"].sum()
    y = plain.latent_attention(plain.dynamic_tanh(u, W, "l0.norm1"), W, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5) * W["l0.ls1"]
    want = x0 * W["l0.hc1.mix"].sum() + 0.6 * W["l0.hc1.out"].sum() * y
    assert torch.allclose(layers[0], want)


def test_cli_info_and_random(tmp_path, capsys):
    """`python -m ember_b200 info` on a folder written by the random-weights mode."""
    from ember_b200 import cli
    d = write_fomanex_dir("p", str(tmp_path / "m"), drop_ranks=False)
    assert cli.main(["info", "-m", d]) in (0, None)
    out = capsys.readouterr().out
    assert "fomanex: 4 layers" in out and "state per request" in out
