"""Pepapel without a device: reading config.json, the tensors a model declares, what its layers ask of the cache, the
random-weights folder, and the plain implementation's own mechanisms on cases whose answer is known."""
import json
import math

import pytest
import torch

from tests.pepapel_configs import PEPAPEL, drawn_pepapel, pepapel_config, plain_inputs, write_pepapel_dir
from tests.plain import pepapel_plain as plain


def test_registered_and_resolved_by_the_architecture_key():
    from ember_b200.config import PepapelConfig, config_from_dict, registered_architectures
    assert "Pepapel" in registered_architectures()
    cfg = config_from_dict(PEPAPEL["a"]["json"])
    assert isinstance(cfg, PepapelConfig) and cfg.width == 128 and len(cfg.layers) == 4 and cfg.alpha == 1.7
    assert config_from_dict(cfg.to_json()) == cfg
    bare = config_from_dict(PEPAPEL["b"]["json"])
    assert (bare.embedding_scale, bare.alpha) == (1.0, 1.0)


@pytest.mark.parametrize("name", sorted(PEPAPEL))
def test_spec_layers_and_cache_needs(name):
    """An attention layer asks for pages; a parallel layer for pages (left), a state slot for the delta rule's matrices
    and convolution inputs (right), and a state slot for the left half's convolution inputs when it has more than one tap."""
    from ember_b200.model.causal_lm import CausalLM
    cfg = pepapel_config(name)
    j = PEPAPEL[name]["json"]
    spec = cfg.to_model_spec()
    needs = CausalLM(spec).cache_needs()
    assert not spec.tie_embeddings and spec.embedding_multiplier == j.get("embedding", {}).get("scale", 1.0)
    kv_bytes, state_floats = 0, 0
    for i, l in enumerate(j["layers"]):
        roles = spec.layers[i].roles()
        assert spec.layers[i].arrangement == "postnorm" and spec.layers[i].constant("alpha", -1.0) == j.get("postln_alpha", 1.0)
        assert ("feed_forward" in roles) == (l["mlp"] is not None) == ("feed_forward_norm" in roles)
        m = l["mixer"]
        if l["type"] == "attention":
            n = needs[i]
            assert (n.kind, n.num_kv_heads, n.head_dim, n.value_dim or n.head_dim) == ("full", m["kv_heads"], m["dim"], m["vdim"])
            kv_bytes += 2 * m["kv_heads"] * (m["dim"] + m["vdim"])
        else:
            a, r = m["left"], m["right"]
            n = needs[(i, "left")]
            assert (n.kind, n.num_kv_heads, n.head_dim, n.value_dim or n.head_dim) == ("full", a["kv_heads"], a["dim"], a["vdim"])
            kv_bytes += 2 * a["kv_heads"] * (a["dim"] + a["vdim"])
            channels = a["heads"] * a["dim"] + a["kv_heads"] * (a["dim"] + a["vdim"])
            assert ((i, "left.conv") in needs) == (a["conv"] > 1)
            if a["conv"] > 1:
                assert needs[(i, "left.conv")].kind == "state" and needs[(i, "left.conv")].state_shape == ((a["conv"] - 1) * channels,)
                state_floats += (a["conv"] - 1) * channels
            rc = 2 * r["kv_heads"] * r["dim"] + r["heads"] * r["vdim"]
            want = r["heads"] * r["dim"] * r["vdim"] + (r["conv"] - 1) * rc
            assert needs[(i, "right")].kind == "state" and needs[(i, "right")].state_shape == (want,)
            state_floats += want
    assert cfg.kv_bytes_per_token(2) == kv_bytes and cfg.state_bytes_per_request() == 4 * state_floats


def test_bad_configurations_are_refused_when_read():
    from ember_b200.config import ConfigError, config_from_dict
    good = PEPAPEL["a"]["json"]
    for edit in (lambda c: c.pop("width"), lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(type="gla"),
                 lambda c: c["layers"][1]["mixer"].pop("scale"), lambda c: c["layers"][0]["mlp"].update(kind="glu"),
                 lambda c: c.update(layers=[]), lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
                 lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                 lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=4),
                 lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=34),
                 lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3),
                 lambda c: c["layers"][0]["mixer"]["right"].update(heads=0), lambda c: c["layers"][0]["mixer"].pop("right"),
                 lambda c: c["layers"][0]["mlp"].pop("limit"), lambda c: c["layers"][1]["mixer"]["q_temp"].pop("every")):
        c = json.loads(json.dumps(good))
        edit(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)


@pytest.mark.parametrize("name", sorted(PEPAPEL))
def test_random_folder_declares_what_the_plain_implementation_reads(name, tmp_path):
    d = write_pepapel_dir(name, str(tmp_path))
    cfg, W = plain_inputs(d)
    layers = []
    logits = plain.forward(cfg, W, [5, 17, 3, 200, 41, 7, 7, 250], layers_out=layers)
    assert logits.shape == (8, cfg["vocab"]) and bool(torch.isfinite(logits).all()) and len(layers) == len(cfg["layers"])
    from ember_b200.config import load_config
    from ember_b200.model.causal_lm import CausalLM
    declared = {x.name: tuple(x.shape) for x in CausalLM(load_config(d).to_model_spec()).weight_decls()}
    assert declared == {k: tuple(v.shape) for k, v in W.items()}


def test_drawn_configurations_are_read():
    from ember_b200.config import config_from_dict
    for seed in range(40):
        c = drawn_pepapel(seed)
        assert config_from_dict(config_from_dict(c).to_json()).to_json()["layers"] == c["layers"]


# ------------------------------------------------------------------ the plain implementation on known cases
def test_plain_convolution_meets_the_current_token_with_its_last_tap():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]                 # 1 2 3 4 5
    taps = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    assert plain.short_conv(u, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    assert plain.short_conv(u, torch.tensor([[2.0]], dtype=torch.float64))[:, 0].tolist() == [2.0, 4.0, 6.0, 8.0, 10.0]


def test_plain_mask_counts_chunks_from_the_start():
    m = plain.visible(7, 3)
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert m[3].tolist() == [False, False, False, True, False, False, False]
    assert m[5].tolist() == [False, False, False, True, True, True, False]
    assert plain.visible(4)[3].tolist() == [True] * 4


def test_plain_temperature_and_rotation():
    t = plain.query_temperature(9, {"coef": 0.5, "every": 4}, torch.float64)
    assert t[2] == 1.0 and abs(float(t[3]) - (1 + 0.5 * math.log(2))) < 1e-12 and abs(float(t[7]) - (1 + 0.5 * math.log(3))) < 1e-12
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0                                                          # pairs (0, 2), (1, 3); 4 and 5 pass
    x[:, 0, 5] = 9.0
    y = plain.rotate_half(x, {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0}})
    assert abs(float(y[2, 0, 0]) - math.cos(2 * 1.0 / 2.0)) < 1e-12 and abs(float(y[2, 0, 2]) - math.sin(1.0)) < 1e-12
    assert float(y[2, 0, 1]) == 0.0 and float(y[1, 0, 5]) == 9.0


def test_plain_router_keeps_the_best_groups_and_weighs_by_the_plain_scores():
    W = {"r.router": torch.eye(6, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 5.0, 0.0], dtype=torch.float64)}
    h = torch.tensor([[3.0, 2.9, 0.0, 0.0, 0.0, 2.0]], dtype=torch.float64)
    s = torch.softmax(h, -1)[0]
    # groups (0, 1), (2, 3), (4, 5): the correction lifts group 2 to the top, group 0 is second, group 1 is out
    chosen, weights = plain.route(h, W, "r.", {"experts": 4, "identity": 2, "top": 3, "groups": {"count": 3, "keep": 2}})
    assert chosen[0].tolist() == [4, 0, 1] and torch.allclose(weights[0], s[[4, 0, 1]])
    # with one group kept, the two largest of the best group alone
    chosen, _ = plain.route(h, W, "r.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert chosen[0].tolist() == [4, 5]
    # a negative choice score still beats an expert outside the kept groups
    W["r.correction"] = torch.tensor([-9.0, -9.0, -1.0, -1.0, -9.5, -9.5], dtype=torch.float64)
    chosen, _ = plain.route(h, W, "r.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert sorted(chosen[0].tolist()) == [2, 3]


def test_plain_identity_expert_returns_the_input():
    W = {"f.router": torch.tensor([[0.0, 0.0], [50.0, 0.0]], dtype=torch.float64), "f.correction": torch.zeros(2, dtype=torch.float64),
         "f.e0.up": torch.ones(3, 2, dtype=torch.float64), "f.e0.down": torch.ones(2, 3, dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0], [-1.0, 0.5]], dtype=torch.float64)
    y = plain.moe_ff(h, W, "f.", {"kind": "moe", "expert": {"ff": 3}, "router": {"experts": 1, "identity": 1, "top": 1}})
    assert torch.allclose(y[0], h[0])                      # the identity output wins at logit 50: weight ~1, output h
    s = torch.softmax(torch.tensor([0.0, -50.0]), -1)[0].double()
    assert torch.allclose(y[1], s * torch.full((2,), 0.0, dtype=torch.float64))     # relu(-0.5)^2 = 0 through expert 0


def test_plain_delta_rule_writes_then_reads():
    """One head, no decay (A_log very negative), beta ~ 1: after one token the read-out of the same key returns the value."""
    hid, D, V = 4, 2, 3
    W = {n: torch.zeros(s, dtype=torch.float64) for n, s in (("m.q", (D, hid)), ("m.k", (D, hid)), ("m.v", (V, hid)), ("m.b", (1, hid)),
                                                              ("m.a", (1, hid)), ("m.g", (V, hid)), ("m.o", (hid, V)))}
    W.update({"m.q.conv": torch.ones(D, 1, dtype=torch.float64), "m.k.conv": torch.ones(D, 1, dtype=torch.float64),
              "m.v.conv": torch.ones(V, 1, dtype=torch.float64), "m.A_log": torch.tensor([-40.0], dtype=torch.float64),
              "m.dt_bias": torch.zeros(1, dtype=torch.float64), "m.norm": torch.ones(V, dtype=torch.float64)})
    W["m.q"][0, 0] = W["m.k"][0, 0] = 1.0
    W["m.v"][:, 1] = torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64)
    W["m.b"][0, 2] = 1.0
    W["m.g"][:, 3] = 1.0
    W["m.o"][:V, :] = torch.eye(V, dtype=torch.float64)
    h = torch.tensor([[5.0, 1.0, 40.0, 30.0]], dtype=torch.float64)          # q = k = silu(5) e0, v = silu(1 2 3), beta = 1, gate = silu(30)
    y = plain.delta_rule_mixer(h, W, "m.", {"heads": 1, "kv_heads": 1, "dim": D, "vdim": V, "conv": 1}, 1e-6)
    v = plain.silu(torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64))
    want = plain.rms_norm(v * D ** -0.5, None, 1e-6) * 30.0                  # o = v (k . q) = v / sqrt(D); rms norm; silu(30) = 30
    assert torch.allclose(y[0, :V], want, rtol=1e-5)


def test_the_command_line_writes_and_describes_a_random_model(tmp_path, capsys):
    """``random`` makes a folder from a config.json of this design, ``info`` reads it back through the registry."""
    from ember_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(PEPAPEL["b"]["json"]))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--out", str(out), "--seed", "3"]) == 0
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "pepapel: 4 layers (attention, parallel, parallel, attention)" in text and "state per request" in text
    W = plain_inputs(str(out))[1]
    assert W["l1.mix.right.dt_bias"].shape == (3,) and W["l1.mix.left.q.conv"].shape == (60, 1) and "l1.mix.left.g" in W
    assert W["l1.mlp.router"].shape == (3, 100) and "l1.mlp.e1.up" in W and "l1.mlp.e2.up" not in W and "l1.mlp.e0.gate" not in W
