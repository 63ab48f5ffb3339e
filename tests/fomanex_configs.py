"""The tests' own small Fomanex configurations.  They differ from one another in every size, in the order and number
of layers, in the constants, in which stretch of layers is run several times, in the number of copies of the residual
stream, and in which values happen to be equal (key and value sizes, the latent and the heads, experts and choices) or 1."""
from __future__ import annotations

import json
import os

import torch


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, rot):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


def _moe(ff, experts, top, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


FOMANEX = {
    # widths the tensor-core product takes; three copies of the stream; a looped stretch of a recurrent and a latent
    # layer run three times; values narrower than keys; a layer without feed-forward; a stretched rotation
    "p": dict(seed=13, json={
        "architecture": "Fomanex", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 9.8},
        "residual_mult": 0.6, "streams": 3, "logit_scale": 1.3, "logit_softcap": 12.0, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [
            {"type": "latent_attention", "mixer": _latent(3, 24, 8, 20, 40, 0.17, _rot(8, 10000.0, (8.0, 64, 16.0, 2.0))), "mlp": _dense(64)},
            {"type": "wkv", "mixer": {"heads": 4, "dim": 16, "decay_rank": 8}, "mlp": _moe(40, 5, 2, 1.5)},
            {"type": "latent_attention", "mixer": _latent(5, 16, 16, 32, 24, 0.2, _rot(16, 500.0, (4.0, 32, 32.0, 1.0))), "mlp": None},
            {"type": "wkv", "mixer": {"heads": 2, "dim": 40, "decay_rank": 5}, "mlp": _dense(48)},
        ]}),
    # a width no tensor-core product takes; one copy of the stream with learned connections; nothing looped; one head;
    # as many choices as experts and a single choice; no cap on the logits; a loop of one pass
    "q": dict(seed=29, json={
        "architecture": "Fomanex", "vocab": 257, "width": 100, "norm": {"eps": 1e-6}, "embedding": {"scale": 14.0},
        "residual_mult": 1.0, "streams": 1, "logit_scale": 3.0, "logit_softcap": 0.0, "loop": {"start": 0, "stop": 2, "times": 1},
        "layers": [
            {"type": "wkv", "mixer": {"heads": 1, "dim": 72, "decay_rank": 3}, "mlp": _moe(30, 3, 3, 0.8)},
            {"type": "latent_attention", "mixer": _latent(1, 32, 4, 48, 72, 0.12, _rot(4, 77.0)), "mlp": _moe(50, 7, 1, 2.0)},
            {"type": "latent_attention", "mixer": _latent(40, 8, 4, 6, 20, 0.3, _rot(4, 1e6, (2.0, 16, 8.0, 0.5))), "mlp": None},
            {"type": "wkv", "mixer": {"heads": 6, "dim": 12, "decay_rank": 16}, "mlp": _dense(36)},
        ]}),
    # head sizes of a real model's layers (a latent of 256 with 64 rotated under heads of 128; recurrent heads of 64 and one
    # of 288 key channels, which the register-resident scan does not take); the whole model looped twice; four copies
    "r": dict(seed=37, json={
        "architecture": "Fomanex", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0},
        "residual_mult": 0.4, "streams": 4, "logit_scale": 2.5, "logit_softcap": 30.0, "loop": {"start": 0, "stop": 3, "times": 2},
        "layers": [
            {"type": "wkv", "mixer": {"heads": 4, "dim": 64, "decay_rank": 32}, "mlp": _moe(128, 8, 2, 2.5)},
            {"type": "latent_attention", "mixer": _latent(4, 128, 64, 128, 256, 0.0722, _rot(64, 1e6, (4.0, 128, 32.0, 1.0))), "mlp": _dense(512)},
            {"type": "wkv", "mixer": {"heads": 1, "dim": 288, "decay_rank": 16}, "mlp": None},
        ]}),
    # no "streams" key: the plain residual sum without connection tensors; no loop, no cap, no embedding scale
    "s": dict(seed=41, json={
        "architecture": "Fomanex", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "layers": [
            {"type": "latent_attention", "mixer": _latent(2, 16, 8, 16, 16, 0.25, _rot(8, 100.0)), "mlp": _moe(24, 4, 2, 1.0)},
            {"type": "wkv", "mixer": {"heads": 2, "dim": 32, "decay_rank": 4}, "mlp": _dense(80)},
        ]}),
}


def fomanex_config(name: str):
    from ember_b200.config import FomanexConfig
    return FomanexConfig.from_json(FOMANEX[name]["json"])


def write_fomanex_dir(name: str, out_dir: str, drop_ranks: bool = True) -> str:
    """A model folder with random weights.  ``drop_ranks``: config.json is written without the low-rank size, as a
    stored model's is (it is read from the tensors' shapes)."""
    from ember_b200.weights import write_model_dir
    write_model_dir(fomanex_config(name), out_dir, seed=FOMANEX[name]["seed"], dtype=torch.bfloat16)
    path = os.path.join(out_dir, "config.json")
    with open(path, "w") as f:                    # the keys exactly as the test wrote them (absent ones stay absent)
        c = json.loads(json.dumps(FOMANEX[name]["json"]))
        if drop_ranks:
            for l in c["layers"]:
                l["mixer"].pop("decay_rank", None)
        json.dump(c, f)
    return out_dir


def plain_inputs(model_dir: str):
    """(config dictionary, name -> float64 tensor) as the plain implementation takes them."""
    from tests.plain.qwen3_plain import read_safetensors
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: (v.double() if v.is_floating_point() else v) for k, v in W.items()}


def drawn_fomanex(seed: int) -> dict:
    """A configuration drawn from a seed: 3 to 7 layers of either mixer in any order, any feed-forward or none, head
    counts and sizes from short lists that include ones no tensor-core kernel takes, 1 to 8 copies of the stream, a looped
    stretch anywhere (also empty, also a single pass), constants from short lists."""
    import numpy as np
    rng = np.random.default_rng(seed)
    pick = lambda *v: v[int(rng.integers(0, len(v)))]                         # noqa: E731
    width, n = pick(128, 192, 256, 384, 448, 136, 200), int(rng.integers(3, 8))
    layers = []
    for _ in range(n):
        if rng.random() < 0.5:
            dim, rot_dim = pick(16, 24, 32, 48, 64, 96, 128), pick(8, 16, 32, 64, 4, 24)
            rot = {"dims": rot_dim, "base": pick(10000.0, 500000.0, 1e6, 50000.0)}
            if rng.random() < 0.8:
                rot["scaling"] = {"factor": pick(2.0, 4.0, 8.0, 16.0, 40.0), "original": pick(64, 128, 256, 512, 4096),
                                  "fast": pick(32.0, 16.0, 8.0), "slow": pick(1.0, 2.0, 0.5)}
            mixer = _latent(pick(2, 3, 4, 5, 8, 12), dim, rot_dim, pick(16, 32, 48, 96, 128, dim), pick(32, 48, 96, 128, 160, 256, 40),
                            float((dim + rot_dim) ** -0.5 * pick(1.0, 0.7, 1.5)), rot)
            kind = "latent_attention"
        else:
            mixer = {"heads": pick(1, 2, 4, 5, 8), "dim": pick(16, 32, 64, 80, 96, 128, 24), "decay_rank": pick(8, 16, 24, 32, 64, 12)}
            kind = "wkv"
        k = rng.random()
        if k < 0.4:
            mlp = _dense(pick(128, 256, 512, 768, 200))
        elif k < 0.9:
            e = pick(4, 8, 16, 32, 64, 6)
            mlp = _moe(pick(32, 64, 128, 192, 40), e, int(rng.integers(1, min(e, 8) + 1)), pick(1.0, 1.5, 2.5, 0.5))
        else:
            mlp = None
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Fomanex", "vocab": pick(384, 512, 640, 768, 1000, 333), "width": width, "norm": {"eps": pick(1e-5, 1e-6)},
           "embedding": {"scale": float(width ** 0.5 * pick(1.0, 0.5))}, "residual_mult": pick(0.5, 1.0, 0.3, 0.7),
           "streams": pick(1, 2, 3, 4, 6, 8), "logit_scale": pick(1.0, 2.0, 0.5, 4.0), "logit_softcap": pick(15.0, 30.0, 50.0, 8.0),
           "layers": layers}
    if rng.random() < 0.85:
        a = int(rng.integers(0, n))
        cfg["loop"] = {"start": a, "stop": int(rng.integers(a, n + 1)), "times": int(rng.integers(1, 4))}
    return cfg


def write_drawn_dir(seed: int, out_dir: str) -> str:
    """A folder for ``drawn_fomanex(seed)`` with random weights whose mix matrices are scaled so that every copy of the
    stream stays a weighted mean of the old ones (columns sum to 1): over a dozen runs the copies keep their size, and
    float32 rounding stays where the arithmetic puts it."""
    from ember_b200.config import FomanexConfig
    from ember_b200.weights import write_model_dir
    from ember_b200.weights.safetensors_io import save_file
    from tests.plain.qwen3_plain import read_safetensors
    cfg = drawn_fomanex(seed)
    write_model_dir(FomanexConfig.from_json(cfg), out_dir, seed=seed, dtype=torch.bfloat16)
    path = os.path.join(out_dir, "model.safetensors")
    W = read_safetensors(path)
    for name in W:
        if name.endswith(".mix"):
            W[name] = (W[name].float() / W[name].float().sum(0, keepdim=True)).bfloat16()
    save_file({k: (v.bfloat16() if v.is_floating_point() else v) for k, v in W.items()}, path)      # stored as written: bfloat16
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        c = json.loads(json.dumps(cfg))
        for l in c["layers"]:
            l["mixer"].pop("decay_rank", None)
        json.dump(c, f)
    return out_dir
