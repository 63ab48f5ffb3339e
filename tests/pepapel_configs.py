"""The tests' own small Pepapel configurations.  They differ from one another in every size, in the order and number of
layers, in the constants, in which optional keys are there, and in which values happen to be equal (key and value
sizes, heads and key heads, experts and choices, groups and kept groups) or 1."""
from __future__ import annotations

import json
import os

import torch


def _attention(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _left(heads, kv_heads, dim, vdim, scale, conv, chunk, rot_dims, base, factor=None):
    rot = {"dims": rot_dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv, "mask": {"size": chunk},
            "rot": rot}


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top, identity=None, groups=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _parallel(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


PEPAPEL = {
    # widths the tensor-core kernels take; chunks of 40 (not a multiple of a page of 16), a partial rotation, a
    # temperature that changes every 24 positions, values wider than keys, identity experts, three groups of which two stay;
    # the last layer's keys and values are both 64 wide (in bfloat16 it runs on the kernels Qwen3's attention uses)
    "a": dict(seed=3, json={
        "architecture": "Pepapel", "vocab": 320, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "postln_alpha": 1.7,
        "layers": [
            _parallel(_left(4, 2, 32, 16, 0.18, 3, 40, 16, 10000.0, 4.0), _right(4, 2, 16, 32, 2), _dense(96, 1.2)),
            {"type": "attention", "mixer": _attention(4, 1, 32, 48, 0.2, softcap=20.0, q_temp=(0.4, 24)), "mlp": _moe(48, 4, 2, identity=2, groups=(3, 2))},
            _parallel(_left(2, 2, 64, 64, 0.125, 4, 33, 64, 500.0), _right(2, 1, 32, 64, 4), _moe(32, 6, 3, groups=(2, 1))),
            {"type": "attention", "mixer": _attention(4, 2, 64, 64, 0.15, softcap=6.0), "mlp": None},
        ]}),
    # a width no tensor-core product takes; odd head sizes; one head; a convolution of one tap (no carried rows) and one
    # of five; a chunk of one page exactly; as many choices as router outputs; a single choice; a cap that binds; no
    # embedding scale and no alpha in the file
    "b": dict(seed=7, json={
        "architecture": "Pepapel", "vocab": 257, "width": 100, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "attention", "mixer": _attention(1, 1, 40, 24, 0.16, softcap=2.0), "mlp": _dense(70, 0.4)},
            _parallel(_left(3, 1, 20, 28, 0.22, 1, 16, 8, 77.0, 2.5), _right(3, 3, 24, 12, 5), _moe(30, 2, 3, identity=1)),
            _parallel(_left(6, 3, 12, 12, 0.3, 5, 70, 12, 1e6), _right(1, 1, 72, 40, 3), _moe(50, 5, 1, identity=0, groups=(5, 5))),
            {"type": "attention", "mixer": _attention(5, 5, 24, 8, 0.2, q_temp=(1.5, 1)), "mlp": _moe(20, 3, 2, identity=5, groups=(4, 3))},
        ]}),
    # head sizes of a real model's layers: 128-wide keys and values, eight query heads on one key head, a delta rule of
    # 128 x 128, chunks of 256, experts of 256; only parallel layers and one attention layer at the start
    "c": dict(seed=11, json={
        "architecture": "Pepapel", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0}, "postln_alpha": 3.0,
        "layers": [
            {"type": "attention", "mixer": _attention(8, 1, 128, 128, 0.0884, softcap=30.0, q_temp=(0.1, 256)), "mlp": _moe(256, 8, 2, identity=8, groups=(4, 2))},
            _parallel(_left(4, 2, 128, 128, 0.0884, 4, 256, 64, 10000.0, 8.0), _right(2, 1, 128, 128, 4), _dense(512, 7.0)),
            _parallel(_left(2, 1, 64, 128, 0.125, 2, 100, 32, 50000.0, 1.0), _right(4, 4, 64, 64, 4), None),
        ]}),
}


def pepapel_config(name: str):
    from ember_b200.config import PepapelConfig
    return PepapelConfig.from_json(PEPAPEL[name]["json"])


def write_pepapel_dir(name_or_json, out_dir: str, seed: int = 0, spread_router: float = 6.0) -> str:
    """A model folder with random weights.  The router matrices are scaled up so that the softmax over the router's
    outputs is far from uniform and a choice is seldom a close call between two scores."""
    from ember_b200.config import PepapelConfig
    from ember_b200.weights import write_model_dir
    from ember_b200.weights.safetensors_io import save_file
    from tests.plain.qwen3_plain import read_safetensors
    cfg_json = PEPAPEL[name_or_json]["json"] if isinstance(name_or_json, str) else name_or_json
    seed = PEPAPEL[name_or_json]["seed"] if isinstance(name_or_json, str) else seed
    write_model_dir(PepapelConfig.from_json(cfg_json), out_dir, seed=seed, dtype=torch.bfloat16)
    path = os.path.join(out_dir, "model.safetensors")
    W = read_safetensors(path)
    g = torch.Generator().manual_seed(seed + 1)
    for name in W:
        if name.endswith(".router"):
            W[name] = (W[name].float() * spread_router).bfloat16()
        if name.endswith(".b") and W[name].dim() == 1:                       # biases that are not zero
            W[name] = (0.2 * torch.randn(W[name].shape, generator=g)).bfloat16()
    save_file({k: (v.bfloat16() if v.is_floating_point() else v) for k, v in W.items()}, path)
    with open(os.path.join(out_dir, "config.json"), "w") as f:        # the keys exactly as the test wrote them
        json.dump(cfg_json, f)
    return out_dir


def plain_inputs(model_dir: str):
    """(config dictionary, name -> float64 tensor) as the plain implementation takes them."""
    from tests.plain.qwen3_plain import read_safetensors
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: (v.double() if v.is_floating_point() else v) for k, v in W.items()}


def drawn_pepapel(seed: int) -> dict:
    """A configuration drawn from a seed: 2 to 6 layers of either mixer in any order, any feed-forward or none, sizes
    and constants from short lists that include ones no tensor-core kernel takes and values that are equal or 1."""
    import numpy as np
    rng = np.random.default_rng(seed)
    pick = lambda *v: v[int(rng.integers(0, len(v)))]                         # noqa: E731
    width = pick(128, 192, 256, 136, 200, 64)
    layers = []
    for _ in range(int(rng.integers(2, 7))):
        k = rng.random()
        if k < 0.35:
            mlp = _dense(pick(64, 128, 200, 384), pick(0.5, 1.5, 7.0))
        elif k < 0.9:
            e, ident = pick(2, 4, 6, 8, 16, 33), pick(None, 0, 1, 2, 4)
            n = e + (ident or 0)
            counts = [c for c in (1, 2, 3, 4, 5, 8) if n % c == 0]
            groups = None
            if rng.random() < 0.7:
                c = counts[int(rng.integers(0, len(counts)))]
                groups = (c, int(rng.integers(1, c + 1)))
            most = n if groups is None else groups[1] * (n // groups[0])
            mlp = _moe(pick(32, 64, 96, 40), e, int(rng.integers(1, min(most, 6) + 1)), identity=ident, groups=groups)
        else:
            mlp = None
        if rng.random() < 0.4:
            kv = pick(1, 2, 3)
            dim = pick(16, 32, 64, 128, 24)
            mixer = _attention(kv * pick(1, 2, 4), kv, dim, pick(16, 32, 48, 64, dim), float(dim ** -0.5 * pick(1.0, 0.7)),
                               softcap=pick(None, 5.0, 30.0, 40.0), q_temp=pick(None, (0.6, 16), (0.2, 50), (1.0, 7)))
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        else:
            kv, dim = pick(1, 2), pick(16, 32, 48, 64, 20)
            rot_dims = pick(dim, dim // 2, 8, 4)
            rot_dims -= rot_dims % 2
            left = _left(kv * pick(1, 2, 3), kv, dim, pick(16, 32, 48, dim), float(dim ** -0.5), pick(1, 2, 3, 4), pick(16, 24, 50, 64, 96, 7),
                         rot_dims, pick(10000.0, 500.0, 1e6), pick(None, 1.0, 4.0, 8.0))
            rkv = pick(1, 2, 3)
            right = _right(rkv * pick(1, 2), rkv, pick(16, 32, 64, 24), pick(16, 32, 64, 40), pick(2, 3, 4))
            layers.append(_parallel(left, right, mlp))
    return {"architecture": "Pepapel", "vocab": pick(384, 512, 640, 333), "width": width, "norm": {"eps": pick(1e-5, 1e-6)},
            "embedding": {"scale": pick(1.0, 2.0, float(width ** 0.5))}, "postln_alpha": pick(1.0, 2.0, 0.8, 4.0), "layers": layers}
