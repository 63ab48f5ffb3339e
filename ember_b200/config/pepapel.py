"""Pepapel: a decoder whose layers are listed one by one in config.json, with the norm *after* the residual sum:
``x = norm1(alpha x + mixer(x)); x = norm2(alpha x + ff(x))``, layer norms with a weight and no bias, both sublayers
reading the stream itself.  Two mixers: "attention" (grouped-query softmax attention with an RMS norm per head on
queries and keys, no rotation, a query temperature that grows with the logarithm of the position, and a tanh cap on
the scores) and "parallel" (two mixers side by side whose results are each RMS-normed over the width and averaged:
left, attention inside chunks of positions with short convolutions on q, k, v, a norm over the whole query and key
projections, a linearly scaled rotate-half rotation and a sigmoid gate per head; right, a gated delta rule with one decay
per head, short convolutions, and a silu output gate).  Two feed-forwards: a dense one with biases and a clamped
activation, and a mixture of experts (softmax scores over all router outputs, a correction for the choice alone, a limit
to the best groups of neighbouring outputs, weights not renormalised, identity experts without tensors, experts
``W_down relu(W_up h)^2``).  The embedded tokens are scaled; the logits are ``head`` applied to the normed stream.

config.json keys: ``architecture`` "Pepapel"; ``vocab``; ``width``; ``norm.eps``; ``embedding.scale``; ``postln_alpha``;
``layers``: a list of ``{"type", "mixer", "mlp"}`` where ``type`` is "attention" (mixer: heads, kv_heads, dim, vdim, scale,
softcap, q_temp {coef, every}; the last two optional) or "parallel" (left: heads, kv_heads, dim, vdim, scale, conv,
mask.size, rot {dims, base, scaling.factor}; right: heads, kv_heads, dim, vdim, conv), and ``mlp`` is
``{"kind": "dense", "ff", "limit"}``, ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity",
"groups": {"count", "keep"}}}`` or null.  Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.`` + norm1,
norm2, ``mix.*``, ``mlp.gate|up|down`` (+ ``.b``) or ``mlp.router``, ``mlp.correction``, ``mlp.e<j>.up|down``.

One optional key is this engine's own: ``max_positions`` (longest sequence; default 1,048,576).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Mapping, Optional, Tuple

from .registry import register_architecture
from .spec import (ConfigError, GatedDeltaSpec, GatedMLPSpec, LayerNormSpec, LayerSpec, ModelSpec, NoPositionSpec,
                   ParallelMixerSpec, RotarySpec, RoutedMLPSpec, SinkAttentionSpec, default_schedule)


def _need(d: Mapping, key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _int(d: Mapping, key: str, where: str, least: int = 1) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {least}, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


MIXERS = ("attention", "parallel")
DELTA_KEY_EPS = 1e-6         # inside the root of the unit norm of the delta rule's q and k: fixed by the design
SWISH_ALPHA = 1.702          # g sigmoid(alpha g) of the dense feed-forward: fixed by the design


@dataclass(frozen=True)
class PepapelConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    alpha: float
    layers: Tuple[dict, ...]            # as config.json lists them (checked)
    max_positions: int = 1 << 20

    architecture = "Pepapel"
    model_type = "pepapel"

    @classmethod
    def from_json(cls, config: Mapping, generation_config: Optional[Mapping] = None) -> "PepapelConfig":
        layers = _need(config, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        emb = config.get("embedding")
        out = cls(vocab=_int(config, "vocab", "the model"), width=_int(config, "width", "the model"),
                  eps=_float(_need(config, "norm", "the model"), "eps", "norm"),
                  embedding_scale=_float(emb, "scale", "embedding") if emb is not None else 1.0,
                  alpha=_float(config, "postln_alpha", "the model") if config.get("postln_alpha") is not None else 1.0,
                  layers=tuple(copy.deepcopy(dict(l)) for l in layers),
                  max_positions=int(config.get("max_positions") or (1 << 20)))
        # every layer's keys are read and every part is built (without a device) now, so that a bad value is
        # refused here and not at the first step
        from ..model.causal_lm import CausalLM
        CausalLM(out.to_model_spec())
        return out

    # ------------------------------------------------------------------ mixers
    def _attention(self, m: Mapping, where: str) -> SinkAttentionSpec:
        """Softmax attention over all earlier positions: a norm per head, no rotation, optional temperature and cap."""
        temp = m.get("q_temp")
        return SinkAttentionSpec(
            hidden_size=self.width, num_heads=_int(m, "heads", where), num_kv_heads=_int(m, "kv_heads", where),
            head_dim=_int(m, "dim", where), value_dim=_int(m, "vdim", where), scale=_float(m, "scale", where),
            bias=False, qk_norm="head", qk_norm_eps=self.eps, sink=False,
            q_temp_coef=_float(temp, "coef", where + ".q_temp") if temp is not None else 0.0,
            q_temp_every=_int(temp, "every", where + ".q_temp") if temp is not None else 0,
            softcap=_float(m, "softcap", where) if m.get("softcap") is not None else 0.0)

    def _chunked_attention(self, m: Mapping, where: str) -> SinkAttentionSpec:
        """The left half of a parallel layer: attention inside chunks, convolutions, whole-projection norms, a rotation,
        a gate per head."""
        dim = _int(m, "dim", where)
        position = NoPositionSpec()
        rot = m.get("rot")
        if rot is not None:
            scaling = rot.get("scaling")
            position = RotarySpec(head_dim=dim, rotary_dim=_int(rot, "dims", where + ".rot"), theta=_float(rot, "base", where + ".rot"),
                                  frequency_precision="float64", layout="half",
                                  linear_factor=_float(scaling, "factor", where + ".rot.scaling") if scaling is not None else 1.0)
        mask = m.get("mask")
        return SinkAttentionSpec(
            hidden_size=self.width, num_heads=_int(m, "heads", where), num_kv_heads=_int(m, "kv_heads", where), head_dim=dim,
            value_dim=_int(m, "vdim", where), scale=_float(m, "scale", where), bias=False, qk_norm="whole", qk_norm_eps=self.eps,
            sink=False, conv_taps=_int(m, "conv", where) if m.get("conv") is not None else 0, position=position,
            chunk=_int(mask, "size", where + ".mask") if mask is not None else 0, head_gate=True)

    def _delta(self, m: Mapping, where: str) -> GatedDeltaSpec:
        return GatedDeltaSpec(hidden_size=self.width, num_heads=_int(m, "heads", where), num_kv_heads=_int(m, "kv_heads", where),
                              head_dim=_int(m, "dim", where), value_dim=_int(m, "vdim", where), conv_taps=_int(m, "conv", where),
                              norm_eps=self.eps, key_eps=DELTA_KEY_EPS, decay="head", gate="silu")

    def _mixer(self, i: int, kind: str, m: Mapping):
        where = f"layers[{i}].mixer"
        if kind == "attention":
            return self._attention(m, where)
        if kind == "parallel":
            return ParallelMixerSpec(hidden_size=self.width, left=self._chunked_attention(_need(m, "left", where), where + ".left"),
                                     right=self._delta(_need(m, "right", where), where + ".right"), left_scale=0.5, right_scale=0.5,
                                     branch_norm=True, norm_eps=self.eps)
        raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this design ({', '.join(MIXERS)})")

    def _feed_forward(self, i: int, mlp: Mapping):
        where = f"layers[{i}].mlp"
        kind = mlp.get("kind")
        if kind == "dense":
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=_int(mlp, "ff", where), activation="clamped_swish",
                                names=("gate", "up", "down"), limit=_float(mlp, "limit", where), alpha=SWISH_ALPHA, up_offset=1.0,
                                bias=True, bias_suffix=".b")
        if kind == "moe":
            router = _need(mlp, "router", where)
            groups = router.get("groups")
            return RoutedMLPSpec(hidden_size=self.width, intermediate_size=_int(_need(mlp, "expert", where), "ff", where + ".expert"),
                                 experts=_int(router, "experts", where + ".router"), top=_int(router, "top", where + ".router"),
                                 limit=0.0, scoring="softmax", correction=True, route_scale=1.0, renormalize=False,
                                 groups=_int(groups, "count", where + ".router.groups") if groups is not None else 0,
                                 keep_groups=_int(groups, "keep", where + ".router.groups") if groups is not None else 0,
                                 identity=_int(router, "identity", where + ".router", least=0) if router.get("identity") is not None else 0,
                                 expert="square_relu")
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design (dense, moe)")

    # --------------------------------------------------------------- as a model
    def _norm(self) -> LayerNormSpec:
        return LayerNormSpec(size=self.width, eps=self.eps, weight_suffix="", bias=False)

    def to_model_spec(self) -> ModelSpec:
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            parts = [("mixer", self._mixer(i, _need(l, "type", f"layers[{i}]"), _need(l, "mixer", f"layers[{i}]")), p + "mix."),
                     ("mixer_norm", self._norm(), p + "norm1")]
            mlp = l.get("mlp")
            if mlp is not None:
                parts += [("feed_forward", self._feed_forward(i, mlp), p + "mlp."), ("feed_forward_norm", self._norm(), p + "norm2")]
            layers.append(LayerSpec("postnorm", tuple(parts), constants=(("alpha", self.alpha),)))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers),
                         schedule=default_schedule(len(layers)), final_norm=self._norm(), final_norm_prefix="final.norm",
                         embedding_name="embed", head_name="head", tie_embeddings=False, head_optional=False,
                         max_positions=self.max_positions, eos_ids=(), init_std=0.05, init_norm_std=0.1,
                         embedding_multiplier=self.embedding_scale)

    def to_json(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embedding_scale}, "postln_alpha": self.alpha,
             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    def _needs(self):
        from ..model.causal_lm import CausalLM
        return CausalLM(self.to_model_spec()).cache_needs()

    def kv_bytes_per_token(self, elem_bytes: int) -> int:
        """Bytes of paged cache one token takes: keys and values of every attention layer and every left half."""
        return sum(n.num_kv_heads * (n.head_dim + (0 if n.keys_only else (n.value_dim or n.head_dim))) * elem_bytes
                   for n in self._needs().values() if n is not None and n.kind in ("full", "window"))

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size fp32 state one request holds: the delta rule's matrices and the convolutions' last inputs."""
        from ..cache.storage import state_bytes_per_request
        return state_bytes_per_request(self._needs())

    def describe(self) -> str:
        kinds = ", ".join(l["type"] for l in self.layers[:8]) + (", ..." if len(self.layers) > 8 else "")
        return f"pepapel: {len(self.layers)} layers ({kinds}), width {self.width}, vocab {self.vocab}"


register_architecture(PepapelConfig.architecture, PepapelConfig, model_type=PepapelConfig.model_type)
