"""Fomanex: a decoder whose layers are listed one by one in config.json and whose residual stream is kept in several
copies joined to the sublayers by hyper-connections.  The embedded tokens are scaled and pass a norm; every norm of the
model is a dynamic tanh (tanh(alpha x) * w + b, no statistics).  A layer is a pre-norm mixer and an optional pre-norm
feed-forward, each multiplied element by element by a learned layer scale and by ``residual_mult`` on its way into the
streams.  Two mixers: latent attention (queries straight from the input, a cached key/value latent with a rotated key
part shared by the heads, rotate-half rotation with frequencies stretched for long contexts, a sink in the softmax) and
"wkv" time mixing with a matrix state per head.  Two feed-forwards: a dense gated one with the tanh form of gelu, and a
mixture of experts with sigmoid scores, a correction added for the choice alone, and weights that are not renormalised.
A stretch of layers may run several times in a row with the same weights and a cache or state of its own for every
pass.  The logits are the embedding table applied to the normed sum of the streams, scaled and capped by a tanh.

config.json keys: ``architecture`` "Fomanex"; ``vocab``; ``width``; ``norm.eps``; ``embedding.scale``; ``residual_mult``;
``streams`` (absent: one stream and the plain residual sum, no hyper-connection tensors); ``logit_scale``;
``logit_softcap`` (absent or 0: none); ``loop`` {start, stop, times} (absent: every layer once); ``layers``: a list of
``{"type", "mixer", "mlp"}`` where ``type`` is "latent_attention" (mixer: heads, dim, rot_dim, vdim, kv_rank, scale, rot.dims,
rot.base, rot.scaling {factor, original, fast, slow}) or "wkv" (heads, dim), and ``mlp`` is ``{"kind": "dense", "ff"}``,
``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"}}`` or null.  Tensor names: ``embed``, ``embed.norm``
(+ ``.b``, ``.alpha``), ``final.norm``, and per layer ``l<i>.`` + norm1, norm2, ls1, ls2, hc1.in|out|mix, hc2.*, ``mix.*``,
``mlp.gate|up|down`` or ``mlp.router``, ``mlp.correction``, ``mlp.e<j>.gate|up|down``.

Two optional keys are this engine's own: ``max_positions`` (longest sequence; default 1,048,576) and, in a "wkv" mixer,
``decay_rank`` (the inner size of the decay's low-rank projection, which a stored model gives by its tensors' shapes;
the random-weights mode needs it written down).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Mapping, Optional, Tuple

from .registry import register_architecture
from .spec import (ConfigError, DynamicTanhSpec, GatedMLPSpec, HyperConnectionSpec, LatentAttentionSpec, LayerSpec, ModelSpec,
                   NoPositionSpec, RotarySpec, RoutedMLPSpec, ScheduleEntry, TimeMixSpec)
from .zufusun import _float, _int, _need

MIXERS = ("latent_attention", "wkv")


@dataclass(frozen=True)
class FomanexConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    streams: int                        # 0: the key is absent (one stream, no hyper-connection tensors)
    logit_scale: float
    logit_softcap: float
    loop: Optional[Tuple[int, int, int]]          # (start, stop, times) or None
    layers: Tuple[dict, ...]            # as config.json lists them (checked)
    max_positions: int = 1 << 20

    architecture = "Fomanex"
    model_type = "fomanex"

    @classmethod
    def from_json(cls, config: Mapping, generation_config: Optional[Mapping] = None) -> "FomanexConfig":
        layers = _need(config, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        loop = None
        if config.get("loop") is not None:
            lp = config["loop"]
            loop = (_int(lp, "start", "loop", least=0), _int(lp, "stop", "loop", least=0), _int(lp, "times", "loop", least=1))
            if not loop[0] <= loop[1] <= len(layers):
                raise ConfigError(f"config.json: loop {loop[0]}..{loop[1]} does not lie within the {len(layers)} layers")
        out = cls(vocab=_int(config, "vocab", "the model"), width=_int(config, "width", "the model"),
                  eps=_float(_need(config, "norm", "the model"), "eps", "norm"),
                  embedding_scale=_float(config["embedding"], "scale", "embedding") if config.get("embedding") is not None else 1.0,
                  residual_mult=_float(config, "residual_mult", "the model") if config.get("residual_mult") is not None else 1.0,
                  streams=_int(config, "streams", "the model") if config.get("streams") is not None else 0,
                  logit_scale=_float(config, "logit_scale", "the model") if config.get("logit_scale") is not None else 1.0,
                  logit_softcap=_float(config, "logit_softcap", "the model") if config.get("logit_softcap") is not None else 0.0,
                  loop=loop, layers=tuple(copy.deepcopy(dict(l)) for l in layers),
                  max_positions=int(config.get("max_positions") or (1 << 20)))
        if out.logit_softcap < 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        # every layer's keys are read and every part is built (without a device) now, so that a bad value is
        # refused here and not at the first step
        from ..model.causal_lm import CausalLM
        CausalLM(out.to_model_spec())
        return out

    # ------------------------------------------------------------------ parts
    def _norm(self) -> DynamicTanhSpec:
        return DynamicTanhSpec(size=self.width, weight_suffix="", bias_suffix=".b", alpha_suffix=".alpha")

    def _mixer(self, i: int, kind: str, m: Mapping):
        where = f"layers[{i}].mixer"
        if kind == "latent_attention":
            rot_dim = _int(m, "rot_dim", where, least=0)
            position = NoPositionSpec()
            if rot_dim:
                rot = _need(m, "rot", where)
                sc = rot.get("scaling")
                scaling = {}
                if sc is not None:
                    w = where + ".rot.scaling"
                    scaling = dict(scaling_factor=_float(sc, "factor", w), scaling_original=_float(sc, "original", w),
                                   scaling_fast=_float(sc, "fast", w), scaling_slow=_float(sc, "slow", w))
                position = RotarySpec(head_dim=rot_dim, rotary_dim=_int(rot, "dims", where + ".rot"),
                                      theta=_float(rot, "base", where + ".rot"), frequency_precision="float64", layout="half",
                                      **scaling)
            return LatentAttentionSpec(hidden_size=self.width, num_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                                       rot_dim=rot_dim, value_dim=_int(m, "vdim", where), q_rank=0,
                                       kv_rank=_int(m, "kv_rank", where), scale=_float(m, "scale", where), norm_eps=self.eps,
                                       sink=True, gate=False, own_kv=True, position=position)
        if kind == "wkv":
            return TimeMixSpec(hidden_size=self.width, num_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                               decay_rank=int(m.get("decay_rank") or 0), norm_eps=self.eps)
        raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this design ({', '.join(MIXERS)})")

    def _feed_forward(self, i: int, mlp: Mapping):
        where = f"layers[{i}].mlp"
        kind = mlp.get("kind")
        if kind == "dense":
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=_int(mlp, "ff", where), activation="gelu_tanh",
                                names=("gate", "up", "down"))
        if kind == "moe":
            expert, router = _need(mlp, "expert", where), _need(mlp, "router", where)
            return RoutedMLPSpec(hidden_size=self.width, intermediate_size=_int(expert, "ff", where + ".expert"),
                                 experts=_int(router, "experts", where + ".router"), top=_int(router, "top", where + ".router"),
                                 limit=0.0, alpha=1.0, up_offset=0.0, scoring="sigmoid", correction=True,
                                 route_scale=_float(router, "scale", where + ".router") if router.get("scale") is not None else 1.0,
                                 renormalize=False)
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design (dense, moe)")

    def _connection(self, sublayer: int) -> HyperConnectionSpec:
        return HyperConnectionSpec(size=self.width, streams=max(self.streams, 1), multiplier=self.residual_mult, layer_scale=True,
                                   learned=self.streams > 0, name=f"hc{sublayer}", scale_name=f"ls{sublayer}")

    def order(self) -> Tuple[Tuple[int, int], ...]:
        """(layer, pass) in run order: the looped stretch runs ``times`` times in a row, then the rest follows."""
        n = len(self.layers)
        if self.loop is None:
            return tuple((i, 0) for i in range(n))
        a, b, times = self.loop
        return (tuple((i, 0) for i in range(a)) + tuple((i, t) for t in range(times) for i in range(a, b))
                + tuple((i, 0) for i in range(b, n)))

    # --------------------------------------------------------------- as a model
    def to_model_spec(self) -> ModelSpec:
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            kind, m = _need(l, "type", f"layers[{i}]"), _need(l, "mixer", f"layers[{i}]")
            parts = [("mixer_norm", self._norm(), p + "norm1"), ("mixer", self._mixer(i, kind, m), p + "mix."),
                     ("mixer_connection", self._connection(1), p)]
            if l.get("mlp") is not None:
                parts += [("feed_forward_norm", self._norm(), p + "norm2"), ("feed_forward", self._feed_forward(i, l["mlp"]), p + "mlp."),
                          ("feed_forward_connection", self._connection(2), p)]
            layers.append(LayerSpec("connected_prenorm", tuple(parts)))
        schedule = tuple(ScheduleEntry(i, instance=t) for i, t in self.order())
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers),
                         schedule=schedule, final_norm=self._norm(), final_norm_prefix="final.norm",
                         embedding_name="embed", head_name="head", tie_embeddings=True, head_optional=True,
                         max_positions=self.max_positions, eos_ids=(), init_std=0.05, init_norm_std=0.1,
                         embedding_multiplier=self.embedding_scale, logit_scale=self.logit_scale,
                         embedding_norm=self._norm(), embedding_norm_prefix="embed.norm",
                         logit_softcap=self.logit_softcap, residual_streams=max(self.streams, 1))

    def to_json(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
             "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap,
             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.streams:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    def _needs(self):
        from ..model.causal_lm import CausalLM
        return CausalLM(self.to_model_spec()).cache_needs()

    def kv_bytes_per_token(self, elem_bytes: int) -> int:
        """Bytes of paged cache one token takes: one latent row per run of every latent layer."""
        return sum(n.num_kv_heads * (n.head_dim + (0 if n.keys_only else (n.value_dim or n.head_dim))) * elem_bytes
                   for n in self._needs().values() if n is not None and n.kind in ("full", "window"))

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size fp32 state one request holds (the matrices and last inputs of the time-mixing layers, once
        per run)."""
        from ..cache.storage import state_bytes_per_request
        return state_bytes_per_request(self._needs())

    def describe(self) -> str:
        kinds = ", ".join(l["type"] for l in self.layers[:8]) + (", ..." if len(self.layers) > 8 else "")
        loop = f", layers {self.loop[0]}..{self.loop[1] - 1} x {self.loop[2]}" if self.loop else ""
        return (f"fomanex: {len(self.layers)} layers ({kinds}){loop}, width {self.width}, {max(self.streams, 1)} streams, "
                f"vocab {self.vocab}")


register_architecture(FomanexConfig.architecture, FomanexConfig, model_type=FomanexConfig.model_type)
