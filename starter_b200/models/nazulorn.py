"""Nazulorn ("Nazulorn"): configuration, layer arrangement, tensor names.

A small decoder whose residual is kept in several 32-bit streams: every branch reads a learned blend of the streams
through an RMS norm and returns to all of them through a learned matrix and a learned vector, scaled by
``residual_mult``.  Two kinds of mixer: sliding-window grouped-query attention with two score maps per head
("attention": partly rotated heads, frequencies stretched by wavelength, a head-wise unit norm of the maps'
difference) and gated linear attention with a matrix state per head ("gla").  The feed-forward is a mixture of
experts with identity experts and a shared expert.  The embedding is scaled, and so are the logits of the untied head.

config.json: ``vocab``, ``width``, ``norm`` {``eps``}, ``embedding`` {``scale``}, ``residual_mult``, ``streams``,
``logit_scale`` and ``layers``, a list of {``type``, ``mixer`` {sizes and constants of that mixer},
``mlp`` {``kind`` "moe", ``router`` {``experts``, ``identity``, ``top``, ``scale``}, ``expert`` {``ff``, ``limit``},
``shared`` {``ff``, ``limit``} or nothing} or null}.  Tensors: ``embed``, ``head``, ``final.norm`` and per layer
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc1.{in,out,mix}``, ``l<i>.hc2.{in,out,mix}``, ``l<i>.mix.*``, ``l<i>.mlp.*``.

The constant the design fixes: the experts' sigmoid factor 1.702.  The one size that config.json does not give, the
inner size of a gla mixer's two decay matrices, is read from the shape of ``l<i>.mix.a1``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..config.registry import ConfigError, ModelConfig, TensorNames, register_architecture
from ..config.specs import (DiffAttentionSpec, GatedMLPSpec, GLASpec, GroupedNormSpec, ModelSpec, MoESpec, ScaledHalfRopeSpec,
                            StreamBlockSpec, StreamNormSpec)

SWISH_ALPHA = 1.702     # g * sigmoid(1.702 g)
MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "diff"),
    "gla": ("heads", "dim", "vdim", "tau"),
}
COUNTS = ("heads", "kv_heads", "dim", "vdim")


def _need(where: str, raw, keys) -> None:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in raw]
    if missing:
        raise ConfigError(f"config.json: {where} lacks " + ", ".join(missing))


def _count(where: str, value, least: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where} must be an integer of at least {least}, got {value!r}")
    return value


@dataclass(frozen=True)
class NazulornConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    streams: int                         # 0: one plain residual
    logit_scale: float
    layers: Tuple[Any, ...]              # the layer entries as read (plain data)

    architecture = "Nazulorn"

    @classmethod
    def from_dict(cls, raw: dict) -> "NazulornConfig":
        _need("the configuration", raw, ("vocab", "width", "norm", "layers"))
        _need("norm", raw["norm"], ("eps",))
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            _need(f"layers[{i}]", entry, ("type", "mixer"))
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is unknown; known: " + ", ".join(sorted(MIXER_KEYS)))
            m = entry["mixer"]
            _need(f"layers[{i}].mixer", m, MIXER_KEYS[kind])
            for key in MIXER_KEYS[kind]:
                if key in COUNTS:
                    _count(f"layers[{i}].mixer.{key}", m[key])
            if kind == "attention":
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: layers[{i}]: {m['heads']} heads cannot share {m['kv_heads']} kv_heads evenly")
                if m.get("mask") is not None:
                    _need(f"layers[{i}].mixer.mask", m["mask"], ("size",))
                    _count(f"layers[{i}].mixer.mask.size", m["mask"]["size"])
                rot = m.get("rot")
                if rot is not None:
                    _need(f"layers[{i}].mixer.rot", rot, ("base", "dims"))
                    dims = rot["dims"]
                    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 2 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"config.json: layers[{i}] rotates {dims!r} of {m['dim']} columns; the rotation covers "
                                          "an even number of a map's first columns")
                    if rot.get("scaling") is not None:
                        _need(f"layers[{i}].mixer.rot.scaling", rot["scaling"], ("factor", "original", "fast", "slow"))
            elif not float(m["tau"]) > 0:
                raise ConfigError(f"config.json: layers[{i}].mixer.tau must be positive")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(f"layers[{i}].mlp", mlp, ("kind", "router", "expert"))
                if mlp["kind"] != "moe":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp['kind']!r} is not built: only 'moe' is")
                _need(f"layers[{i}].mlp.router", mlp["router"], ("experts", "top"))
                r = mlp["router"]
                _count(f"layers[{i}].mlp.router.experts", r["experts"], 0)
                _count(f"layers[{i}].mlp.router.identity", r.get("identity", 0), 0)
                _count(f"layers[{i}].mlp.router.top", r["top"])
                if r["top"] > r["experts"] + r.get("identity", 0):
                    raise ConfigError(f"config.json: layers[{i}].mlp.router chooses {r['top']} of {r['experts'] + r.get('identity', 0)}")
                for part in ("expert", "shared"):
                    if mlp.get(part) is not None:
                        _need(f"layers[{i}].mlp.{part}", mlp[part], ("ff", "limit"))
                        _count(f"layers[{i}].mlp.{part}.ff", mlp[part]["ff"])
            layers.append(copy.deepcopy(entry))
        streams = raw.get("streams")
        return cls(vocab=_count("vocab", raw["vocab"]), width=_count("width", raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                   residual_mult=float(raw.get("residual_mult", 1.0)),
                   streams=0 if streams is None else _count("streams", streams),
                   logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(layers))

    # ---- layers -------------------------------------------------------------------------

    def with_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "NazulornConfig":
        """The configuration with the one size that only a tensor's shape gives: the inner size of a gla mixer's decay
        matrices, ``l<i>.mix.a1`` [rank, width].  A mixer entry may also name it itself (``decay_rank``; a configuration
        made for random weights has no shapes to read)."""
        layers = copy.deepcopy(list(self.layers))
        for i, entry in enumerate(layers):
            name = f"l{i}.mix.a1"
            if entry["type"] == "gla" and name in shapes and "decay_rank" not in entry["mixer"]:
                entry["mixer"]["decay_rank"] = int(shapes[name][0])
        return NazulornConfig(self.vocab, self.width, self.norm_eps, self.embedding_scale, self.residual_mult, self.streams,
                              self.logit_scale, tuple(layers))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": copy.deepcopy(list(self.layers)), "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.streams:
            out["streams"] = self.streams
        return out

    def _mixer_spec(self, i: int):
        m, kind = self.layers[i]["mixer"], self.layers[i]["type"]
        if kind == "gla":
            rank = int(m.get("decay_rank") or 0)
            if rank <= 0:
                raise ConfigError(f"layers[{i}]: the inner size of the decay matrices comes from the shape of l{i}.mix.a1; "
                                  "give the configuration the checkpoint's shapes first (with_shapes)")
            return GLASpec(hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], v_dim=m["vdim"], tau=float(m["tau"]),
                           decay_rank=rank, norm_eps=self.norm_eps)
        position = None
        rot = m.get("rot")
        if rot is not None:
            sc = rot.get("scaling") or {}
            position = ScaledHalfRopeSpec(theta=float(rot["base"]), rotary_dim=int(rot["dims"]),
                                          factor=float(sc["factor"]) if sc else None,
                                          original=float(sc["original"]) if sc else None,
                                          fast=float(sc["fast"]) if sc else None, slow=float(sc["slow"]) if sc else None)
        mask = m.get("mask")
        return DiffAttentionSpec(hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                 v_dim=m["vdim"], scale=float(m["scale"]), diff=float(m["diff"]), norm_eps=self.norm_eps,
                                 window=int(mask["size"]) if mask is not None else None, position=position)

    def _ff_spec(self, i: int) -> Optional[MoESpec]:
        mlp = self.layers[i].get("mlp")
        if mlp is None:
            return None

        def gated(part):
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=int(part["ff"]), activation="clamped_swish",
                                limit=float(part["limit"]), alpha=SWISH_ALPHA)

        r = mlp["router"]
        return MoESpec(hidden_size=self.width, n_experts=int(r["experts"]), n_identity=int(r.get("identity", 0)), top=int(r["top"]),
                       route_scale=float(r.get("scale", 1.0)), expert=gated(mlp["expert"]),
                       shared=gated(mlp["shared"]) if mlp.get("shared") is not None else None)

    def model_spec(self) -> ModelSpec:
        norm = StreamNormSpec(size=self.width, eps=self.norm_eps, streams=self.streams, mult=self.residual_mult)
        blocks = []
        for i in range(len(self.layers)):
            ff = self._ff_spec(i)
            blocks.append(StreamBlockSpec(mixer_norm=norm, mixer=self._mixer_spec(i), ff_norm=norm if ff is not None else None, ff=ff))
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=tuple(blocks),
                         final_norm=GroupedNormSpec(size=self.width, eps=self.norm_eps, groups=1), tie_embeddings=False,
                         embedding_scale=self.embedding_scale, logit_scale=self.logit_scale, residual_float32=True,
                         streams=max(self.streams, 1))

    def tensor_names(self) -> TensorNames:
        layers = []
        for i, entry in enumerate(self.layers):
            p = f"l{i}."

            def norm(q):
                names = {"weight": p + "norm" + q}
                if self.streams:
                    names.update({r: p + f"hc{q}." + r for r in ("in", "out", "mix")})
                return names

            if entry["type"] == "gla":
                mixer = {r: r for r in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
                mixer["a2_bias"] = "a2.b"
            else:
                mixer = {r: r for r in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")}
            names = {"mixer_norm": norm("1"), "mixer": {role: p + "mix." + n for role, n in mixer.items()}}
            mlp = entry.get("mlp")
            if mlp is not None:
                ff = {"router": "router", "correction": "correction"}
                for e in range(int(mlp["router"]["experts"])):
                    ff.update({f"e{e}_{r}": f"e{e}.{r}" for r in ("gate", "up", "down")})
                if mlp.get("shared") is not None:
                    ff.update({"shared_" + r: "shared." + r for r in ("gate", "up", "down")})
                names["ff_norm"] = norm("2")
                names["ff"] = {role: p + "mlp." + n for role, n in ff.items()}
            layers.append(names)
        return TensorNames(embedding="embed", lm_head="head", final_norm={"weight": "final.norm"}, layers=layers)

    def random_init(self, name: str, shape) -> Tuple[float, float]:
        """(mean, standard deviation) of a tensor's seeded random fill: matrices so that a product keeps its input's
        size, stream weights near a plain residual, decays neither instant nor absent, a router that spreads."""
        last = name.rsplit(".", 1)[-1]
        if ".hc" in name:
            return (0.6, 0.3) if last in ("in", "out") else (0.5, 0.3)
        if last in ("lq1", "lk1", "lq2", "lk2"):
            return 0.0, 0.3
        if name.endswith("a2.b"):
            return 2.0, 1.5
        if last == "correction":
            return 0.0, 0.05
        if last == "router":
            return 0.0, 2.0 * float(shape[-1]) ** -0.5
        if len(shape) == 1:
            return 1.0, 0.1
        if name == "embed":
            return 0.0, 1.0
        return 0.0, float(shape[-1]) ** -0.5


register_architecture(NazulornConfig.architecture, NazulornConfig)
