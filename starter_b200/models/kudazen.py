"""Kudazen ("Kudazen"): configuration, layer arrangement, tensor names.

A small decoder of parallel layers (one grouped RMS norm per layer, read by the mixer and by the feed-forward;
x += mixer(n) + ff(n)) over three kinds of mixer: attention through low-rank latents with a sink in the softmax
("latent_attention"), a linear recurrence with a matrix state per head ("wkv"), and grouped-query attention inside
fixed chunks with a distance penalty ("attention").  The output head is the embedding table; the residual stream is
32-bit in every run.

config.json: ``vocab``, ``width``, ``norm`` {``eps``, ``groups``} and ``layers``, a list of
{``type``, ``mixer`` {sizes and constants of that mixer}, ``mlp`` {``kind`` "dense", ``ff``, ``limit``} or null,
optionally ``weights_of``: the index of the layer whose tensors this one runs with (its cache or state stays its
own)}.  Tensors: ``embed``, ``final.norm``, and per layer that owns weights ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.mlp.{gate,up,down}``.

Constants the design fixes: the penalty's slopes 2**(-8 (h + 1) / heads) and the feed-forward's sigmoid factor 1.702.
The rotation covers the first ``rot.dims`` columns of the rotated part (all of it in the models seen so far).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from ..config.registry import ConfigError, ModelConfig, TensorNames, register_architecture
from ..config.specs import (BiasedAttentionSpec, GatedMLPSpec, GroupedNormSpec, LatentAttentionSpec, ModelSpec, PairRopeSpec,
                            ParallelBlockSpec, WKVSpec)

SLOPE_LOG2 = 8.0        # slope_h = 2**(-8 (h + 1) / heads)
SWISH_ALPHA = 1.702     # g * sigmoid(1.702 g)
MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"),
    "wkv": ("heads", "dim"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "mask"),
}


def _need(where: str, raw: dict, keys) -> None:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in raw]
    if missing:
        raise ConfigError(f"config.json: {where} lacks " + ", ".join(missing))


def _count(where: str, value) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {where} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class KudazenConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[Any, ...]              # the layer entries as read (plain data), weights_of included

    architecture = "Kudazen"

    @classmethod
    def from_dict(cls, raw: dict) -> "KudazenConfig":
        _need("the configuration", raw, ("vocab", "width", "norm", "layers"))
        _need("norm", raw["norm"], ("eps", "groups"))
        width = _count("width", raw["width"])
        groups = _count("norm.groups", raw["norm"]["groups"])
        if width % groups:
            raise ConfigError(f"config.json: width {width} cannot be cut into {groups} equal groups")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            _need(f"layers[{i}]", entry, ("type", "mixer"))
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is unknown; known: " + ", ".join(sorted(MIXER_KEYS)))
            _need(f"layers[{i}].mixer", entry["mixer"], MIXER_KEYS[kind])
            m = entry["mixer"]
            for key in MIXER_KEYS[kind]:
                if key not in ("scale", "rot", "mask"):
                    _count(f"layers[{i}].mixer.{key}", m[key])
            if kind == "latent_attention":
                _need(f"layers[{i}].mixer.rot", m["rot"], ("base", "dims"))
                dims = m["rot"]["dims"]
                if isinstance(dims, bool) or not isinstance(dims, int) or dims < 2 or dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"config.json: layers[{i}] rotates {dims!r} of {m['rot_dim']} columns; the rotation "
                                      "covers an even number of the rotated part's first columns")
            if kind == "attention":
                _need(f"layers[{i}].mixer.mask", m["mask"], ("size",))
                _count(f"layers[{i}].mixer.mask.size", m["mask"]["size"])
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: layers[{i}]: {m['heads']} heads cannot share {m['kv_heads']} kv_heads evenly")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(f"layers[{i}].mlp", mlp, ("kind", "ff", "limit"))
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp['kind']!r} is not built: only 'dense' is")
                _count(f"layers[{i}].mlp.ff", mlp["ff"])
            owner = entry.get("weights_of")
            if owner is not None and (isinstance(owner, bool) or not isinstance(owner, int) or not 0 <= owner < len(raw["layers"])
                                      or owner == i):
                raise ConfigError(f"config.json: layers[{i}].weights_of must name another layer, got {owner!r}")
            layers.append(copy.deepcopy(entry))
        cfg = cls(vocab=_count("vocab", raw["vocab"]), width=width, norm_eps=float(raw["norm"]["eps"]), norm_groups=groups,
                  layers=tuple(layers))
        for i in range(len(layers)):
            j = cfg.owner(i)
            if layers[j]["type"] != layers[i]["type"]:
                raise ConfigError(f"config.json: layers[{i}] runs with the weights of layers[{j}], which is of another type")
        return cfg

    # ---- layers -------------------------------------------------------------------------

    def owner(self, i: int) -> int:
        """Index of the layer whose tensors layer i runs with."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError("config.json: weights_of runs in a circle")
            seen.add(i)
            i = self.layers[i]["weights_of"]
        return i

    def owners(self) -> List[int]:
        """The layers that hold tensors, in order."""
        return [i for i in range(len(self.layers)) if self.owner(i) == i]

    def with_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "KudazenConfig":
        """The configuration with the one size that only a tensor's shape gives: the inner size of a wkv mixer's
        decay matrices, ``l<i>.mix.w1`` [rank, width].  A mixer entry may also name it itself (``decay_rank``; a
        configuration made for random weights has no shapes to read)."""
        layers = copy.deepcopy(list(self.layers))
        for i, entry in enumerate(layers):
            name = f"l{self.owner(i)}.mix.w1"
            if entry["type"] == "wkv" and name in shapes and "decay_rank" not in entry["mixer"]:
                entry["mixer"]["decay_rank"] = int(shapes[name][0])
        return KudazenConfig(self.vocab, self.width, self.norm_eps, self.norm_groups, tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "vocab": self.vocab, "width": self.width}

    def _mixer_spec(self, i: int):
        entry = self.layers[i]
        m, kind = entry["mixer"], entry["type"]
        if kind == "latent_attention":
            return LatentAttentionSpec(
                hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
                q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=float(m["scale"]), norm_eps=self.norm_eps,
                position=PairRopeSpec(theta=float(m["rot"]["base"]), rotary_dim=int(m["rot"]["dims"])), sink=True)
        if kind == "wkv":
            rank = int(m.get("decay_rank") or self.layers[self.owner(i)]["mixer"].get("decay_rank") or 0)
            if rank <= 0:
                raise ConfigError(f"layers[{i}]: the inner size of the decay matrices comes from the shape of l{self.owner(i)}.mix.w1; "
                                  "give the configuration the checkpoint's shapes first (with_shapes)")
            return WKVSpec(hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], decay_rank=rank, norm_eps=self.norm_eps)
        return BiasedAttentionSpec(
            hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
            scale=float(m["scale"]), value_norm_eps=self.norm_eps, head_temperature=True, slope_log2=SLOPE_LOG2,
            chunk=int(m["mask"]["size"]))

    def model_spec(self) -> ModelSpec:
        norm = GroupedNormSpec(size=self.width, eps=self.norm_eps, groups=self.norm_groups)
        owners = self.owners()
        blocks = []
        for i in owners:
            mlp = self.layers[i].get("mlp")
            ff = None
            if mlp is not None:
                ff = GatedMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="clamped_swish",
                                  limit=float(mlp["limit"]), alpha=SWISH_ALPHA)
            blocks.append(ParallelBlockSpec(norm=norm, mixer=self._mixer_spec(i), ff=ff))
        where = {i: n for n, i in enumerate(owners)}
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=tuple(blocks), final_norm=norm,
                         tie_embeddings=True, schedule=tuple(where[self.owner(i)] for i in range(len(self.layers))),
                         residual_float32=True)

    def tensor_names(self) -> TensorNames:
        layers = []
        for i in self.owners():
            p, kind = f"l{i}.", self.layers[i]["type"]
            if kind == "latent_attention":
                mixer = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                         "uv": "uv", "o": "o", "sink": "sink"}
            elif kind == "wkv":
                mixer = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k",
                         "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "o": "o"}
            else:
                mixer = {"q": "q", "k": "k", "v": "v", "o": "o", "temp": "temp"}
            names = {"norm": {"weight": p + "norm1"}, "mixer": {role: p + "mix." + n for role, n in mixer.items()}}
            if self.layers[i].get("mlp") is not None:
                names["ff"] = {r: p + "mlp." + r for r in ("gate", "up", "down")}
            layers.append(names)
        # the output head is the embedding table: no tensor of this name is ever stored
        return TensorNames(embedding="embed", lm_head="head", final_norm={"weight": "final.norm"}, layers=layers)

    def random_init(self, name: str, shape) -> Tuple[float, float]:
        """(mean, standard deviation) of a tensor's seeded random fill: matrices so that a product keeps its input's
        size, blends inside (0, 1), decays neither instant nor absent, sinks and temperatures of either sign."""
        last = name.rsplit(".", 1)[-1]
        if ".mix.mu." in name:
            return 0.5, 0.2
        if last in ("w0",):
            return -1.0, 1.0
        if last in ("sink",):
            return 0.0, 1.0
        if last in ("temp",):
            return 1.0, 0.3
        if last == "u":
            return 0.3, 0.3
        if len(shape) == 1:
            return 1.0, 0.1
        if name == "embed":
            return 0.0, 1.0
        return 0.0, float(shape[-1]) ** -0.5


register_architecture(KudazenConfig.architecture, KudazenConfig)
