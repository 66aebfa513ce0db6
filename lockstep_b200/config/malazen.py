"""Malazen: a decoder whose layers pair softmax attention with a linear recurrence, or attend
over a cached latent, and whose middle layers may run several times.

``config.json`` holds ``vocab``, ``width``, ``norm`` (``eps``, ``groups``), an optional ``loop``
(``start``, ``stop``, ``times``) and a list ``layers``; every entry gives ``type`` (which mixer),
``mixer`` (its sizes and constants) and ``mlp`` (its feed-forward, or null for none).

- ``parallel``: two mixers read the same normed rows and the layer adds ``left_scale`` x left +
  ``right_scale`` x right.  Left: grouped-query softmax attention over every earlier key, with
  biases on its four projections, no rotation, a query temperature (``q_temp``), ``scale`` on the
  scores and a bias r1 ln(1 + r2 distance) per head taken off them.  Right: gated linear attention,
  a decayed sum of outer products per head with a decay per key channel sigmoid(z)^(1/``tau``).
- ``latent_attention``: per token one normed latent of ``kv_rank`` elements and one rotated key
  part of ``rot_dim`` elements are cached; heads of ``dim`` plain + ``rot_dim`` rotated query
  elements, values of ``vdim``; rotation of neighbouring pairs with stretched frequencies
  (``rot.scaling``), a sliding window (``mask.size``), a sink per head in the softmax.

The feed-forward (``kind`` "dense") is a gated unit with clamps at ``limit`` and biases.  Norms are
RMS norms in ``groups`` equal parts.  With ``loop``, layers start .. stop-1 run ``times`` times in a
row with the same weights and a cache of their own each time, and the embedding's output is added
to the residual stream before every pass but the first.  The head is the embedding table.  Layer
i's tensors start with ``l<i>.``: ``norm1``, ``mix.*``, ``norm2``, ``mlp.*``.
"""

from __future__ import annotations

import copy
from typing import Any, Mapping

from .registry import register_architecture
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec

MIXERS = ("parallel", "latent_attention")
DEFAULT_MAX_POSITIONS = 32768
GLU_ALPHA = 1.702          # the sigmoid's slope in the feed-forward's activation


def _positive(where: str, raw: Mapping[str, Any], *keys: str) -> None:
    for k in keys:
        if k not in raw:
            raise ConfigError(f"{where} lacks {k!r}")
        if not (isinstance(raw[k], int) and not isinstance(raw[k], bool) and raw[k] > 0):
            raise ConfigError(f"{where}: {k} must be a positive integer, got {raw[k]!r}")


def _number(where: str, raw: Mapping[str, Any], *keys: str) -> None:
    for k in keys:
        if not isinstance(raw.get(k), (int, float)) or isinstance(raw.get(k), bool):
            raise ConfigError(f"{where}: {k} must be a number, got {raw.get(k)!r}")


@register_architecture("Malazen")
class MalazenConfig:
    def __init__(self, raw: Mapping[str, Any]):
        self.raw = copy.deepcopy(dict(raw))
        self.validate()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MalazenConfig":
        return cls(raw)

    def to_dict(self) -> dict[str, Any]:
        return copy.deepcopy(self.raw)

    # -- reading ------------------------------------------------------------
    @property
    def width(self) -> int:
        return int(self.raw["width"])

    @property
    def vocab(self) -> int:
        return int(self.raw["vocab"])

    @property
    def eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @property
    def groups(self) -> int:
        return int(self.raw["norm"].get("groups", 1))

    @property
    def layers(self) -> list[dict]:
        return self.raw["layers"]

    def validate(self) -> None:
        r = self.raw
        _positive("config.json", r, "vocab", "width")
        norm = r.get("norm")
        if not isinstance(norm, Mapping) or "eps" not in norm or not float(norm["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be a positive number")
        groups = norm.get("groups", 1)
        if not (isinstance(groups, int) and groups > 0 and r["width"] % groups == 0):
            raise ConfigError(f"config.json: norm.groups must divide the width, got {groups!r}")
        if not isinstance(r.get("layers"), list) or not r["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        loop = r.get("loop")
        if loop is not None:
            _positive("loop", loop, "stop", "times")
            if not (isinstance(loop.get("start"), int) and 0 <= loop["start"] < loop["stop"] <= len(r["layers"])):
                raise ConfigError("loop: 0 <= start < stop <= number of layers must hold")
        for i, layer in enumerate(r["layers"]):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}: type {kind!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where} lacks its mixer's sizes")
            if kind == "parallel":
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, Mapping) or not isinstance(right, Mapping):
                    raise ConfigError(f"{where}: a parallel mixer needs 'left' and 'right'")
                _positive(where + ".left", left, "heads", "dim", "vdim")
                if "kv_heads" in left:
                    _positive(where + ".left", left, "kv_heads")
                _number(where + ".left", left, "scale")
                if left["heads"] % left.get("kv_heads", left["heads"]):
                    raise ConfigError(f"{where}.left: heads must be a multiple of kv_heads")
                temp = left.get("q_temp")
                if temp is not None:
                    _positive(where + ".left.q_temp", temp, "every")
                    _number(where + ".left.q_temp", temp, "coef")
                _positive(where + ".right", right, "heads", "dim", "vdim")
                _number(where + ".right", right, "tau")
                if not float(right["tau"]) > 0:
                    raise ConfigError(f"{where}.right: tau must be positive")
                _number(where, m, "left_scale", "right_scale")
            else:
                _positive(where, m, "heads", "dim", "rot_dim", "vdim", "kv_rank")
                _number(where, m, "scale")
                rot = m.get("rot")
                if not isinstance(rot, Mapping):
                    raise ConfigError(f"{where} lacks 'rot'")
                _positive(where + ".rot", rot, "dims")
                if rot["dims"] != m["rot_dim"] or rot["dims"] % 2 or not float(rot.get("base", 0)) > 0:
                    raise ConfigError(f"{where}: rot.dims must be even and equal rot_dim, rot.base positive")
                scaling = rot.get("scaling")
                if scaling is not None:
                    _number(where + ".rot.scaling", scaling, "factor", "original", "fast", "slow")
                    if not float(scaling["factor"]) > 0 or not float(scaling["original"]) > 0:
                        raise ConfigError(f"{where}.rot.scaling: factor and original must be positive")
                mask = m.get("mask")
                if mask is not None:
                    _positive(where + ".mask", mask, "size")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not supported (dense)")
                _positive(where + ".mlp", f, "ff")
                _number(where + ".mlp", f, "limit")

    # -- the model as data --------------------------------------------------
    def _mixer(self, layer: Mapping[str, Any]) -> tuple[PartSpec, PartSpec]:
        m, width, eps = layer["mixer"], self.width, self.eps
        if layer["type"] == "parallel":
            left, right = m["left"], m["right"]
            attention = PartSpec("gqa_attention", {
                "hidden_size": width, "num_heads": int(left["heads"]), "num_kv_heads": int(left.get("kv_heads", left["heads"])),
                "head_dim": int(left["dim"]), "value_dim": int(left["vdim"]), "scale": float(left["scale"]),
                "window": 0, "qk_norm_eps": None, "bias": True, "q_temp": left.get("q_temp"),
                "score_bias": "log_distance",
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                          "o_bias": "o.b", "r1": "r1", "r2": "r2"}})
            linear = PartSpec("gated_linear", {
                "hidden_size": width, "num_heads": int(right["heads"]), "key_dim": int(right["dim"]),
                "value_dim": int(right["vdim"]), "tau": float(right["tau"]), "norm_eps": eps,
                # the rank of the decay's low-rank map is the stored tensors' own; a configuration
                # may name it (random weights need it)
                "decay_rank": right.get("decay_rank")})
            mixer = PartSpec("parallel", {"hidden_size": width, "branches": (
                {"name": "left", "mixer": attention, "position": None, "scale": float(m["left_scale"])},
                {"name": "right", "mixer": linear, "position": None, "scale": float(m["right_scale"])})})
            return mixer, PartSpec("none")
        rot = m["rot"]
        position = PartSpec("scaled_rotary", {"dim": int(rot["dims"]), "theta": float(rot["base"]),
                                              "scaling": rot.get("scaling"), "interleaved": True})
        mixer = PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
            "value_dim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]),
            "window": int((m.get("mask") or {}).get("size", 0)), "norm_eps": eps, "sink": True})
        return mixer, position

    def schedule(self) -> list[LayerRun]:
        """Every run of a layer has a cache entry of its own; the first layer of every pass of the
        loop but the first gets the embedding's output added in front of it."""
        n = len(self.layers)
        loop = self.raw.get("loop")
        order = [(i, False) for i in range(n)]
        if loop:
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            order = [(i, False) for i in range(start)]
            for t in range(times):
                order += [(i, t > 0 and i == start) for i in range(start, stop)]
            order += [(i, False) for i in range(stop, n)]
        return [LayerRun(layer=i, cache=entry, add_embedding=add) for entry, (i, add) in enumerate(order)]

    def model_spec(self) -> ModelSpec:
        width, vocab = self.width, self.vocab
        norm = PartSpec("rmsnorm", {"width": width, "eps": self.eps, "tensor": "", "groups": self.groups})
        layers, optional = [], []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer)
            f = layer.get("mlp")
            if f is None:
                feed_forward = PartSpec("none")
                optional.append(f"l{i}.norm2")
            else:
                feed_forward = PartSpec("clamped_glu", {"hidden_size": width, "intermediate_size": int(f["ff"]),
                                                        "limit": float(f["limit"]), "alpha": GLU_ALPHA, "bias": True})
            block = PartSpec("pre_norm", {"names": {"mixer_norm": "norm1", "mixer": "mix",
                                                    "feed_forward_norm": "norm2", "feed_forward": "mlp"}})
            layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=feed_forward,
                                    mixer_norm=norm, feed_forward_norm=norm, position=position))
        return ModelSpec(
            architecture="Malazen", hidden_size=width, vocab_size=vocab,
            max_positions=int(self.raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "width": width, "tensor": ""}),
            final_norm=norm,
            head=PartSpec("linear_head", {"vocab_size": vocab, "width": width, "tied": True}),
            layers=tuple(layers), schedule=tuple(self.schedule()),
            names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
            optional_tensors=tuple(optional))
