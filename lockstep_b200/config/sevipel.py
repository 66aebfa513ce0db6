"""Sevipel: a decoder whose layers each name their own mixer.

``config.json`` holds ``vocab``, ``width``, ``norm.eps`` and a list ``layers``; every entry gives
``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (its feed-forward, or
null for none).  Three mixers:

- ``attention``: grouped-query attention over a sliding window (``mask.size``; absent: every
  earlier key), RMSNorm of the whole query and of the whole key projection before the heads are
  split, rotation of the first ``rot.dims`` elements of each head (halves layout, base
  ``rot.base``), ``scale`` on the scores, a value size ``vdim`` of its own.  With ``kv_from: j``
  the layer has no key or value tensors and reads the cache entry of layer j.
- ``channel_delta``: the gated delta rule with a decay per head and key channel, short causal
  convolutions on q, k, v, and a gated per-head RMSNorm of the read-out.
- ``wkv``: token-shift mixes, a per-channel decay from a low-rank map, a bonus for the current
  token, a gated per-head RMSNorm of the read-out.

The feed-forward is a mixture of experts: sigmoid scores, the ``top`` largest chosen, each chosen
expert run on the token's row times its score, squared-ReLU experts without biases.  A norm's
tensor w holds its gain minus one (the gain is 1 + w).  The head is the embedding table.  Layer i's tensors start with
``l<i>.``: ``norm1``, ``mix.*``, ``norm2``, ``mlp.*``.
"""

from __future__ import annotations

import copy
from typing import Any, Mapping

from .registry import register_architecture
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec

MIXERS = ("attention", "channel_delta", "wkv")
DEFAULT_MAX_POSITIONS = 32768


def _positive(where: str, raw: Mapping[str, Any], *keys: str) -> None:
    for k in keys:
        if k not in raw:
            raise ConfigError(f"{where} lacks {k!r}")
        if not (isinstance(raw[k], int) and not isinstance(raw[k], bool) and raw[k] > 0):
            raise ConfigError(f"{where}: {k} must be a positive integer, got {raw[k]!r}")


@register_architecture("Sevipel")
class SevipelConfig:
    def __init__(self, raw: Mapping[str, Any]):
        self.raw = copy.deepcopy(dict(raw))
        self.validate()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SevipelConfig":
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
    def layers(self) -> list[dict]:
        return self.raw["layers"]

    def validate(self) -> None:
        r = self.raw
        _positive("config.json", r, "vocab", "width")
        if not isinstance(r.get("norm"), Mapping) or "eps" not in r["norm"] or not float(r["norm"]["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be a positive number")
        if not isinstance(r.get("layers"), list) or not r["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        for i, layer in enumerate(r["layers"]):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}: type {kind!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where} lacks its mixer's sizes")
            if kind == "attention":
                _positive(where, m, "heads", "kv_heads", "dim", "vdim")
                if "scale" not in m:
                    raise ConfigError(f"{where} lacks 'scale'")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
                rot = m.get("rot")
                if rot is not None:
                    _positive(where + ".rot", rot, "dims")
                    if rot["dims"] % 2 or rot["dims"] > m["dim"] or not float(rot.get("base", 0)) > 0:
                        raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base positive")
                mask = m.get("mask")
                if mask is not None:
                    _positive(where + ".mask", mask, "size")
                src = m.get("kv_from")
                if src is not None:
                    if not (isinstance(src, int) and 0 <= src < i) or r["layers"][src].get("type") != "attention" \
                            or r["layers"][src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from must name an earlier attention layer with keys of its own")
                    other = r["layers"][src]["mixer"]
                    for k in ("kv_heads", "dim", "vdim"):
                        if other[k] != m[k]:
                            raise ConfigError(f"{where}: {k} differs from layer {src}, whose keys and values it reads")
            elif kind == "channel_delta":
                _positive(where, m, "heads", "kv_heads", "dim", "vdim", "conv")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
            else:
                _positive(where, m, "heads", "dim")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not supported (moe)")
                _positive(where + ".mlp.expert", f.get("expert") or {}, "ff")
                _positive(where + ".mlp.router", f.get("router") or {}, "experts", "top")
                if f["router"]["top"] > f["router"]["experts"]:
                    raise ConfigError(f"{where}: top exceeds the number of experts")

    # -- the model as data --------------------------------------------------
    def _mixer(self, layer: Mapping[str, Any]) -> tuple[PartSpec, PartSpec]:
        m, width, eps = layer["mixer"], self.width, self.eps
        position = PartSpec("none")
        if layer["type"] == "attention":
            rot = m.get("rot")
            if rot is not None:
                position = PartSpec("rotary", {"dim": int(rot["dims"]), "theta": float(rot["base"])})
            mixer = PartSpec("gqa_attention", {
                "hidden_size": width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
                "window": int((m.get("mask") or {}).get("size", 0)), "qk_norm_eps": eps,
                "qk_norm_scope": "projection", "borrows_kv": m.get("kv_from") is not None,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"},
            })
        elif layer["type"] == "channel_delta":
            mixer = PartSpec("gated_delta", {
                "hidden_size": width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "conv_taps": int(m["conv"]),
                "norm_eps": eps, "unit_eps": 1e-6,
                # the ranks of the low-rank maps are the stored tensors' own; a configuration may
                # name them (random weights need them)
                "decay_rank": m.get("decay_rank"), "gate_rank": m.get("gate_rank")})
        else:
            mixer = PartSpec("wkv", {"hidden_size": width, "num_heads": int(m["heads"]),
                                     "head_dim": int(m["dim"]), "norm_eps": eps,
                                     "decay_rank": m.get("decay_rank")})
        return mixer, position

    def model_spec(self) -> ModelSpec:
        width, vocab = self.width, self.vocab
        norm = PartSpec("rmsnorm", {"width": width, "eps": self.eps, "offset": 1.0, "tensor": ""})
        layers, schedule, optional = [], [], []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer)
            f = layer.get("mlp")
            if f is None:
                feed_forward = PartSpec("none")
                optional.append(f"l{i}.norm2")
            else:
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": width, "expert_size": int(f["expert"]["ff"]),
                    "experts": int(f["router"]["experts"]), "top": int(f["router"]["top"])})
            block = PartSpec("pre_norm", {"names": {"mixer_norm": "norm1", "mixer": "mix",
                                                    "feed_forward_norm": "norm2", "feed_forward": "mlp"}})
            layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=feed_forward,
                                    mixer_norm=norm, feed_forward_norm=norm, position=position))
            src = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            schedule.append(LayerRun(layer=i, cache=i) if src is None
                            else LayerRun(layer=i, cache=int(src), writes_cache=False))
        return ModelSpec(
            architecture="Sevipel", hidden_size=width, vocab_size=vocab,
            max_positions=int(self.raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "width": width, "tensor": ""}),
            final_norm=norm,
            head=PartSpec("linear_head", {"vocab_size": vocab, "width": width, "tied": True}),
            layers=tuple(layers), schedule=tuple(schedule),
            names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
            optional_tensors=tuple(optional))
