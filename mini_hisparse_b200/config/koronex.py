"""Typed Koronex configuration, read from the design's own config.json.

Keys: ``architecture`` ("Koronex"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``postln_alpha``, ``token_side.dim`` (absent or null: no per-layer token input) and ``layers``, a list
whose entries give ``type`` ("lightning" or "attention"), the mixer's sizes ``mixer`` and the
feed-forward ``mlp`` (null: none; else ``kind`` "dense" and ``ff``).  No size has a default; a key this
reader does not know is refused, so that a variant it cannot compute never runs as something else.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .qwen2 import ConfigError


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


def _only(d: Mapping[str, Any], known: tuple[str, ...], where: str) -> None:
    extra = sorted(set(d) - set(known))
    if extra:
        raise ConfigError(f"config.json: unknown key(s) in {where}: {', '.join(extra)}")


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_dims: int
    rot_base: float
    kv_from: int | None


@dataclass(frozen=True)
class KoronexLayer:
    type: str
    mixer: LightningMixer | AttentionMixer
    ff: int | None            # feed-forward width; None: the layer has none


@dataclass(frozen=True)
class KoronexConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    alpha: float
    side_dim: int | None
    layers: tuple[KoronexLayer, ...]
    architecture: str = "Koronex"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "KoronexConfig":
        _only(d, ("architecture", "architectures", "vocab", "width", "embedding", "norm", "postln_alpha",
                  "token_side", "layers"), "the top level")
        emb = _need(d, "embedding", "")
        _only(emb, ("scale",), "embedding")
        norm = _need(d, "norm", "")
        _only(norm, ("eps",), "norm")
        side = d.get("token_side")
        if side is not None:
            _only(side, ("dim",), "token_side")
        layers = []
        raw_layers = _need(d, "layers", "")
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]."
            _only(raw, ("type", "mixer", "mlp"), where[:-1])
            kind = _need(raw, "type", where)
            m = _need(raw, "mixer", where)
            if kind == "lightning":
                _only(m, ("heads", "dim", "vdim", "decay"), where + "mixer")
                mixer = LightningMixer(int(_need(m, "heads", where)), int(_need(m, "dim", where)),
                                       int(_need(m, "vdim", where)), tuple(float(x) for x in _need(m, "decay", where)))
                if len(mixer.decay) != mixer.heads:
                    raise ConfigError(f"{where}mixer: {len(mixer.decay)} decays for {mixer.heads} heads")
            elif kind == "attention":
                _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot", "kv_from"), where + "mixer")
                mask, rot = _need(m, "mask", where), _need(m, "rot", where)
                _only(mask, ("size",), where + "mixer.mask")
                _only(rot, ("dims", "base"), where + "mixer.rot")
                mixer = AttentionMixer(
                    int(_need(m, "heads", where)), int(_need(m, "kv_heads", where)), int(_need(m, "dim", where)),
                    int(_need(m, "vdim", where)), float(_need(m, "scale", where)), int(_need(mask, "size", where)),
                    int(_need(rot, "dims", where)), float(_need(rot, "base", where)),
                    None if m.get("kv_from") is None else int(m["kv_from"]))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}mixer: {mixer.heads} heads over {mixer.kv_heads} kv_heads")
                if mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.dim:
                    raise ConfigError(f"{where}mixer.rot.dims {mixer.rot_dims} must be even and at most dim")
                if mixer.window < 1:
                    raise ConfigError(f"{where}mixer.mask.size must be positive")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design")
            mlp = raw.get("mlp")
            ff = None
            if mlp is not None:
                _only(mlp, ("kind", "ff"), where + "mlp")
                if _need(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"{where}mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
                ff = int(_need(mlp, "ff", where + "mlp."))
            layers.append(KoronexLayer(kind, mixer, ff))
        for i, layer in enumerate(layers):
            j = getattr(layer.mixer, "kv_from", None)
            if j is None:
                continue
            if not 0 <= j < i or layers[j].type != "attention" or layers[j].mixer.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from {j} must name an earlier attention layer with keys of its own")
            a, b = layer.mixer, layers[j].mixer
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"layers[{i}] reads the keys of layer {j}, whose sizes differ")
        if not layers:
            raise ConfigError("config.json: no layers")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  embedding_scale=float(_need(emb, "scale", "embedding.")), eps=float(_need(norm, "eps", "norm.")),
                  alpha=float(_need(d, "postln_alpha", "")),
                  side_dim=None if side is None else int(_need(side, "dim", "token_side.")), layers=tuple(layers))
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.eps > 0:
            raise ConfigError("vocab and width must be positive and norm.eps above zero")
        return cfg

    @classmethod
    def from_json(cls, path) -> "KoronexConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))
