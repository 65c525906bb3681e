"""Typed Dotivik configuration, read from the design's own config.json.

Keys: ``architecture`` ("Dotivik"), ``vocab``, ``width``, ``norm.eps``, ``layers`` (a list whose entries
give ``type``, "attention" or "latent_attention", the mixer's sizes ``mixer`` and the feed-forward ``mlp``:
null for none, else ``kind`` "dense" and ``ff``) and ``loop`` (``start``, ``stop``, ``times``: layers
start .. stop-1 run ``times`` times in a row; absent or null: every layer runs once).  No size has a
default; a key this reader does not know is refused, so that a variant it cannot compute never runs as
something else.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .koronex import _need, _only
from .qwen2 import ConfigError


@dataclass(frozen=True)
class MapsMixer:
    """"attention": heads with two score maps each over shared values."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    diff: float
    rot_dims: int
    rot_base: float
    window: int | None


@dataclass(frozen=True)
class LatentMixer:
    """"latent_attention": a low-rank row per position from which keys and values are expanded."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    window: int | None


@dataclass(frozen=True)
class DotivikLayer:
    type: str
    mixer: MapsMixer | LatentMixer
    ff: int | None            # feed-forward width; None: the layer has none


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


def _window(m: Mapping[str, Any], where: str) -> int | None:
    mask = m.get("mask")
    if mask is None:
        return None
    _only(mask, ("size",), where + "mixer.mask")
    size = int(_need(mask, "size", where + "mixer.mask."))
    if size < 1:
        raise ConfigError(f"{where}mixer.mask.size must be positive")
    return size


@dataclass(frozen=True)
class DotivikConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[DotivikLayer, ...]
    loop: Loop | None
    architecture: str = "Dotivik"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DotivikConfig":
        _only(d, ("architecture", "architectures", "vocab", "width", "norm", "layers", "loop"), "the top level")
        norm = _need(d, "norm", "")
        _only(norm, ("eps",), "norm")
        layers = []
        for i, raw in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            _only(raw, ("type", "mixer", "mlp"), where[:-1])
            kind = _need(raw, "type", where)
            m = _need(raw, "mixer", where)
            if kind == "attention":
                _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "diff", "rot", "mask"), where + "mixer")
                rot = _need(m, "rot", where)
                _only(rot, ("dims", "base"), where + "mixer.rot")
                cap = m.get("softcap")
                mixer = MapsMixer(
                    int(_need(m, "heads", where)), int(_need(m, "kv_heads", where)), int(_need(m, "dim", where)),
                    int(_need(m, "vdim", where)), float(_need(m, "scale", where)),
                    None if cap is None else float(cap), float(_need(m, "diff", where)),
                    int(_need(rot, "dims", where)), float(_need(rot, "base", where)), _window(m, where))
                if mixer.kv_heads < 1 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{where}mixer: {mixer.heads} heads over {mixer.kv_heads} kv_heads")
                if mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.dim:
                    raise ConfigError(f"{where}mixer.rot.dims {mixer.rot_dims} must be even and at most dim")
                if mixer.softcap is not None and not mixer.softcap > 0:
                    raise ConfigError(f"{where}mixer.softcap must be positive")
            elif kind == "latent_attention":
                _only(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot", "mask"), where + "mixer")
                rot = _need(m, "rot", where)
                _only(rot, ("dims", "base"), where + "mixer.rot")
                mixer = LatentMixer(
                    int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(_need(m, "rot_dim", where)),
                    int(_need(m, "vdim", where)), int(_need(m, "kv_rank", where)), float(_need(m, "scale", where)),
                    float(_need(rot, "base", where)), _window(m, where))
                if int(_need(rot, "dims", where)) != mixer.rot_dim:
                    raise ConfigError(f"{where}mixer.rot.dims must equal rot_dim: the whole rotated part turns")
                if mixer.rot_dim % 2 or mixer.rot_dim < 0:
                    raise ConfigError(f"{where}mixer.rot_dim {mixer.rot_dim} must be even")
                if mixer.kv_rank < 1:
                    raise ConfigError(f"{where}mixer.kv_rank must be positive")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design")
            if min(mixer.heads, mixer.dim, mixer.vdim) < 1:
                raise ConfigError(f"{where}mixer: heads, dim and vdim must be positive")
            mlp = raw.get("mlp")
            ff = None
            if mlp is not None:
                _only(mlp, ("kind", "ff"), where + "mlp")
                if _need(mlp, "kind", where + "mlp.") != "dense":
                    raise ConfigError(f"{where}mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
                ff = int(_need(mlp, "ff", where + "mlp."))
            layers.append(DotivikLayer(kind, mixer, ff))
        if not layers:
            raise ConfigError("config.json: no layers")
        loop = None
        raw_loop = d.get("loop")
        if raw_loop is not None:
            _only(raw_loop, ("start", "stop", "times"), "loop")
            loop = Loop(int(_need(raw_loop, "start", "loop.")), int(_need(raw_loop, "stop", "loop.")),
                        int(_need(raw_loop, "times", "loop.")))
            if not 0 <= loop.start <= loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"loop {raw_loop} does not fit {len(layers)} layers")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(norm, "eps", "norm.")), layers=tuple(layers), loop=loop)
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.eps > 0:
            raise ConfigError("vocab and width must be positive and norm.eps above zero")
        return cfg

    @classmethod
    def from_json(cls, path) -> "DotivikConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))
