"""Typed configuration of the Zemivik design, read from its own config.json keys.

A Zemivik model is a list of layers, each with one mixer and an optional feed-forward, between an embedding
stage (scaled token embedding plus a learned position vector, then a norm) and a final norm with a head of its
own. Every layer carries its own sizes, so two layers of one model may differ in heads, head sizes, window and
feed-forward width, and a layer may have no feed-forward at all. Nothing has a default in code: a missing or
ill-typed key is a `ConfigError` that names it.

    architecture      "Zemivik"
    vocab, width, max_positions
    embedding.scale   factor on the token embedding
    norm.eps          the one epsilon of every RMS norm of the model
    layers[i].type    which mixer the layer has ("attention")
    layers[i].mixer   heads, kv_heads, dim (query/key head size), vdim (value head size), scale (on the
                      scores), v_mix (bool), mask {size, keep_first} or null (every earlier token)
    layers[i].mlp     null, or {kind: "dense", ff}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import ConfigError


def _obj(d, where: str) -> dict:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object, got {d!r}")
    return d


def _num(d: dict, key: str, where: str, kind):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {where}{key!r} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float) if kind is float else int):
        raise ConfigError(f"config.json: key {where}{key!r} must be {'a number' if kind is float else 'an integer'}, "
                          f"got {v!r}")
    return kind(v)


def _pos_int(d: dict, key: str, where: str) -> int:
    v = _num(d, key, where, int)
    if v <= 0:
        raise ConfigError(f"config.json: key {where}{key!r} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class WindowMask:
    """Token i sees j <= i when i - j < size or j < keep_first."""
    size: int
    keep_first: int


@dataclass(frozen=True)
class ZemivikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    v_mix: bool
    mask: Optional[WindowMask]


@dataclass(frozen=True)
class ZemivikMLP:
    kind: str
    ff: int


@dataclass(frozen=True)
class ZemivikLayer:
    type: str
    mixer: ZemivikAttention
    mlp: Optional[ZemivikMLP]


MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense",)


def _attention(d: dict, where: str) -> ZemivikAttention:
    heads, kv_heads = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    mask = d.get("mask")
    if mask is not None:
        m = _obj(mask, where + "'mask'")
        keep = _num(m, "keep_first", where + "mask.", int)
        if keep < 0:
            raise ConfigError(f"config.json: key {where}mask.'keep_first' must not be negative, got {keep}")
        mask = WindowMask(size=_pos_int(m, "size", where + "mask."), keep_first=keep)
    v_mix = d.get("v_mix", False)
    if not isinstance(v_mix, bool):
        raise ConfigError(f"config.json: key {where}'v_mix' must be true or false, got {v_mix!r}")
    return ZemivikAttention(heads=heads, kv_heads=kv_heads, dim=_pos_int(d, "dim", where),
                            vdim=_pos_int(d, "vdim", where), scale=_num(d, "scale", where, float), v_mix=v_mix,
                            mask=mask)


@dataclass(frozen=True)
class ZemivikConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[ZemivikLayer, ...]

    @staticmethod
    def from_dict(cfg: dict) -> "ZemivikConfig":
        layers_json = cfg.get("layers")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            e = _obj(entry, f"layers[{i}]")
            kind = e.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: key {where}'type' must be one of {list(MIXER_TYPES)}, got {kind!r}")
            mixer = _attention(_obj(e.get("mixer"), where + "'mixer'"), where + "mixer.")
            mlp = e.get("mlp")
            if mlp is not None:
                m = _obj(mlp, where + "'mlp'")
                if m.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: key {where}mlp.'kind' must be one of {list(MLP_KINDS)}, "
                                      f"got {m.get('kind')!r}")
                mlp = ZemivikMLP(kind=m["kind"], ff=_pos_int(m, "ff", where + "mlp."))
            layers.append(ZemivikLayer(type=kind, mixer=mixer, mlp=mlp))
        mixed = [l.mixer for l in layers if l.mixer.v_mix]
        if mixed and any((m.kv_heads, m.vdim) != (mixed[0].kv_heads, mixed[0].vdim) for m in mixed):
            raise ConfigError("config.json: layers with 'v_mix' share the first such layer's values and must have "
                              "its 'kv_heads' and 'vdim'")
        return ZemivikConfig(
            vocab=_pos_int(cfg, "vocab", ""), width=_pos_int(cfg, "width", ""),
            max_positions=_pos_int(cfg, "max_positions", ""),
            embedding_scale=_num(_obj(cfg.get("embedding"), "'embedding'"), "scale", "embedding.", float),
            norm_eps=_num(_obj(cfg.get("norm"), "'norm'"), "eps", "norm.", float), layers=tuple(layers))
