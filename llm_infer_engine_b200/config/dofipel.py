"""Typed configuration of the Dofipel design, read from its own config.json keys.

A Dofipel model is a list of layers between a token embedding and a final Dynamic-Tanh norm whose output is
multiplied by the embedding table again (times a constant) to give the logits. A layer is u = norm(x);
x += mixer(u) + ff(u). Every layer carries its own sizes and constants; nothing has a default in code: a missing or
ill-typed key is a `ConfigError` that names it.

    architecture      "Dofipel"
    vocab, width, logit_scale
    norm.eps          the epsilon of the RMS norms inside mixers
    layers[i].type    "attention" | "latent_attention"
    layers[i].mixer   attention: heads, kv_heads, dim, vdim, scale, softcap, bias_max, mask {size} or null
                      latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims},
                      kv_from (optional: the layer whose latent this one reads instead of making its own)
    layers[i].mlp     null | {kind: "dense", ff} | {kind: "moe", router {experts, top}, expert {ff},
                      shared {ff} or null}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .registry import ConfigError
from .zemivik import _num, _obj, _pos_int


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    bias_max: float
    window: int                     # 0 = every earlier token


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int]


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class DofipelLayer:
    type: str
    mixer: Union[WindowAttention, LatentAttention]
    mlp: Union[None, DenseFF, RoutedFF]


MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _window_attention(d: dict, where: str) -> WindowAttention:
    heads, kv_heads = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    window = 0
    if d.get("mask") is not None:
        window = _pos_int(_obj(d["mask"], where + "'mask'"), "size", where + "mask.")
    softcap = _num(d, "softcap", where, float)
    if softcap <= 0:
        raise ConfigError(f"config.json: key {where}'softcap' must be positive, got {softcap}")
    return WindowAttention(heads=heads, kv_heads=kv_heads, dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                           scale=_num(d, "scale", where, float), softcap=softcap,
                           bias_max=_num(d, "bias_max", where, float), window=window)


def _latent_attention(d: dict, where: str, index: int) -> LatentAttention:
    rot = _obj(d.get("rot"), where + "'rot'")
    rot_dim, rot_dims = _pos_int(d, "rot_dim", where), _pos_int(rot, "dims", where + "rot.")
    if rot_dims % 2 or rot_dims > rot_dim:
        raise ConfigError(f"config.json: key {where}rot.'dims' ({rot_dims}) must be even and at most 'rot_dim' ({rot_dim})")
    kv_from = d.get("kv_from")
    if kv_from is not None:
        kv_from = _num(d, "kv_from", where, int)
        if not 0 <= kv_from < index:
            raise ConfigError(f"config.json: key {where}'kv_from' ({kv_from}) must name an earlier layer")
    return LatentAttention(heads=_pos_int(d, "heads", where), dim=_pos_int(d, "dim", where), rot_dim=rot_dim,
                           vdim=_pos_int(d, "vdim", where), kv_rank=_pos_int(d, "kv_rank", where),
                           scale=_num(d, "scale", where, float), rot_base=_num(rot, "base", where + "rot.", float),
                           rot_dims=rot_dims, kv_from=kv_from)


def _mlp(m, where: str):
    if m is None:
        return None
    m = _obj(m, where + "'mlp'")
    kind = m.get("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: key {where}mlp.'kind' must be one of {list(MLP_KINDS)}, got {kind!r}")
    if kind == "dense":
        return DenseFF(ff=_pos_int(m, "ff", where + "mlp."))
    router = _obj(m.get("router"), where + "mlp.'router'")
    experts, top = _pos_int(router, "experts", where + "mlp.router."), _pos_int(router, "top", where + "mlp.router.")
    if top > experts:
        raise ConfigError(f"config.json: key {where}mlp.router.'top' ({top}) exceeds 'experts' ({experts})")
    shared = m.get("shared")
    shared_ff = None if shared is None else _pos_int(_obj(shared, where + "mlp.'shared'"), "ff", where + "mlp.shared.")
    return RoutedFF(experts=experts, top=top,
                    expert_ff=_pos_int(_obj(m.get("expert"), where + "mlp.'expert'"), "ff", where + "mlp.expert."),
                    shared_ff=shared_ff)


@dataclass(frozen=True)
class DofipelConfig:
    vocab: int
    width: int
    logit_scale: float
    norm_eps: float
    layers: Tuple[DofipelLayer, ...]

    @staticmethod
    def from_dict(cfg: dict) -> "DofipelConfig":
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
            m = _obj(e.get("mixer"), where + "'mixer'")
            mixer = _window_attention(m, where + "mixer.") if kind == "attention" else \
                _latent_attention(m, where + "mixer.", i)
            layers.append(DofipelLayer(type=kind, mixer=mixer, mlp=_mlp(e.get("mlp"), where)))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, LatentAttention) and m.kv_from is not None:
                src = layers[m.kv_from].mixer
                if not isinstance(src, LatentAttention) or src.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.'kv_from' must name a latent-attention layer "
                                      "that makes its own latent")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                    raise ConfigError(f"config.json: layers[{i}] reads the latent of layers[{m.kv_from}] and must have "
                                      "its 'kv_rank', 'rot_dim' and 'rot'")
        return DofipelConfig(vocab=_pos_int(cfg, "vocab", ""), width=_pos_int(cfg, "width", ""),
                             logit_scale=_num(cfg, "logit_scale", "", float),
                             norm_eps=_num(_obj(cfg.get("norm"), "'norm'"), "eps", "norm.", float), layers=tuple(layers))
