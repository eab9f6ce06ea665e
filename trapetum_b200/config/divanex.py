"""Divanex's configuration, read from the keys of its config.json.

Top level: ``architecture`` ("Divanex"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``postln_alpha``, ``logit_scale``, ``token_side.dim`` (the key or the object may be absent: no side input)
and ``layers``, a list whose entries give ``type`` ("attention" or "mamba2"), ``mixer`` (that mixer's sizes
and constants) and ``mlp`` (``{"kind": "dense", "ff", "limit"}`` or null).  Every size and constant is read
by key, with an error that names the key; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, _get

MIXERS = ("attention", "mamba2")


def _obj(d: Dict[str, Any], key: str, where: str, nullable: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None:
        if nullable:
            return None
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: key '{where}{key}' must be an object, got {v!r}")
    return v


def _sub(d: Dict[str, Any], key: str, typ, where: str, *args, **kw):
    try:
        return _get(d, key, typ, *args, **kw)
    except ConfigError as e:
        raise ConfigError(str(e).replace(f"'{key}'", f"'{where}{key}'")) from None


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    q_temp_coef: float
    q_temp_every: int


@dataclass(frozen=True)
class Mamba2Mixer:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float


@dataclass(frozen=True)
class DivanexLayer:
    type: str
    mixer: Any                       # AttentionMixer | Mamba2Mixer
    mlp: Optional[DenseMlp]


@dataclass(frozen=True)
class DivanexConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    postln_alpha: float
    logit_scale: float
    side_dim: Optional[int]
    layers: Tuple[DivanexLayer, ...]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DivanexConfig":
        vocab = _get(d, "vocab", int)
        width = _get(d, "width", int)
        emb = _obj(d, "embedding", "", nullable=True) or {}
        norm = _obj(d, "norm", "")
        side = _obj(d, "token_side", "", nullable=True)
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            typ = _sub(L, "type", str, where)
            m = _obj(L, "mixer", where)
            mw = where + "mixer."
            if typ == "attention":
                heads = _sub(m, "heads", int, mw)
                kv = _sub(m, "kv_heads", int, mw, heads)
                dim = _sub(m, "dim", int, mw)
                vdim = _sub(m, "vdim", int, mw, dim)
                if vdim != dim:
                    raise ConfigError(f"config.json: {mw}vdim is {vdim}, but v is the k projection itself, whose heads have size {dim}")
                if heads < 1 or kv < 1 or heads % kv:
                    raise ConfigError(f"config.json: {mw}heads={heads} cannot share kv_heads={kv}")
                qt = _obj(m, "q_temp", mw, nullable=True) or {}
                coef = _sub(qt, "coef", float, mw + "q_temp.", 0.0)
                every = _sub(qt, "every", int, mw + "q_temp.", 1) if qt else 0
                if qt and every < 1:
                    raise ConfigError(f"config.json: {mw}q_temp.every must be at least 1, got {every}")
                mixer = AttentionMixer(heads, kv, dim, vdim, _sub(m, "scale", float, mw),
                                       _sub(m, "softcap", float, mw, None, nullable=True), coef, every)
            elif typ == "mamba2":
                mixer = Mamba2Mixer(_sub(m, "heads", int, mw), _sub(m, "vdim", int, mw), _sub(m, "state", int, mw),
                                    _sub(m, "groups", int, mw, 1), _sub(m, "conv", int, mw),
                                    _sub(m, "norm_groups", int, mw, 1))
                if mixer.groups < 1 or mixer.heads % mixer.groups:
                    raise ConfigError(f"config.json: {mw}heads={mixer.heads} cannot share groups={mixer.groups}")
                if mixer.norm_groups < 1 or (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json: {mw}norm_groups={mixer.norm_groups} does not divide "
                                      f"{mixer.heads * mixer.vdim} inner columns")
                if mixer.conv < 1:
                    raise ConfigError(f"config.json: {mw}conv must be at least 1, got {mixer.conv}")
            else:
                raise ConfigError(f"config.json: {where}type is '{typ}'; known mixers: {', '.join(MIXERS)}")
            mlp = None
            ml = _obj(L, "mlp", where, nullable=True)
            if ml is not None:
                kind = _sub(ml, "kind", str, where + "mlp.")
                if kind != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind is '{kind}'; known kinds: dense")
                mlp = DenseMlp(_sub(ml, "ff", int, where + "mlp."), _sub(ml, "limit", float, where + "mlp."))
                if not mlp.limit > 0:
                    raise ConfigError(f"config.json: {where}mlp.limit must be positive, got {mlp.limit}")
            layers.append(DivanexLayer(typ, mixer, mlp))
        side_dim = _sub(side, "dim", int, "token_side.") if side else None
        return cls(vocab=vocab, width=width, embedding_scale=_sub(emb, "scale", float, "embedding.", 1.0),
                   norm_eps=_sub(norm, "eps", float, "norm."), postln_alpha=_get(d, "postln_alpha", float, 1.0),
                   logit_scale=_get(d, "logit_scale", float, 1.0), side_dim=side_dim, layers=tuple(layers))
