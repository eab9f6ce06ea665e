"""Lofirax's configuration, read from the keys of its config.json.

Top level: ``architecture`` ("Lofirax"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``logit_softcap`` (absent or null: no cap), ``loop`` (``start``, ``stop``, ``times``; absent: every layer runs
once) and ``layers``, a list whose entries give ``type`` ("gla" or "latent_attention"), ``mixer`` (that mixer's
sizes and constants) and ``mlp`` (``{"kind": "dense", "ff"}``, ``{"kind": "moe", "expert": {"ff"}, "router":
{"experts", "top", "groups": {"count", "keep"}}, "shared": {"ff"}}`` or null).  Every size and constant is
read by key, with an error that names the key; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, _get
from .divanex import _obj, _sub

MIXERS = ("gla", "latent_attention")


@dataclass(frozen=True)
class GlaMixer:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None       # the decay's rank; absent: the weight file's shapes decide


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int            # unrotated query/key dims per head
    rot_dim: int        # rotated query/key dims per head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int       # how many of the rot_dim dims the rotation turns
    rot_base: float


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    ff: int
    groups: int         # 1: no groups
    keep: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class LofiraxLayer:
    type: str
    mixer: Any                       # GlaMixer | LatentMixer
    mlp: Any                         # DenseMlp | MoeMlp | None


@dataclass(frozen=True)
class LofiraxConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: Optional[float]
    loop: Optional[Loop]
    layers: Tuple[LofiraxLayer, ...]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LofiraxConfig":
        vocab = _get(d, "vocab", int)
        width = _get(d, "width", int)
        emb = _obj(d, "embedding", "", nullable=True) or {}
        norm = _obj(d, "norm", "")
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
            if typ == "gla":
                mixer = GlaMixer(_sub(m, "heads", int, mw), _sub(m, "dim", int, mw), _sub(m, "vdim", int, mw),
                                 _sub(m, "tau", float, mw), _sub(m, "rank", int, mw, None, nullable=True))
                if min(mixer.heads, mixer.dim, mixer.vdim) < 1 or not mixer.tau > 0:
                    raise ConfigError(f"config.json: {mw}heads, dim, vdim and tau must be positive")
            elif typ == "latent_attention":
                rot = _obj(m, "rot", mw)
                rot_dim = _sub(m, "rot_dim", int, mw)
                mixer = LatentMixer(_sub(m, "heads", int, mw), _sub(m, "dim", int, mw), rot_dim,
                                    _sub(m, "vdim", int, mw), _sub(m, "kv_rank", int, mw), _sub(m, "scale", float, mw),
                                    _sub(rot, "dims", int, mw + "rot.", rot_dim), _sub(rot, "base", float, mw + "rot."))
                if min(mixer.heads, mixer.vdim, mixer.kv_rank) < 1 or mixer.dim < 0 or mixer.rot_dim < 0 \
                        or mixer.dim + mixer.rot_dim < 1:
                    raise ConfigError(f"config.json: {mw}heads, vdim, kv_rank and dim + rot_dim must be positive")
                if mixer.rot_dims % 2 or not (0 <= mixer.rot_dims <= mixer.rot_dim):
                    raise ConfigError(f"config.json: {mw}rot.dims={mixer.rot_dims} must be even and at most "
                                      f"rot_dim={mixer.rot_dim}")
            else:
                raise ConfigError(f"config.json: {where}type is '{typ}'; known mixers: {', '.join(MIXERS)}")
            mlp = None
            ml = _obj(L, "mlp", where, nullable=True)
            if ml is not None:
                lw = where + "mlp."
                kind = _sub(ml, "kind", str, lw)
                if kind == "dense":
                    mlp = DenseMlp(_sub(ml, "ff", int, lw))
                elif kind == "moe":
                    r = _obj(ml, "router", lw)
                    g = _obj(r, "groups", lw + "router.", nullable=True)
                    sh = _obj(ml, "shared", lw, nullable=True)
                    mlp = MoeMlp(_sub(r, "experts", int, lw + "router."), _sub(r, "top", int, lw + "router."),
                                 _sub(_obj(ml, "expert", lw), "ff", int, lw + "expert."),
                                 _sub(g, "count", int, lw + "router.groups.") if g else 1,
                                 _sub(g, "keep", int, lw + "router.groups.") if g else 1,
                                 _sub(sh, "ff", int, lw + "shared.") if sh else None)
                    if mlp.experts < 1 or not (1 <= mlp.top <= mlp.experts):
                        raise ConfigError(f"config.json: {lw}router: top={mlp.top} of experts={mlp.experts}")
                    if mlp.groups < 1 or mlp.experts % mlp.groups or not (1 <= mlp.keep <= mlp.groups):
                        raise ConfigError(f"config.json: {lw}router.groups: {mlp.experts} experts do not form "
                                          f"{mlp.groups} equal groups of which {mlp.keep} are kept")
                    if mlp.keep * (mlp.experts // mlp.groups) < mlp.top:
                        raise ConfigError(f"config.json: {lw}router: {mlp.keep} kept groups hold fewer than "
                                          f"top={mlp.top} experts")
                else:
                    raise ConfigError(f"config.json: {lw}kind is '{kind}'; known kinds: dense, moe")
            layers.append(LofiraxLayer(typ, mixer, mlp))
        loop = None
        lp = _obj(d, "loop", "", nullable=True)
        if lp is not None:
            loop = Loop(_sub(lp, "start", int, "loop."), _sub(lp, "stop", int, "loop."), _sub(lp, "times", int, "loop."))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError(f"config.json: loop start={loop.start} stop={loop.stop} times={loop.times} does not "
                                  f"fit {len(layers)} layers")
        return cls(vocab=vocab, width=width, embedding_scale=_sub(emb, "scale", float, "embedding.", 1.0),
                   norm_eps=_sub(norm, "eps", float, "norm."),
                   logit_softcap=_get(d, "logit_softcap", float, None, nullable=True), loop=loop, layers=tuple(layers))
