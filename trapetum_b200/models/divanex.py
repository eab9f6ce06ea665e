"""Divanex as data: its configuration turned into a :class:`ModelSpec`.

Nothing here computes.  A Divanex layer is a ``post_norm`` block (the norm after the sum, the stream scaled
by ``postln_alpha`` on the way in) around one of two mixers and an optional dense feed-forward, followed by a
side input that is looked up by token id:

* ``attention``: no rotation; no v matrix (v is the raw output of the k projection); q and k heads divided by their root mean
  square; a query temperature that grows with the logarithm of the position; scaled, soft-capped scores; causal
  softmax.  All of it is the framework's attention part with the matching parameters.
* ``mamba2``: the state-space part of :mod:`trapetum_b200.parts.mamba2`.
* feed-forward: the gated part with the ``clamped_swish`` activation and the layer's limit.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``l<i>.side.{gate,proj,norm}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
from ..config.divanex import DivanexConfig

MAX_POSITIONS = 1 << 30          # positions enter only through a logarithm: nothing bounds them but the cache


def divanex_spec(cfg: DivanexConfig) -> ModelSpec:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "unit_offset": False, "weight": name, "role": "gain"})

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "attention":
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "scale": m.scale, "softcap": m.softcap, "window": None,
                "position": PartSpec("none", {"head_dim": m.dim}),
                "head_unit_norm": {"q": True, "k": True, "eps": cfg.norm_eps},
                "q_temp": {"coef": m.q_temp_coef, "every": m.q_temp_every} if m.q_temp_every else None,
                "q": "mix.q", "k": "mix.k", "v": None, "o": "mix.o",
            })
        else:
            mixer = PartSpec("mamba2", {
                "hidden_size": W, "heads": m.heads, "head_dim": m.vdim, "state": m.state, "groups": m.groups,
                "conv": m.conv, "norm_groups": m.norm_groups, "eps": cfg.norm_eps,
                "in": "mix.in", "conv_w": "mix.conv", "conv_b": "mix.conv.b", "dt_bias": "mix.dt_bias",
                "A_log": "mix.A_log", "D": "mix.D", "norm": "mix.norm", "o": "mix.o",
            })
        if L.mlp is not None:
            ffn = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": L.mlp.ff, "activation": "clamped_swish",
                                         "limit": L.mlp.limit, "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
        else:
            ffn = PartSpec("none", {})
        side = None
        if cfg.side_dim:
            side = PartSpec("token_gated", {"hidden_size": W, "dim": cfg.side_dim, "vocab_size": cfg.vocab,
                                            "table_width": cfg.side_dim * len(cfg.layers), "first_col": i * cfg.side_dim,
                                            "table": "side.embed", "gate": "side.gate", "proj": "side.proj"})
        block = PartSpec("post_norm", {"alpha": cfg.postln_alpha, "mixer_norm": norm("norm1"),
                                       "ffn_norm": norm("norm2") if L.mlp is not None else None,
                                       "side": side, "side_norm": norm("side.norm") if side else None})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, prefix=f"l{i}."))

    return ModelSpec(
        architecture="Divanex",
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale,
                                         "weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "softcap": None,
                                      "scale": cfg.logit_scale, "weight": "head", "tied_to": None}),
        max_positions=MAX_POSITIONS,
        stop_ids=(),
    )


register_architecture("Divanex", DivanexConfig, divanex_spec, native=False)
