"""Lofirax as data: its configuration turned into a :class:`ModelSpec`.

Nothing here computes.  A Lofirax layer is a ``pre_norm`` block whose two norms are layer norms with weight and
bias, around one of two mixers and a feed-forward (or none):

* ``gla``: gated linear attention with a per-channel decay of low rank (:mod:`trapetum_b200.parts.gla`);
* ``latent_attention``: attention whose keys and values are made from one cached latent row per token, with a
  rotated key part shared by the heads and a learned sink in the softmax
  (:mod:`trapetum_b200.parts.latent_attention`);
* feed-forward: the gated part with ``gelu_tanh``, or experts behind a router with a gated shared expert
  (:mod:`trapetum_b200.parts.experts`).

A span of layers may run several times in a row with the same weights: the schedule names those layers once
per pass, every call owns a cache of its own, and the first call of a pass carries a ``pass_input`` that adds
the pass's row of ``loop.step`` (and, from the second pass on, the embedding's output) to the stream first.

Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1.b``, ``l<i>.norm2``, ``l<i>.norm2.b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``final.norm.b``, ``head``.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
from ..config.lofirax import DenseMlp, LofiraxConfig, MoeMlp

MAX_POSITIONS = 1 << 24          # angles are position x frequency in 32-bit: every integer up to here is exact


def lofirax_spec(cfg: LofiraxConfig) -> ModelSpec:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"size": W, "eps": cfg.norm_eps, "weight": name, "bias": name + ".b"})

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "gla":
            mixer = PartSpec("gla", {
                "hidden_size": W, "heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "tau": m.tau,
                "q_scale": m.dim ** -0.5, "eps": cfg.norm_eps, "decay_rank": m.rank,
                "q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o", "norm": "mix.norm",
                "a1": "mix.a1", "a2": "mix.a2", "a2_bias": "mix.a2.b",
            })
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "heads": m.heads, "plain_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "rotary_dims": m.rot_dims, "theta": m.rot_base,
                "eps": cfg.norm_eps, "sink": "mix.sink",
                "q": "mix.q", "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o",
            })
        if isinstance(L.mlp, DenseMlp):
            ffn = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": L.mlp.ff, "activation": "gelu_tanh",
                                         "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
        elif isinstance(L.mlp, MoeMlp):
            shared = None
            if L.mlp.shared_ff:
                shared = {"intermediate_size": L.mlp.shared_ff, "gate": "mlp.shared.gate", "up": "mlp.shared.up",
                          "down": "mlp.shared.down", "token_gate": "mlp.shared.sg"}
            ffn = PartSpec("routed_experts", {
                "hidden_size": W, "experts": L.mlp.experts, "top": L.mlp.top, "intermediate_size": L.mlp.ff,
                "activation": "silu", "score": "sigmoid", "groups": L.mlp.groups, "keep_groups": L.mlp.keep,
                "group_score_of": 2, "weight_eps": 1e-20,
                "router": "mlp.router", "correction": "mlp.correction",
                "expert": "mlp.e{}.", "gate": "gate", "up": "up", "down": "down", "shared": shared,
            })
        else:
            ffn = PartSpec("none", {})
        block = PartSpec("pre_norm", {"pre_mixer_norm": norm("norm1"),
                                      "pre_ffn_norm": norm("norm2") if L.mlp is not None else None})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, prefix=f"l{i}."))

    n = len(layers)
    if cfg.loop is None:
        schedule = [ScheduleEntry(i) for i in range(n)]
    else:
        lp = cfg.loop
        schedule = [ScheduleEntry(i) for i in range(lp.start)]
        for t in range(lp.times):
            for i in range(lp.start, lp.stop):
                before = None
                if i == lp.start:
                    before = PartSpec("pass_input", {"hidden_size": W, "rows": lp.times, "row": t, "table": "loop.step",
                                                     "add_embedding": t > 0})
                schedule.append(ScheduleEntry(i, before=before))
        schedule += [ScheduleEntry(i) for i in range(lp.stop, n)]

    return ModelSpec(
        architecture="Lofirax",
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale,
                                         "weight": "embed"}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "softcap": cfg.logit_softcap,
                                      "scale": None, "weight": "head", "tied_to": None}),
        max_positions=MAX_POSITIONS,
        stop_ids=(),
    )


register_architecture("Lofirax", LofiraxConfig, lofirax_spec, native=False)
