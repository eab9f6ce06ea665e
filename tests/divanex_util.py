"""Shared pieces of the Divanex tests: small configurations (none with the sizes of a released model), model
folders with random weights made here (not by the library), prompts and tolerances."""
import json
import math
import os

import torch

import plain_divanex as plain


def attn(heads, kv, dim, scale, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(vocab, width, layers, alpha=1.0, logit_scale=1.0, emb_scale=1.0, eps=1e-5, side=None):
    c = {"architecture": "Divanex", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale},
         "norm": {"eps": eps}, "postln_alpha": alpha, "logit_scale": logit_scale,
         "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


# A: the state-space layer first and with a feed-forward, attention without one; two kv heads, two groups, two
#    norm groups, three taps, a temperature that steps every 4 positions, head sizes 16 and 32.
CFG_A = config(200, 64, [
    ("mamba2", ssm(2, 16, 8, 2, 3, 2), dense(96, 2.5)),
    ("attention", attn(4, 2, 16, 0.9, softcap=20.0, q_temp=(0.3, 4)), None),
    ("attention", attn(2, 2, 32, 0.6), dense(80, 0.75)),
], alpha=1.5, logit_scale=0.5, emb_scale=3.0, eps=1e-5, side=8)
# B: widths that are multiples of neither 16 nor 8, one kv head for three heads, a head size of 24, two taps, a state
#    of 20, no side input, alpha and the logit scale equal to 1.
CFG_B = config(301, 72, [
    ("attention", attn(3, 1, 24, 1.1, softcap=8.0, q_temp=(0.8, 7)), dense(100, 1.0)),
    ("mamba2", ssm(3, 24, 20, 1, 2, 3), None),
    ("mamba2", ssm(6, 12, 20, 3, 5, 1), dense(52, 3.0)),
], alpha=1.0, logit_scale=1.0, emb_scale=1.0, eps=1e-4)
# C: sizes that the tensor-core kernels take in bfloat16 (head size 64, a state of 64, widths that are multiples
#    of 64), four query heads per kv head.
CFG_C = config(512, 128, [
    ("attention", attn(4, 1, 64, 0.5, softcap=25.0, q_temp=(0.4, 32)), dense(256, 1.5)),
    ("mamba2", ssm(4, 32, 64, 2, 4, 1), None),
    ("attention", attn(2, 2, 64, 0.4), None),
    ("mamba2", ssm(2, 64, 32, 1, 4, 2), dense(128, 1.0)),
], alpha=1.75, logit_scale=0.125, emb_scale=8.0, eps=1e-6, side=32)

# D: sizes that fit no fast path: a head size of 40 and one of 96, one state-space head, a state of 256 beside
#    head values of 8, one tap, as many groups and norm groups as heads, a width of 1,000, an odd vocabulary, a side
#    input of 12 columns; attention only at the end.
CFG_D = config(1001, 1000, [
    ("mamba2", ssm(1, 8, 256, 1, 1, 1), None),
    ("mamba2", ssm(5, 16, 24, 5, 2, 5), dense(72, 0.5)),
    ("attention", attn(5, 5, 40, 0.7, q_temp=(1.5, 3)), None),
    ("attention", attn(6, 2, 96, 0.3, softcap=12.0), dense(200, 4.0)),
], alpha=0.8, logit_scale=2.0, emb_scale=0.5, eps=1e-3, side=12)
# E: heads of 128 (the tensor-core attention kernels in bfloat16, four query heads per kv head), a state of 128,
#    every layer of one kind with a feed-forward, then every layer of the other without.
CFG_E = config(384, 256, [
    ("attention", attn(8, 2, 128, 0.25, softcap=40.0, q_temp=(0.2, 16)), dense(512, 2.0)),
    ("attention", attn(2, 1, 128, 0.35), dense(384, 1.25)),
    ("mamba2", ssm(8, 32, 128, 4, 3, 2), None),
    ("mamba2", ssm(4, 64, 128, 1, 4, 4), None),
], alpha=1.25, logit_scale=0.75, emb_scale=2.0, eps=1e-5, side=8)

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D, "E": CFG_E}


def random_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 weights, drawn here: matrices N(0, 1/fan_in), gains near 1, decays and step sizes spread."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def mat(o, i, scale=1.0):
        return torch.randn(o, i, generator=g) * (scale / math.sqrt(i))

    def gain(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)
    out["embed"] = torch.randn(V, W, generator=g)
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = torch.randn(V, side["dim"] * len(cfg["layers"]), generator=g)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = gain(W)
        if L["type"] == "attention":
            out[p + "mix.q"] = mat(m["heads"] * m["dim"], W)
            out[p + "mix.k"] = mat(m["kv_heads"] * m["dim"], W)
            out[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        else:
            inner = m["heads"] * m["vdim"]
            ch = inner + 2 * m["groups"] * m["state"]
            out[p + "mix.in"] = mat(inner + ch + m["heads"], W)
            out[p + "mix.conv"] = torch.randn(ch, m["conv"], generator=g) * 0.5
            out[p + "mix.conv.b"] = torch.randn(ch, generator=g) * 0.2
            out[p + "mix.dt_bias"] = torch.randn(m["heads"], generator=g) - 1.0
            out[p + "mix.A_log"] = torch.rand(m["heads"], generator=g) * 2.0 - 1.5
            out[p + "mix.D"] = gain(m["heads"])
            out[p + "mix.norm"] = gain(inner)
            out[p + "mix.o"] = mat(W, inner)
        if L["mlp"] is not None:
            out[p + "norm2"] = gain(W)
            out[p + "mlp.gate"] = mat(L["mlp"]["ff"], W, 1.5)
            out[p + "mlp.up"] = mat(L["mlp"]["ff"], W, 1.5)
            out[p + "mlp.down"] = mat(W, L["mlp"]["ff"])
        if side:
            out[p + "side.gate"] = mat(side["dim"], W)
            out[p + "side.proj"] = mat(W, side["dim"])
            out[p + "side.norm"] = gain(W) * 0.5
    out["final.norm"] = gain(W)
    out["head"] = mat(V, W)
    return {k: v.to(torch.bfloat16).contiguous() for k, v in out.items()}


def write_folder(folder: str, cfg: dict, weights: dict) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(weights, os.path.join(folder, "model.safetensors"))
    return folder


def prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def position_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: the difference with its mean taken off, root mean square over the vocabulary, relative to
    the root mean square of the wanted logits (their mean taken off too)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(dim=-1, keepdim=True)
    w = want - want.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)


def logit_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """The largest of :func:`position_errors`."""
    return float(position_errors(got, want).max())


TOL32 = 3e-5
BF16_FLOOR, BF16_FACTOR = 2e-2, 3.0
_BUDGET = {}


def tolerance(key, cfg, w, ids, dtype: str) -> torch.Tensor:
    """One tolerance per position of the sequence.  float32: rounding only.  bfloat16: the largest of 2e-2, three
    times what the oracle itself loses AT THAT POSITION when it rounds what a 16-bit engine stores, and what it loses
    at its worst position of this sequence; taken from the oracle alone.  This design has positions where rounding
    costs ten times the usual (a state-space output that nearly cancels before its norm multiplies whatever error its
    input carries): which positions those are is a property of the weights and the tokens, but how large the error
    comes out at one of them is a draw, the engine's and the oracle's being two draws of the same wide distribution
    (a state-space mixer run wholly in 32-bit inside the 16-bit engine leaves such a position's error where it was)."""
    if dtype == "float32":
        return torch.full((len(ids),), TOL32, dtype=torch.float64)
    k = (key, tuple(ids))
    if k not in _BUDGET:
        exact = plain.forward(cfg, w, ids)
        rounded = plain.forward(cfg, w, ids, rnd=plain.to_bf16)
        lost = position_errors(rounded, exact)
        _BUDGET[k] = torch.clamp(BF16_FACTOR * lost, min=max(BF16_FLOOR, float(lost.max())))
    return _BUDGET[k]


def worst_ratio(got: torch.Tensor, want: torch.Tensor, tol: torch.Tensor) -> float:
    """How far the positions' errors are from failing, 1 being the border: no position may be over one and a half
    times its tolerance, and at most one position in fifty (or one) over its tolerance at all.  ``tol``: one number
    per position, or one for all."""
    r = position_errors(got, want) / tol
    over = int((r > 1.0).sum())
    allowed = max(1, r.numel() // 50)
    return max(float(r.max()) / 1.5, over / (allowed + 0.5))
