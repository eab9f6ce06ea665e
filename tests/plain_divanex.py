"""A plain, slow Divanex: whole sequences or token by token, no cache manager, no batching, one
function per mechanism.

This file is the oracle of the Divanex tests.  It shares no code with ``trapetum_b200``: it reads a
model folder with the ``safetensors`` library and computes with ordinary torch operations on the CPU,
one sequence at a time, in float64 unless asked otherwise.

The design in this file's own notation (x is the residual stream, one row per token; t a token's
position in its sequence, counted from 0; ``rms(v) = sqrt(mean(v^2) + eps)``):

    x0        = E[token] * embedding.scale
    layer     : x <- N1(alpha x + mixer(x));   if the layer has a feed-forward: x <- N2(alpha x + ff(x));
                then the per-layer token input:  x <- x + Ns(side(x, token))
    N(v)      = v / rms(v) * w
    attention : q = Wq x, k = Wk x, v = k (before any norm); q, k <- q / rms(q), k / rms(k) per head;
                q <- q * (1 + coef * ln(floor((t + 1) / every) + 1));
                s = cap * tanh(scale * q.k / cap) over keys j <= t; softmax; out = Wo concat(heads)
    mamba2    : [z | xs | B | C | dt] = Win x;  [xs | B | C] <- silu(causal conv + bias);
                dt <- softplus(dt + dt_bias);  S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t xs_t^T;
                y_t = S_t^T C_t + D xs_t;  y <- y * silu(z);  y <- grouped rms norm * w;  out = Wo y
    ff        : g = min(Wg x, L), u = clamp(Wu x, -L, L);  out = Wd (g sigmoid(1.702 g) (u + 1))
    side      : e = Es[token][i*d : (i+1)*d];  out = Wp (gelu_tanh(Wsg x) * e)
    logits    = head N(x) * logit_scale
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

DT = torch.float64


def load_folder(folder: str, dtype=DT) -> Tuple[dict, Dict[str, torch.Tensor]]:
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    for k, v in load_file(os.path.join(folder, "model.safetensors")).items():
        w[k] = v.to(dtype) if v.is_floating_point() else v
    return cfg, w


def _same(x):
    return x


def to_bf16(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 and back: what a 16-bit activation buffer does to its contents."""
    return x.to(torch.bfloat16).to(x.dtype)


# ----------------------------------------------------------------------------
# Mechanisms
# ----------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def embed(ids: Sequence[int], table: torch.Tensor, scale: float) -> torch.Tensor:
    return table[torch.tensor(list(ids), dtype=torch.long)] * scale


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((t + 1) / every) + 1), one factor per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(DT) + 1.0)


def attention_scores(q: torch.Tensor, k: torch.Tensor, scale: float, cap: Optional[float]) -> torch.Tensor:
    """q [Tq, d], k [Tk, d] -> [Tq, Tk] scores before the mask."""
    s = (q @ k.T) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    return s


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict, eps: float,
                    pos0: int = 0, past: Optional[dict] = None, rnd=_same) -> torch.Tensor:
    """h [T, width]: the tokens at positions pos0.. of one sequence.  ``past`` holds the earlier tokens'
    normed keys and values under "k" and "v" and is extended in place."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[pre + "q"].T).view(T, H, d)
    kraw = (h @ w[pre + "k"].T).view(T, G, d)
    v = rnd(kraw)                                            # v is the raw k projection (taken before k is normed)
    q = unit_rms(q, eps)
    k = rnd(unit_rms(kraw, eps))
    pos = torch.arange(pos0, pos0 + T)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, qt["coef"], qt["every"])[:, None, None].to(q.dtype)
    q = rnd(q)
    if past is not None:
        if "k" in past:
            k, v = torch.cat([past["k"], k]), torch.cat([past["v"], v])
        past["k"], past["v"] = k, v
    Tk = k.shape[0]
    kpos = torch.arange(Tk)
    mask = kpos[None, :] <= pos[:, None]                      # causal: key j is seen from position i >= j
    out = torch.empty(T, H, m["vdim"], dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = attention_scores(q[:, hh], k[:, g], m["scale"], m.get("softcap"))
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, hh] = p @ v[:, g]
    return rnd(out.reshape(T, H * m["vdim"])) @ w[pre + "o"].T


def causal_conv(u: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, before: torch.Tensor) -> torch.Tensor:
    """u [T, C]; weight [C, taps], whose last column multiplies the current token; ``before`` [taps-1, C]
    holds the inputs that came before u's first row (zeros at a sequence's start)."""
    taps = weight.shape[1]
    full = torch.cat([before, u])
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + full[j:j + u.shape[0]] * weight[:, j]
    return out + bias


def ssm_scan(xs: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor,
             D: torch.Tensor, S: torch.Tensor, groups: int) -> torch.Tensor:
    """xs [T, heads, P], Bm and Cm [T, groups, N], dt [T, heads] (already positive), S [heads, N, P] is
    updated in place.  Returns y [T, heads, P]."""
    T, H, P = xs.shape
    y = torch.empty_like(xs)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // groups)
            a = torch.exp(-torch.exp(A_log[hh]) * dt[t, hh])
            S[hh] = a * S[hh] + dt[t, hh] * torch.outer(Bm[t, g], xs[t, hh])
            y[t, hh] = S[hh].T @ Cm[t, g] + D[hh] * xs[t, hh]
    return y


def grouped_rmsnorm(y: torch.Tensor, w: torch.Tensor, parts: int, eps: float) -> torch.Tensor:
    T, n = y.shape
    return (unit_rms(y.view(T, parts, n // parts), eps).reshape(T, n)) * w


def mamba2_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict, eps: float,
                 state: Optional[dict] = None, rnd=_same) -> torch.Tensor:
    """``state`` holds "S" [heads, N, P] and "conv" [taps-1, channels] of the sequence and is updated in place."""
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    ch = inner + 2 * G * N
    if state is None:
        state = {}
    if "S" not in state:
        state["S"] = torch.zeros(H, N, P, dtype=h.dtype)
        state["conv"] = torch.zeros(taps - 1, ch, dtype=h.dtype)
    proj = h @ w[pre + "in"].T
    z, xbc, dt = proj[:, :inner], rnd(proj[:, inner:inner + ch]), proj[:, inner + ch:]
    conv = causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"], state["conv"])
    state["conv"] = torch.cat([state["conv"], xbc])[-(taps - 1):] if taps > 1 else state["conv"]
    xbc = rnd(silu(conv))
    xs = xbc[:, :inner].view(T, H, P)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    y = ssm_scan(xs, Bm, Cm, dt, w[pre + "A_log"], w[pre + "D"], state["S"], G).reshape(T, inner)
    y = y * silu(rnd(z))
    y = rnd(grouped_rmsnorm(y, w[pre + "norm"], m["norm_groups"], eps))
    return y @ w[pre + "o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, limit: float, rnd=_same) -> torch.Tensor:
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def token_side(h: torch.Tensor, ids: Sequence[int], w: Dict[str, torch.Tensor], pre: str, layer: int, dim: int,
               rnd=_same) -> torch.Tensor:
    e = w["side.embed"][torch.tensor(list(ids), dtype=torch.long)][:, layer * dim:(layer + 1) * dim]
    g = rnd(gelu_tanh(h @ w[pre + "gate"].T) * e)
    return g @ w[pre + "proj"].T


# ----------------------------------------------------------------------------
# The model
# ----------------------------------------------------------------------------
def new_state(cfg: dict) -> List[dict]:
    return [{} for _ in cfg["layers"]]


def layer(x: torch.Tensor, ids: Sequence[int], w, cfg: dict, i: int, pos0: int, st: dict, rnd=_same) -> torch.Tensor:
    L = cfg["layers"][i]
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    pre = f"l{i}."
    if L["type"] == "attention":
        b = attention_mixer(rnd(x), w, pre + "mix.", L["mixer"], eps, pos0, st, rnd)
    elif L["type"] == "mamba2":
        b = mamba2_mixer(rnd(x), w, pre + "mix.", L["mixer"], eps, st, rnd)
    else:
        raise ValueError(L["type"])
    x = rmsnorm(alpha * x + b, w[pre + "norm1"], eps)
    if L.get("mlp") is not None:
        if L["mlp"]["kind"] != "dense":
            raise ValueError(L["mlp"]["kind"])
        x = rmsnorm(alpha * x + dense_ff(rnd(x), w, pre + "mlp.", L["mlp"]["limit"], rnd), w[pre + "norm2"], eps)
    side = cfg.get("token_side")
    if side:
        y = token_side(rnd(x), ids, w, pre + "side.", i, side["dim"], rnd)
        x = x + rmsnorm(y, w[pre + "side.norm"], eps)
    return x


def forward(cfg: dict, w, ids: Sequence[int], state: Optional[List[dict]] = None, pos0: int = 0, rnd=_same,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of the tokens ``ids`` at positions pos0.. of one sequence; ``state`` (from
    :func:`new_state`) carries the sequence from call to call."""
    if state is None:
        state = new_state(cfg)
    x = embed(ids, w["embed"], cfg["embedding"]["scale"])
    for i in range(len(cfg["layers"])):
        x = layer(x, ids, w, cfg, i, pos0, state[i], rnd)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rnd(rmsnorm(x, w["final.norm"], cfg["norm"]["eps"]))
    return (x @ w["head"].T) * cfg["logit_scale"]


def forward_stepwise(cfg: dict, w, ids: Sequence[int], first: int = 1) -> torch.Tensor:
    """The same logits, computed from ``first`` tokens at once and the rest one token at a time."""
    st = new_state(cfg)
    outs = [forward(cfg, w, ids[:first], st, 0)]
    for t in range(first, len(ids)):
        outs.append(forward(cfg, w, ids[t:t + 1], st, t))
    return torch.cat(outs)


def generate_greedy(cfg: dict, w, prompt: Sequence[int], n_new: int) -> List[int]:
    st = new_state(cfg)
    logits = forward(cfg, w, list(prompt), st, 0)
    out: List[int] = []
    pos = len(prompt)
    for _ in range(n_new):
        tok = int(torch.argmax(logits[-1]))          # the smallest id on a tie
        out.append(tok)
        logits = forward(cfg, w, [tok], st, pos)
        pos += 1
    return out
