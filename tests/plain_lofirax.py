"""Lofirax, stated plainly: one slow function per mechanism, in 64-bit floats on the CPU.

This file is the tests' oracle.  It shares no code with the library: it reads a
configuration dictionary (the keys of config.json) and a dictionary of tensors by
name, and runs one sequence token by token where the mechanism is a recurrence.

Notation: ``W`` is the model's width, ``h`` a mixer's or feed-forward's input
[tokens, W], all matrices are stored [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def f64(t: torch.Tensor) -> torch.Tensor:
    return t.to(F)


def same(x):
    return x


def to_bf16(x: torch.Tensor) -> torch.Tensor:
    """What a 16-bit engine stores: the value rounded to bfloat16 (used only to size the tests' tolerances)."""
    return x.to(torch.bfloat16).to(F)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def gated(h, gate, up, down, act, rnd=same):
    return rnd(act(h @ gate.T) * (h @ up.T)) @ down.T


def gla(h, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float, state: Optional[torch.Tensor] = None, rnd=same):
    """Gated linear attention over one sequence.  ``state`` [heads, dim, vdim] is carried in and returned."""
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = rnd(h @ t[p + "q"].T).view(T, H, D) * D ** -0.5
    k = rnd(h @ t[p + "k"].T).view(T, H, D)
    v = rnd(h @ t[p + "v"].T).view(T, H, V)
    z = (h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        S = alpha[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hdv,hd->hv", S, q[i])
    o = rms_norm(o, t[p + "norm"], eps).reshape(T, H * V)
    return rnd(o * silu(rnd(h @ t[p + "g"].T))) @ t[p + "o"].T, S


def rotate_half(x, pos, dims: int, base: float):
    """The first ``dims`` entries of the last axis, pair (i, i + dims/2), turned by pos * base^(-2i/dims)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = pos.to(F)[:, None] * f
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(a).view(shape), torch.sin(a).view(shape)
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], dim=-1)


def latent_attention(h, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float, first_pos: int = 0, past=None, rnd=same):
    """Latent attention over one sequence.  ``past`` = (latents, rotated key parts) of earlier tokens."""
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(first_pos, first_pos + T)
    q = (h @ t[p + "q"].T).view(T, H, D + R)
    q_plain, q_rot = rnd(q[..., :D]), rnd(rotate_half(q[..., D:], pos, m["rot"]["dims"], float(m["rot"]["base"])))
    d = h @ t[p + "dkv"].T
    c = rnd(rms_norm(d[:, :C], t[p + "dkv.norm"], eps))
    k_rot = rnd(rotate_half(d[:, C:], pos, m["rot"]["dims"], float(m["rot"]["base"])))
    if past is not None:
        c, k_rot = torch.cat([past[0], c]), torch.cat([past[1], k_rot])
    n = c.shape[0]
    k_plain = rnd(c @ t[p + "uk"].T).view(n, H, D)
    v = rnd(c @ t[p + "uv"].T).view(n, H, V)
    s = (torch.einsum("thd,nhd->htn", q_plain, k_plain) + torch.einsum("thr,nr->htn", q_rot, k_rot)) * float(m["scale"])
    qpos = pos[:, None]
    kpos = torch.arange(n)[None, :]
    s = s.masked_fill((kpos > qpos)[None], float("-inf"))
    sink = t[p + "sink"]
    mx = torch.maximum(s.max(-1).values, sink[:, None].expand(H, T))
    e = torch.exp(s - mx[..., None])
    w = e / (e.sum(-1) + torch.exp(sink[:, None] - mx))[..., None]
    o = rnd(torch.einsum("htn,nhv->thv", rnd(w), v).reshape(T, H * V))      # tensor-core kernels round the weights that meet v
    return o @ t[p + "o"].T, (c, k_rot)


MARGINS = None          # a list to collect, per router call, every token's smallest margin (see route)


def route(h, r: dict, t: Dict[str, torch.Tensor], p: str):
    """(chosen experts [tokens, top], their weights [tokens, top]).  If MARGINS is a list, also appends [tokens]: how far
    the choice was from going another way (the last winner's lead over the best loser, and the last kept group's lead
    over the best group left out), so that a test can set aside tokens whose choice a rounding error may turn."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ t[p + "router"].T)
    choice = s + t[p + "correction"]
    margin = torch.full((h.shape[0],), float("inf"), dtype=F)
    g = r.get("groups")
    if g:
        per = E // g["count"]
        grouped = choice.view(-1, g["count"], per)
        gs = grouped.topk(min(2, per), dim=-1).values.sum(-1)
        keep = gs.topk(g["keep"], dim=-1).indices
        if g["keep"] < g["count"]:
            both = gs.topk(g["keep"] + 1, dim=-1).values
            margin = both[:, -2] - both[:, -1]
        ok = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, keep, True)
        choice = grouped.masked_fill(~ok[..., None], float("-inf")).reshape(-1, E)
    idx = choice.topk(top, dim=-1).indices
    if top < E:
        both = choice.topk(top + 1, dim=-1).values
        margin = torch.minimum(margin, both[:, -2] - both[:, -1])
    if MARGINS is not None:
        MARGINS.append(margin)
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20)


def routing_margins(cfg: dict, tensors, ids) -> torch.Tensor:
    """Per position: the smallest margin of any of its routing decisions (infinite for a model without experts)."""
    global MARGINS
    MARGINS = []
    try:
        forward(cfg, tensors, ids)
        out = torch.full((len(ids),), float("inf"), dtype=F)
        for m in MARGINS:
            out = torch.minimum(out, m)
        return out
    finally:
        MARGINS = None


def moe(h, mlp: dict, t: Dict[str, torch.Tensor], p: str, rnd=same):
    idx, w = route(h, mlp["router"], t, p)
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F)
    for i in range(h.shape[0]):
        for j, e in enumerate(idx[i].tolist()):
            q = f"{p}e{e}."
            out[i] += w[i, j] * gated(h[i:i + 1], t[q + "gate"], t[q + "up"], t[q + "down"], silu, rnd)[0]
    if mlp.get("shared"):
        q = p + "shared."
        out = out + torch.sigmoid(h @ t[q + "sg"].T) * gated(h, t[q + "gate"], t[q + "up"], t[q + "down"], silu, rnd)
    return out


def schedule(cfg: dict) -> List[tuple]:
    """The layer runs in order: (layer, number of the pass if it is the first layer of a pass, else None)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for rep in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, rep if i == loop["start"] else None))
    return runs + [(i, None) for i in range(loop["stop"], n)]


class Plain:
    """One sequence, fed in pieces: ``feed(tokens)`` returns (logits of these tokens, stream after every layer run)."""

    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor], rnd=same):
        self.cfg = cfg
        self.rnd = rnd
        self.t = {k: f64(v) for k, v in tensors.items()}
        self.runs = schedule(cfg)
        self.memory = [None] * len(self.runs)
        self.n = 0

    def feed(self, tokens):
        cfg, t = self.cfg, self.t
        eps = float(cfg["norm"]["eps"])
        x0 = t["embed"][torch.as_tensor(tokens)] * float(cfg["embedding"]["scale"])
        x = x0.clone()
        after = []
        for r, (i, rep) in enumerate(self.runs):
            L = cfg["layers"][i]
            if rep is not None:
                if rep > 0:
                    x = x + x0
                x = x + t["loop.step"][rep]
            p = f"l{i}."
            rnd = self.rnd
            h = rnd(layer_norm(x, t[p + "norm1"], t[p + "norm1.b"], eps))
            if L["type"] == "gla":
                y, self.memory[r] = gla(h, L["mixer"], t, p + "mix.", eps, self.memory[r], rnd)
            elif L["type"] == "latent_attention":
                y, self.memory[r] = latent_attention(h, L["mixer"], t, p + "mix.", eps, self.n, self.memory[r], rnd)
            else:
                raise ValueError(L["type"])
            x = x + y
            if L.get("mlp"):
                h = rnd(layer_norm(x, t[p + "norm2"], t[p + "norm2.b"], eps))
                if L["mlp"]["kind"] == "dense":
                    y = gated(h, t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"], gelu_tanh, rnd)
                else:
                    y = moe(h, L["mlp"], t, p + "mlp.", rnd)
                x = x + y
            after.append(x.clone())
        self.n += len(tokens)
        z = self.rnd(layer_norm(x, t["final.norm"], t["final.norm.b"], eps)) @ t["head"].T
        cap = cfg.get("logit_softcap")
        if cap:
            z = float(cap) * torch.tanh(z / float(cap))
        return z, torch.stack(after)


def forward(cfg: dict, tensors, ids, rnd=same) -> torch.Tensor:
    """Logits of a whole sequence, [tokens, vocab]."""
    return Plain(cfg, tensors, rnd).feed(list(ids))[0]


def forward_stepwise(cfg: dict, tensors, ids, first: int = 1) -> torch.Tensor:
    """The same logits, from ``first`` tokens at once and then one token at a time."""
    m = Plain(cfg, tensors)
    out = [m.feed(list(ids[:first]))[0]] + [m.feed([t])[0] for t in ids[first:]]
    return torch.cat(out)


def generate_greedy(cfg: dict, tensors, prompt, n_new: int) -> List[int]:
    m = Plain(cfg, tensors)
    z = m.feed(list(prompt))[0]
    out = []
    for _ in range(n_new):
        out.append(int(z[-1].argmax()))
        z = m.feed([out[-1]])[0]
    return out


def load_folder(folder: str):
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: f64(v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
