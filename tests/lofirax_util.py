"""Shared pieces of the Lofirax tests: small configurations made up here, model folders with random weights drawn
here (not by the library), prompts and tolerances."""
import json
import math
import os

import torch

import plain_lofirax as plain


def gla(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(vocab, width, layers, loop=None, emb_scale=1.0, eps=1e-5, softcap=None):
    c = {"architecture": "Lofirax", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "norm": {"eps": eps},
         "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if softcap:
        c["logit_softcap"] = softcap
    return c


# A: attention first; the middle layer alone runs three times; experts in three groups of two of which two are kept;
#    value heads wider than key heads; a gla layer without a feed-forward.
CFG_A = config(200, 64, [
    ("latent_attention", latent(2, 16, 8, 40, 40, 0.3, base=100.0), moe(6, 2, 32, groups=(3, 2), shared=48)),
    ("gla", gla(3, 8, 16, 4.0), dense(96)),
    ("gla", gla(2, 24, 8, 1.0), None),
], loop=(1, 2, 3), emb_scale=3.0, eps=1e-5, softcap=10.0)
# B: no repeated span, no cap; one gla head; a rotation that turns only half of the rotated part; experts without
#    groups and without a shared expert, one of three chosen; a width that is no multiple of 16.
CFG_B = config(301, 72, [
    ("gla", gla(1, 20, 40, 2.0), moe(3, 1, 24)),
    ("latent_attention", latent(3, 24, 16, 24, 24, 0.25, base=500.0, dims=8), dense(100)),
    ("latent_attention", latent(1, 8, 32, 16, 48, 0.2), moe(8, 3, 16, groups=(2, 1), shared=24)),
], emb_scale=1.0, eps=1e-4)
# C: sizes that the tensor-core kernels take in bfloat16; the whole model is one repeated span that runs twice.
CFG_C = config(512, 128, [
    ("gla", gla(4, 32, 32, 8.0), dense(256)),
    ("latent_attention", latent(4, 32, 32, 64, 64, 0.125), moe(8, 2, 64, groups=(4, 2), shared=128)),
    ("gla", gla(2, 64, 64, 12.0), moe(4, 4, 64, groups=(4, 4))),
    ("latent_attention", latent(2, 96, 32, 128, 80, 0.09, base=250000.0), dense(128)),
], loop=(0, 4, 2), emb_scale=8.0, eps=1e-6, softcap=25.0)

# D: sizes that fit no fast path and no vector load: a width of 50, a vocabulary of 77, a latent of 20, heads of 6, 10 and 14,
#    as many groups as experts, an attention layer without a feed-forward at the end, the first layer alone repeated.
CFG_D = config(77, 50, [
    ("gla", gla(2, 6, 10, 3.0), moe(5, 2, 12, groups=(5, 3), shared=20)),
    ("latent_attention", latent(2, 10, 6, 14, 20, 0.3, base=50.0, dims=4), None),
], loop=(0, 1, 2), emb_scale=0.5, eps=1e-3, softcap=5.0)

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
RANKS = {"A": [0, 4, 7], "B": [5, 0, 0], "C": [16, 0, 8, 0], "D": [3, 0]}          # the decay's rank per gla layer: the files decide it


def random_weights(cfg: dict, seed: int, ranks) -> dict:
    """bfloat16 weights, drawn here: matrices N(0, 1/fan_in), gains near 1, biases and sinks spread."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def mat(o, i, scale=1.0):
        return torch.randn(o, i, generator=g) * (scale / math.sqrt(i))

    def gain(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)

    def small(n, s=0.2):
        return s * torch.randn(n, generator=g)
    out["embed"] = torch.randn(V, W, generator=g)
    if cfg.get("loop"):
        out["loop.step"] = torch.randn(cfg["loop"]["times"], W, generator=g) * 0.5
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"], out[p + "norm1.b"] = gain(W), small(W)
        if L["type"] == "gla":
            HD, HV = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out[p + "mix.q"], out[p + "mix.k"] = mat(HD, W, 2.0), mat(HD, W, 2.0)
            out[p + "mix.v"], out[p + "mix.g"] = mat(HV, W), mat(HV, W, 2.0)
            out[p + "mix.o"] = mat(W, HV)
            out[p + "mix.norm"] = gain(m["vdim"])
            out[p + "mix.a1"] = mat(ranks[i], W, 2.0)
            out[p + "mix.a2"] = mat(HD, ranks[i], 2.0)
            out[p + "mix.a2.b"] = 2.0 + torch.randn(HD, generator=g)
        else:
            H, D, R, Vd, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out[p + "mix.q"] = mat(H * (D + R), W, 3.0)
            out[p + "mix.dkv"] = mat(C + R, W, 3.0)
            out[p + "mix.dkv.norm"] = gain(C)
            out[p + "mix.uk"], out[p + "mix.uv"] = mat(H * D, C, 2.0), mat(H * Vd, C)
            out[p + "mix.sink"] = torch.randn(H, generator=g)
            out[p + "mix.o"] = mat(W, H * Vd)
        f = L["mlp"]
        if f is not None:
            out[p + "norm2"], out[p + "norm2.b"] = gain(W), small(W)
        if f is not None and f["kind"] == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = mat(f["ff"], W, 1.5), mat(f["ff"], W, 1.5), mat(W, f["ff"])
        elif f is not None:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            out[p + "mlp.router"] = mat(E, W, 2.0)
            out[p + "mlp.correction"] = small(E, 0.3)
            for e in range(E):
                q = f"{p}mlp.e{e}."
                out[q + "gate"], out[q + "up"], out[q + "down"] = mat(ff, W, 1.5), mat(ff, W, 1.5), mat(W, ff)
            if f.get("shared"):
                q, sf = p + "mlp.shared.", f["shared"]["ff"]
                out[q + "gate"], out[q + "up"], out[q + "down"] = mat(sf, W, 1.5), mat(sf, W, 1.5), mat(W, sf)
                out[q + "sg"] = mat(1, W, 2.0)
    out["final.norm"], out["final.norm.b"] = gain(W), small(W)
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
    """Per position: the difference with its mean taken off, root mean square over the vocabulary, relative to the
    root mean square of the wanted logits (their mean taken off too)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(dim=-1, keepdim=True)
    w = want - want.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)


TOL32 = 3e-5
ROUTING_MARGIN = 0.03          # choice scores are sigmoids of sums of a few dozen products of 16-bit numbers
ROUTING_TURNS = 0.005          # under this margin the 16-bit engine is taken to have chosen otherwise
BF16_FLOOR, BF16_FACTOR = 2e-2, 3.0
_BUDGET = {}


def tolerance(key, cfg, w, ids, dtype: str) -> torch.Tensor:
    """One tolerance per position.  float32: rounding only.  bfloat16: the larger of 2e-2 and three times what the plain
    implementation itself loses at that position when it rounds what a 16-bit engine stores (never taken from the
    library's output); positions whose routing hangs on less than ROUTING_MARGIN are not compared."""
    if dtype == "float32":
        return torch.full((len(ids),), TOL32, dtype=torch.float64)
    k = (key, tuple(ids))
    if k not in _BUDGET:
        lost = position_errors(plain.forward(cfg, w, ids, rnd=plain.to_bf16), plain.forward(cfg, w, ids))
        tol = torch.clamp(BF16_FACTOR * lost, min=max(BF16_FLOOR, float(lost.median()) * BF16_FACTOR))
        # a routing decision that hangs on less than the rounding of its inputs may go either way in 16 bits: such a
        # position is no test of anything (the design's own checks rest on no close call either)
        margins = plain.routing_margins(cfg, w, ids)
        tol[margins < ROUTING_MARGIN] = float("inf")
        turned = (margins < ROUTING_TURNS).nonzero().flatten()
        if turned.numel():
            # ... and a token that did go another way changes what every later token reads from the cache and the state
            tol[int(turned[0]):] = float("inf")
        _BUDGET[k] = tol
    return _BUDGET[k]


def worst_ratio(got: torch.Tensor, want: torch.Tensor, tol) -> float:
    """1 is the border: no position over one and a half times its tolerance, at most one in fifty (or one) over it."""
    r = position_errors(got, want) / tol
    over = int((r > 1.0).sum())
    allowed = max(1, r.numel() // 50)
    return max(float(r.max()) / 1.5, over / (allowed + 0.5))
