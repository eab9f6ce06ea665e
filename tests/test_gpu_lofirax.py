"""Lofirax on the GPU against the plain implementation: each mechanism alone, then the model through the engine
(whole prompts, the stream after every layer run, token by token, unequal batches, reused slots and pages, far keys,
sinks, long decoding, greedy generation, trace replay)."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lofirax as plain
import trapetum_b200 as tb
from conftest import ROOT, within
from lofirax_util import (CFG_A, CFG_B, CONFIGS, RANKS, TOL32, config, dense, gla, latent, moe, position_errors, prompts,
                          random_weights, tolerance, worst_ratio, write_folder)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F = torch.float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_folder(str(tmp_path_factory.mktemp("lofirax" + name)), cfg, random_weights(cfg, 21 + ord(name), RANKS[name]))
            for name, cfg in CONFIGS.items()}


@pytest.fixture(scope="module")
def oracles(folders):
    return {name: plain.load_folder(d) for name, d in folders.items()}


_MODELS = {}


def model_of(folders, name, dtype):
    if (name, dtype) not in _MODELS:
        _MODELS[(name, dtype)] = tb.load_model(folders[name], dtype, DEV)
    return _MODELS[(name, dtype)]


def close(got, want, tol, what, dtype):
    within(worst_ratio(got, want, tol), 1.0, dtype, what + " (error / tolerance)")


def near(got, want, dtype, what, rel32=2e-5, rel16=2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (rel32 if dtype == "float32" else rel16), f"{what} [{dtype}]: {err:.3e}"


def dev(t, dt=None):
    return t.to(device=DEV, dtype=dt) if dt is not None else t.to(DEV)


# =================================================================================================================
# Mechanisms alone
# =================================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows, width, splits", [(5, 72, 1), (130, 320, 3), (3, 1000, 2)])
def test_layer_norm_with_the_sum_before_it(rows, width, splits, dtype):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    h = torch.randn(rows, width, generator=g) * 4 + 3.0              # a mean far from zero: the variance is about the mean
    a = torch.randn(splits, rows, width, generator=g)
    w, b = 1 + 0.3 * torch.randn(width, generator=g), torch.randn(width, generator=g)
    hd = dev(h)
    out = ops.add_layernorm(hd, dev(a) if splits > 1 else dev(a[0]), dev(w), dev(b), 1e-5, DTYPES[dtype])
    s = h.double() + a.double().sum(0)
    near(hd, s, "float32", "the sum")
    near(out, plain.layer_norm(s, w.double(), b.double(), 1e-5), dtype, "layer norm")
    plain_only = ops.add_layernorm(dev(h), None, dev(w), dev(b), 1e-5, torch.float32)
    near(plain_only, plain.layer_norm(h.double(), w.double(), b.double(), 1e-5), "float32", "layer norm alone")
    x0, vec = torch.randn(rows, width, generator=g), torch.randn(width, generator=g)
    hd = dev(h)
    ops.add_rows(hd, dev(x0), dev(vec))
    near(hd, h.double() + x0.double() + vec.double(), "float32", "rows and a vector")
    ops.add_rows(hd, None, dev(vec))
    near(hd, h.double() + x0.double() + 2 * vec.double(), "float32", "a vector alone")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, D, V, rank, lens", [(3, 8, 16, 4, [19, 1, 8]), (1, 20, 40, 5, [33]), (2, 64, 70, 16, [9, 70]),
                                                 (2, 130, 32, 3, [12, 5]), (1, 16, 32, 2, [300, 64, 129])])
def test_gated_linear_attention_between_its_products(H, D, V, rank, lens, dtype):
    """Whole sequences in one call, then the same sequences continued from the states the first call left.  The
    longest case is cut into chunks in time (a chunk's edge at 64 and at 128: one sequence ends on it, one just after)."""
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(D * V)
    Wd, tau, eps = 48, 3.0, 1e-4
    m = {"heads": H, "dim": D, "vdim": V, "tau": tau}
    t = {"q": torch.randn(H * D, Wd, generator=g) / 5, "k": torch.randn(H * D, Wd, generator=g) / 5,
         "v": torch.randn(H * V, Wd, generator=g) / 5, "g": torch.randn(H * V, Wd, generator=g) / 3,
         "o": torch.eye(H * V), "norm": 1 + 0.2 * torch.randn(V, generator=g), "a1": torch.randn(rank, Wd, generator=g) / 4,
         "a2": torch.randn(H * D, rank, generator=g), "a2.b": 1.5 + torch.randn(H * D, generator=g)}
    t = {k: v.to(torch.bfloat16).double() for k, v in t.items()}
    B = len(lens)
    state = torch.zeros(B + 2, H * D * V, device=DEV)
    slots = torch.tensor([B + 1 - i for i in range(B)], dtype=torch.int32)        # slots in another order than the batch
    want_state = [None] * B
    for part in range(2):
        xs = [(torch.randn(n, Wd, generator=g)).to(torch.bfloat16).double() for n in lens]
        x = torch.cat(xs)
        proj = torch.cat([x @ t[k].T for k in ("q", "k", "v", "g")], dim=1)
        low = (x @ t["a1"].T)
        low3 = torch.stack([low * 0.25, low * 0.75])                               # two partial sums
        starts = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        tok_seq = torch.repeat_interleave(torch.arange(B), torch.tensor(lens)).int()
        out = ops.gla(dev(proj, dt), dev(low3, torch.float32), dev(t["a2"], torch.float32), dev(t["a2.b"], torch.float32), tau,
                      D ** -0.5, dev(t["norm"], torch.float32), eps, H, D, V, state, dev(starts), dev(tok_seq), dev(slots), B,
                      max_seq_len=max(lens))
        for b in range(B):
            # the oracle gets what the kernel gets: products rounded to the activations' dtype
            rnd = plain.to_bf16 if dtype == "bfloat16" else plain.same
            y, want_state[b] = plain.gla(xs[b], m, t, "", eps, want_state[b], rnd=rnd)
            near(out[starts[b]:starts[b + 1]], y, dtype, f"gla outputs, part {part}, sequence {b}", rel16=1.5e-2)
            near(state[slots[b]].view(H, D, V), want_state[b], dtype, "gla state", rel32=3e-5, rel16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, C, R, dims", [(2, 40, 8, 8), (3, 24, 16, 8), (4, 112, 16, 16), (1, 200, 64, 64), (20, 128, 32, 32),
                                           (8, 448, 64, 64), (5, 80, 0, 0)])
def test_latent_rows_and_decoding_over_them(H, C, R, dims, dtype):
    """Rows written at positions across three pages (in pages that are out of order), then one query per sequence."""
    from trapetum_b200.csrc import ops
    from trapetum_b200.csrc.ops import PAGE_ROWS
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(C + R)
    lens = [2 * PAGE_ROWS + 1, PAGE_ROWS, 5]                        # one key into the third page; a full page; the first tokens
    T, B = sum(lens), len(lens)
    part = torch.randn(2, T, C + R, generator=g)
    w = 1 + 0.2 * torch.randn(C, generator=g)
    inv_freq = torch.tensor([100.0 ** (-2.0 * i / dims) for i in range(dims // 2)])
    positions = torch.cat([torch.arange(n) for n in lens]).int()
    tok_seq = torch.repeat_interleave(torch.arange(B), torch.tensor(lens)).int()
    table = torch.tensor([[5, 0, 3], [2, 6, 6], [4, 6, 6]], dtype=torch.int32)
    pool = torch.zeros(7, 1, PAGE_ROWS, C + R, dtype=dt, device=DEV)
    rows = ops.latent_rows(dev(part), dev(w), 1e-5, dev(inv_freq), dims, C, R, dev(positions), dev(tok_seq), pool, dev(table), dt)
    d = part.double().sum(0)
    want = torch.cat([plain.rms_norm(d[:, :C], w.double(), 1e-5),
                      plain.rotate_half(d[:, C:], positions, dims, 100.0)], dim=1)
    near(rows, want, dtype, "latent rows", rel16=8e-3)
    for b in range(B):
        for pos in (0, lens[b] - 1):
            r = pool[table[b, pos // PAGE_ROWS], 0, pos % PAGE_ROWS]
            assert torch.equal(r, rows[sum(lens[:b]) + pos]), "the cache holds the packed row"
    # decoding: every head's mapped query against all rows of its sequence, with and without a sink
    q = torch.randn(B, H * (C + R), generator=g)
    kv = rows.double().cpu()
    for sink in (None, torch.tensor([0.5 * h - 1 for h in range(H)]), torch.full((H,), 30.0)):
        out = ops.latent_decode(dev(q, dt), pool, dev(table), dev(torch.tensor(lens, dtype=torch.int32)),
                                dev(sink) if sink is not None else None, H, C, R, 0.3, 1024)
        qq = q.to(dt).double()
        for b in range(B):
            k = kv[sum(lens[:b]):sum(lens[:b + 1])]
            s = torch.einsum("hd,nd->hn", qq[b].view(H, C + R), k) * 0.3
            if sink is not None:
                s = torch.cat([s, sink.double()[:, None]], dim=1)
            p = torch.softmax(s, dim=-1)[:, :k.shape[0]]
            near(out[b].view(H, C), p @ k[:, :C], dtype, f"latent decode, sequence {b}", rel32=5e-5, rel16=1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_per_head_products_and_attention_with_a_sink(dtype):
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(3)
    T, H, i, o = 11, 3, 40, 24
    x, w = torch.randn(T, H * i + 8, generator=g).to(dt), torch.randn(H, o, i, generator=g).to(dt)
    y = ops.head_linear(dev(x)[:, 8:], dev(w), H)
    near(y.view(T, H, o), torch.einsum("thi,hoi->tho", x[:, 8:].double().reshape(T, H, i), w.double()), dtype, "per-head product")
    for hd in (24, 48, 64, 128):                                # the generic kernel; in bfloat16 the mma.sync and the tcgen05 kernels
        lens = [70, 3, 129]
        T = sum(lens)
        q, k, v = (torch.randn(T, H * hd, generator=g).to(dt) for _ in range(3))
        sink = torch.tensor([-2.0, 0.7, 9.0])
        starts = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        tok_seq = torch.repeat_interleave(torch.arange(3), torch.tensor(lens)).int()
        out = ops.attn_prefill_sink(dev(q), dev(k), dev(v), dev(starts), dev(tok_seq), H, hd, 0.4, dev(sink), max(lens), lens)
        for b in range(3):
            a, e = int(starts[b]), int(starts[b + 1])
            qq, kk, vv = (z[a:e].double().view(e - a, H, hd) for z in (q, k, v))
            s = torch.einsum("thd,nhd->htn", qq, kk) * 0.4
            s = s.masked_fill(torch.triu(torch.ones(e - a, e - a, dtype=torch.bool), 1)[None], float("-inf"))
            s = torch.cat([s, sink.double()[:, None, None].expand(H, e - a, 1)], dim=-1)
            p = torch.softmax(s, dim=-1)[..., :e - a]
            near(out[a:e].view(e - a, H, hd), torch.einsum("htn,nhd->thd", p, vv), dtype, f"attention with a sink, head size {hd}",
                 rel32=5e-5)


@pytest.mark.parametrize("E, top, groups, keep", [(6, 2, 3, 2), (8, 3, 1, 1), (10, 4, 5, 3), (12, 1, 12, 5), (64, 6, 8, 3), (5, 5, 1, 1)])
def test_router_choices_and_weights(E, top, groups, keep):
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(E * top)
    T, W = 57, 40
    x = torch.randn(T, W, generator=g)
    t = {"router": torch.randn(E, W, generator=g) / 3, "correction": torch.randn(E, generator=g) - 1.5}   # choice scores below zero too
    sg = torch.randn(W, generator=g) / 3
    z = torch.cat([x.double() @ t["router"].double().T, (x.double() @ sg.double())[:, None], torch.zeros(T, 3, dtype=F)], dim=1)
    parts = torch.stack([0.3 * z, 0.7 * z]).float()               # two partial sums, columns past the gate's unused
    idx, wt, gate = ops.moe_route(dev(parts), E, dev(t["correction"]), True, top, groups, keep, 2, 1e-20)
    r = {"experts": E, "top": top}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    wi, ww = plain.route(x.double(), r, {k: v.double() for k, v in t.items()}, "")
    got = [sorted(zip(a, b)) for a, b in zip(idx.cpu().tolist(), wt.cpu().tolist())]
    for tkn in range(T):
        want = sorted(zip(wi[tkn].tolist(), ww[tkn].tolist()))
        assert [a for a, _ in got[tkn]] == [a for a, _ in want], f"token {tkn}: experts {got[tkn]} != {want}"
        assert max(abs(a[1] - b[1]) for a, b in zip(got[tkn], want)) < 1e-5
    near(gate, torch.sigmoid(x.double() @ sg.double()), "float32", "the shared expert's gate")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, W, E, ff, top", [(21, 72, 5, 24, 2), (150, 72, 5, 24, 2), (333, 128, 16, 200, 3), (70, 40, 3, 8, 3),
                                              (400, 128, 6, 48, 3), (700, 256, 5, 256, 2)])
def test_experts_weighted_sum_with_a_shared_expert(T, W, E, ff, top, dtype):
    """Few pairs run one by one, many (in bfloat16) grouped by expert on the tensor cores: tiles that are not full,
    experts that nobody chose, widths that are no multiples of the tile."""
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(8)
    x = torch.randn(T, W, generator=g).to(dt)
    gw, uw, dw = (torch.randn(E, a, b, generator=g).to(dt) / 5 for a, b in ((ff, W), (ff, W), (W, ff)))
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    wt = torch.rand(T, top, generator=g)
    shared, gate = torch.randn(2, T, W, generator=g), torch.rand(T, generator=g)
    gu = None
    if dtype == "bfloat16" and ff % 16 == 0:         # many pairs then run on the tcgen05 product, experts padded to whole tiles
        gu = torch.stack([ops.interleave_gate_up(dev(gw[e]), dev(uw[e])) for e in range(E)]).contiguous()
    out = ops.moe_experts(dev(x), dev(gw), dev(uw), dev(dw), dev(idx), dev(wt), dev(shared), dev(gate), gu)
    rnd = plain.to_bf16 if dtype == "bfloat16" else plain.same
    want = gate.double()[:, None] * shared.double().sum(0)
    for tk in range(T):
        for j in range(top):
            e = int(idx[tk, j])
            want[tk] += wt[tk, j].double() * plain.gated(x[tk:tk + 1].double(), gw[e].double(), uw[e].double(), dw[e].double(),
                                                         plain.silu, rnd)[0]
    near(out, want, dtype, "experts", rel16=1e-2)


# =================================================================================================================
# The model through the engine
# =================================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    model = model_of(folders, name, dtype)
    eng = tb.Engine(model, max_tokens=1024)
    for ids in prompts(cfg["vocab"], [1, 2, 64, 65, 150], seed=1):
        s = eng.start(1)
        got = eng.step(s, [ids], [list(range(len(ids)))])
        eng.release(s)
        close(got, plain.forward(cfg, w, ids), tolerance(name, cfg, w, ids, dtype), f"{name}: whole prompt of {len(ids)}", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_stream_after_every_layer_run(folders, oracles, name, monkeypatch):
    from trapetum_b200.parts.block import PreNormBlock
    cfg, w = oracles[name]
    ids = prompts(cfg["vocab"], [37], seed=2)[0]
    want = plain.Plain(cfg, w).feed(ids)[1]
    seen, orig = [], PreNormBlock.forward

    def spy(self, stream, ctx, cache):
        orig(self, stream, ctx, cache)
        seen.append(stream.value().clone())
    monkeypatch.setattr(PreNormBlock, "forward", spy)
    eng = tb.Engine(model_of(folders, name, "float32"), max_tokens=256)
    eng.step(eng.start(1), [ids], [[0]])
    assert len(seen) == want.shape[0] == len(plain.schedule(cfg))
    for r, x in enumerate(seen):
        near(x, want[r], "float32", f"{name}: the stream after layer run {r}", rel32=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, first", [("A", 1), ("A", 2), ("B", 63), ("B", 64), ("C", 65), ("C", 7), ("D", 3)])
def test_prompt_then_token_by_token(folders, oracles, name, first, dtype):
    """Decoding runs across a page's border (64, 128) and through the capture of the step's graph."""
    cfg, w = oracles[name]
    ids = prompts(cfg["vocab"], [140], seed=first)[0]
    truth = plain.forward(cfg, w, ids)
    assert float(position_errors(plain.forward_stepwise(cfg, w, ids[:70], first), truth[:70]).max()) < 1e-9
    eng = tb.Engine(model_of(folders, name, dtype), max_tokens=512)
    s = eng.start(1)
    got = [eng.step(s, [ids[:first]], [list(range(first))])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[first:]]
    eng.release(s)
    assert dtype == "float32" or eng.graphs_captured >= 1
    close(torch.cat(got), truth, tolerance(name, cfg, w, ids, dtype), f"{name}: {first} tokens, then one by one", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_batch_equals_each_alone_and_slots_are_reused(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    eng = tb.Engine(model_of(folders, name, dtype), max_tokens=1024, max_slots=4)
    rounds = [prompts(cfg["vocab"], [1, 90, 33], seed=4), prompts(cfg["vocab"], [70, 2, 129], seed=5)]
    for ps in rounds:                                            # the second round takes the first one's slots and pages
        n_new = 6
        full = [p + q for p, q in zip(ps, prompts(cfg["vocab"], [n_new] * 3, seed=6))]
        truth = [plain.forward(cfg, w, f) for f in full]
        s = eng.start(3)
        got = [[] for _ in ps]
        out = eng.step(s, ps, [[len(p) - 1] for p in ps])
        for i in range(3):
            got[i].append(out[i:i + 1].clone())
        live = [0, 1, 2]
        for j in range(n_new):
            if j == 3:
                eng.release([s[1]])                              # the middle one ends early; the others go on
                live = [0, 2]
            out = eng.step([s[i] for i in live], [[full[i][len(ps[i]) + j]] for i in live], [[0]] * len(live))
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1].clone())
        eng.release([s[i] for i in live])
        eng.cache.check()
        for i in range(3):
            g = torch.cat(got[i])
            lo = len(ps[i]) - 1
            close(g, truth[i][lo:lo + g.shape[0]], tolerance(name + "u", cfg, w, full[i], dtype)[lo:lo + g.shape[0]],
                  f"{name}: request {i} of an unequal batch", dtype)
    eng.check_kernels()


def _needle(tmp_path, key_pos, n, dtype, sink=None):
    """A one-layer model and a prompt of one repeated token with a single other token at ``key_pos``, chosen (with the
    plain implementation) as the one that the last query's sharpened scores single out most: its loss must show."""
    cfg = config(50, 32, [("latent_attention", latent(2, 8, 8, 16, 16, 1.0, base=10000.0), None)], emb_scale=1.0, eps=1e-5)
    w = {k: v.float() for k, v in random_weights(cfg, 5, [0]).items()}
    w["l0.mix.q"][:] *= 3.0
    w["l0.mix.uk"][:] *= 3.0
    if sink is not None:
        w["l0.mix.sink"][:] = sink
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    wd = {k: v.double() for k, v in w.items()}
    base = [3] * n
    without = plain.forward(cfg, wd, base)[-1:]
    best, ids = -1.0, None
    for cand in range(4, 24):
        trial = list(base)
        trial[key_pos] = cand
        e = float(position_errors(plain.forward(cfg, wd, trial)[-1:], without))
        if e > best:
            best, ids = e, trial
    assert best > 0.2, best
    folder = write_folder(str(tmp_path / f"needle{key_pos}_{n}"), cfg, w)
    return cfg, wd, ids, folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key_pos, n", [(0, 200), (63, 130), (64, 130), (127, 129), (5, 700)])
def test_a_far_key_is_found_in_prompts_and_in_decoding(tmp_path, key_pos, n, dtype):
    cfg, w, ids, folder = _needle(tmp_path, key_pos, n, dtype)
    truth = plain.forward(cfg, w, ids)
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=1024)
    tol = 3e-5 if dtype == "float32" else 3e-2
    s = eng.start(1)
    close(eng.step(s, [ids], [[n - 1]]), truth[-1:], tol, f"needle at {key_pos} of {n}, prompt", dtype)
    eng.release(s)
    s = eng.start(1)
    eng.step(s, [ids[:n - 3]], [[]])
    got = torch.cat([eng.step(s, [[t]], [[0]]).clone() for t in ids[n - 3:]])
    close(got, truth[-3:], tol, f"needle at {key_pos} of {n}, decoded", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sink_takes_its_share(tmp_path, dtype):
    """A sink as large as the best score halves the attention's output; one left out would show in every logit."""
    cfg, w, ids, folder = _needle(tmp_path, 4, 40, dtype, sink=6.0)
    truth = plain.forward(cfg, w, ids)
    w0 = dict(w)
    w0["l0.mix.sink"] = torch.full((2,), -1e4, dtype=torch.float64)
    assert float(position_errors(plain.forward(cfg, w0, ids), truth).max()) > 0.05
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=256)
    s = eng.start(1)
    tol = 3e-5 if dtype == "float32" else 3e-2
    got = [eng.step(s, [ids[:30]], [list(range(30))])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[30:]]
    close(torch.cat(got), truth, tol, "a large sink, prompt then decoding", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_slow_state_is_carried_through_long_decoding(tmp_path, dtype):
    """A gla layer whose decay is nearly one: what the first tokens wrote is still felt 300 tokens later."""
    cfg = config(40, 32, [("gla", gla(2, 8, 16, 64.0), dense(48))], emb_scale=2.0, eps=1e-5)
    w = {k: v.float() for k, v in random_weights(cfg, 6, [4]).items()}
    w["l0.mix.a2.b"][:] = 6.0
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    folder = write_folder(str(tmp_path / "slow"), cfg, w)
    wd = {k: v.double() for k, v in w.items()}
    ids = prompts(40, [300], seed=8)[0]
    truth = plain.forward(cfg, wd, ids)
    other = [(t + 1) % 40 for t in ids[:5]] + ids[5:]
    # five of three hundred tokens: a small share of the state, but two hundred times the 32-bit tolerance
    assert float(position_errors(plain.forward(cfg, wd, other)[-1:], truth[-1:])) > 0.005
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), max_tokens=512)
    s = eng.start(1)
    got = [eng.step(s, [ids[:10]], [[9]])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[10:]]
    close(torch.cat(got), truth[9:], tolerance("slow", cfg, wd, ids, dtype)[9:], "slow state, prompt then long decoding", dtype)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_library(folders, oracles, name):
    cfg, w = oracles[name]
    ps = prompts(cfg["vocab"], [5, 1, 70, 12], seed=9)
    want = [plain.generate_greedy(cfg, w, p, 10) for p in ps]
    model = model_of(folders, name, "float32")
    assert tb.generate(model, ps, max_tokens=10, stop_ids=[]) == want
    assert tb.generate(model, ps, max_tokens=10, stop_ids=[], max_batch=2) == want      # two batches, slots used again
    got16 = tb.generate(model_of(folders, name, "bfloat16"), ps, max_tokens=10, stop_ids=[])
    assert all(len(o) == 10 for o in got16)


def test_command_line_runs_the_model(folders, oracles):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gemma_run"), folders["B"], "--prompt_ids", "5,17,3",
                           "--max_tokens", "5", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    cfg, w = oracles["B"]
    assert f"continuation ids: {plain.generate_greedy(cfg, w, [5, 17, 3], 5)}" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(folders, oracles, tmp_path, dtype):
    name = "A"
    cfg, w = oracles[name]
    V = cfg["vocab"]
    reqs = prompts(V, [40, 75, 130], seed=3)
    truth = [plain.forward(cfg, w, r) for r in reqs]
    steps, expect = [], {}

    def add(entries, end=()):
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})
        return len(steps) - 1
    n = add([{"id": "w", "tokens": reqs[0], "want": list(range(40))}], end=["w"])
    expect[n] = truth[0]
    cut = [1, 60, 33]                                                # together; one starts with a single token
    ids = [f"b{i}" for i in range(3)]
    n = add([{"id": ids[i], "tokens": reqs[i][:cut[i]], "want": [cut[i] - 1]} for i in range(3)])
    expect[n] = torch.cat([truth[i][cut[i] - 1:cut[i]] for i in range(3)])
    live, t = [0, 1, 2], 0
    while live:
        nxt = [i for i in live if cut[i] + t + 1 < len(reqs[i])]
        quiet = t % 5 == 3
        n = add([{"id": ids[i], "tokens": [reqs[i][cut[i] + t]], "want": [] if quiet else [0]} for i in live],
                end=[ids[i] for i in live if i not in nxt])
        if not quiet:
            expect[n] = torch.stack([truth[i][cut[i] + t] for i in live])
        live, t = nxt, t + 1
    out = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", dtype,
                           "--out", out, "--max-tokens", str(40 + 75 + 130)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    assert sorted(os.listdir(out)) == sorted(f"{n}.f32" for n in expect)
    tol = max(float(tolerance(name, cfg, w, r, dtype).max()) for r in reqs)
    for n, want in expect.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
        assert got.shape == want.shape
        close(got, want, tol, f"replay step {n}", dtype)
