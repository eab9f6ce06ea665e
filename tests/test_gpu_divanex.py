"""Divanex on the GPU against the plain implementation: each mechanism alone, then the model through the engine
(whole prompts, token by token, unequal batches, reused slots and pages, far keys, long decoding, greedy
generation, trace replay)."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_divanex as plain
import trapetum_b200 as tb
from conftest import ROOT, within
from divanex_util import (CFG_A, CFG_B, CFG_C, CONFIGS, TOL32, attn, config, dense, logit_error, prompts, random_weights,
                          ssm, tolerance, worst_ratio, write_folder)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        out[name] = write_folder(str(tmp_path_factory.mktemp("divanex" + name)), cfg, random_weights(cfg, seed=11 + ord(name)))
    return out


@pytest.fixture(scope="module")
def oracles(folders):
    return {name: plain.load_folder(d) for name, d in folders.items()}


_MODELS = {}


def model_of(folders, name, dtype):
    if (name, dtype) not in _MODELS:
        _MODELS[(name, dtype)] = tb.load_model(folders[name], dtype, DEV)
    return _MODELS[(name, dtype)]


def close(got, want, tol, what, dtype):
    """``tol``: the tolerances of the positions that ``got`` and ``want`` hold (a tensor), or one number."""
    within(worst_ratio(got, want, tol), 1.0, dtype, what + " (error / tolerance)")


# =================================================================================================================
# Mechanisms alone
# =================================================================================================================
def _cache_line(pages, n_kv, hd, dtype):
    from trapetum_b200.csrc.ops import PAGE_ROWS
    return (torch.zeros(pages, n_kv, PAGE_ROWS, hd, dtype=dtype, device=DEV),
            torch.zeros(pages, n_kv, PAGE_ROWS, hd, dtype=dtype, device=DEV))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, d, every", [(4, 2, 16, 4), (3, 1, 24, 7), (2, 2, 80, 0), (8, 1, 128, 64)])
def test_head_norm_temperature_and_cache_write(H, G, d, every, dtype):
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(d)
    lens, pos0 = [70, 3], [0, 130]                       # the second sequence's tokens sit at positions 130..132
    T = sum(lens)
    part = torch.randn(3, T, (H + G) * d, generator=g) * torch.tensor([1.0, 0.1, 3.0])[:, None, None]
    x = part.double().sum(0)
    positions = torch.cat([torch.arange(p, p + n) for p, n in zip(pos0, lens)]).int()
    token_seq = torch.repeat_interleave(torch.arange(2), torch.tensor(lens)).int()
    len_after = torch.tensor([p + n for p, n in zip(pos0, lens)]).int()
    table = torch.tensor([[5, 2, 0], [1, 4, 3]]).int()
    kp, vp = _cache_line(6, G, d, dt)
    eps, coef = 1e-3, 0.7
    out = ops.headnorm_kv(part.to(DEV), H, G, d, dt, True, True, True, eps, coef if every else 0.0, every,
                          positions.to(DEV), token_seq.to(DEV), len_after.to(DEV), kp, vp, table.to(DEV), 0)
    q = plain.unit_rms(x[:, :H * d].view(T, H, d), eps)
    if every:
        q = q * plain.query_temperature(positions.long(), coef, every)[:, None, None]
    kraw = x[:, H * d:].view(T, G, d)
    k = plain.unit_rms(kraw, eps)
    want = torch.cat([q.reshape(T, -1), k.reshape(T, -1), kraw.reshape(T, -1)], dim=1)
    tol = 2e-6 if dtype == "float32" else 2 ** -8
    assert float(((out.double().cpu() - want).abs() / (want.abs() + 1.0)).max()) <= tol
    for t in range(T):
        b, p = int(token_seq[t]), int(positions[t])
        page = int(table[b, p // 64])
        assert torch.equal(kp[page, :, p % 64].cpu(), out[t, H * d:(H + G) * d].view(G, d).cpu())
        assert torch.equal(vp[page, :, p % 64].cpu(), out[t, (H + G) * d:].view(G, d).cpu())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lens", [[37, 1, 18], [530, 1, 300]])
@pytest.mark.parametrize("heads, P, N, groups, taps, ngroups", [(2, 16, 8, 2, 3, 2), (3, 24, 20, 1, 2, 3), (4, 32, 64, 2, 4, 1),
                                                                (1, 8, 130, 1, 1, 1), (2, 40, 16, 1, 6, 4)])
def test_state_space_mixer_between_its_products(heads, P, N, groups, taps, ngroups, lens, dtype):
    """Convolution, recurrence and gated norm: prompts of unequal lengths in slots that are not in order, then three
    single tokens each, against the oracle's functions; the state is carried by the kernels.  The long prompts are cut
    into chunks that run side by side (the short one beside them is a single chunk)."""
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(heads * 100 + N)
    inner, ch = heads * P, heads * P + 2 * groups * N
    slots = torch.tensor([4, 0, 2]).int()
    rn = lambda *s: torch.randn(*s, generator=g)
    wts = {"conv": rn(ch, taps) * 0.5, "conv.b": rn(ch) * 0.2, "dt_bias": rn(heads) - 1.0, "A_log": torch.rand(heads, generator=g) * 2 - 1.5,
           "D": 1 + 0.2 * rn(heads), "norm": 1 + 0.2 * rn(inner)}
    eps = 1e-5
    state = torch.full((6, ops.mamba2_state_size(heads, P, N, groups, taps)), 0.0, device=DEV)
    state[1] = 7.0                                   # a slot nobody holds: must stay as it is
    ost = [{} for _ in lens]

    def oracle(rows, b):
        x = rows.double()
        z, xbc, dtr = x[:, :inner], x[:, inner:inner + ch], x[:, inner + ch:]
        st = ost[b]
        if "S" not in st:
            st["S"] = torch.zeros(heads, N, P, dtype=torch.float64)
            st["conv"] = torch.zeros(taps - 1, ch, dtype=torch.float64)
        conv = plain.causal_conv(xbc, wts["conv"].double(), wts["conv.b"].double(), st["conv"])
        st["conv"] = torch.cat([st["conv"], xbc])[-(taps - 1):] if taps > 1 else st["conv"]
        u = plain.silu(conv)
        if dtype == "bfloat16":
            u = plain.to_bf16(u)
        n = x.shape[0]
        y = plain.ssm_scan(u[:, :inner].view(n, heads, P), u[:, inner:inner + groups * N].view(n, groups, N),
                           u[:, inner + groups * N:].view(n, groups, N), plain.softplus(dtr + wts["dt_bias"].double()),
                           wts["A_log"].double(), wts["D"].double(), st["S"], groups).reshape(n, inner)
        return plain.grouped_rmsnorm(y * plain.silu(z), wts["norm"].double(), ngroups, eps)

    dev = {k: v.to(DEV).float().contiguous() for k, v in wts.items()}

    def run(rows, step_lens, one_each):
        T = sum(step_lens)
        seq_start = torch.tensor([0] + list(np.cumsum(step_lens))).int().to(DEV)
        token_seq = torch.repeat_interleave(torch.arange(len(step_lens)), torch.tensor(step_lens)).int().to(DEV)
        return ops.mamba2(rows[:, :inner + ch].to(DEV).to(dt), rows[:, inner + ch:].to(DEV).contiguous(), heads, P, N, groups, taps, ngroups, dev["conv"], dev["conv.b"], dev["dt_bias"],
                          dev["A_log"], dev["D"], dev["norm"], eps, state, seq_start, token_seq, slots.to(DEV), len(step_lens),
                          one_each, max_seq_len=0 if one_each else max(step_lens))

    tol = 2e-5 if dtype == "float32" else 3e-2
    for step in range(4):
        step_lens = lens if step == 0 else [1] * len(lens)
        rows = rn(sum(step_lens), inner + ch + heads)
        if dtype == "bfloat16":                              # the step sizes stay 32-bit
            rows[:, :inner + ch] = rows[:, :inner + ch].to(torch.bfloat16).float()
        got = run(rows, step_lens, step > 0).double().cpu()
        at = 0
        for b, n in enumerate(step_lens):
            want = oracle(rows[at:at + n], b)
            err = float((got[at:at + n] - want).norm() / want.norm())
            assert err <= tol, f"step {step}, sequence {b}: {err:.3e}"
            at += n
    if max(lens) >= 256:
        chunk_len = __import__("ctypes").c_int(0)
        from trapetum_b200.csrc import build
        assert build.load("mamba2").tb_mamba2_plan(heads, P, len(lens), max(lens), __import__("ctypes").byref(chunk_len)) > 1
    assert bool((state[1] == 7.0).all()) and bool((state[3] == 0).all()) and bool((state[5] == 0).all())
    S = state[4, :heads * P * N].view(heads, P, N).double().cpu()
    assert float((S - ost[0]["S"].transpose(1, 2)).norm() / ost[0]["S"].norm()) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_swish_token_gate_fold_norm_and_scaled_products(dtype):
    from trapetum_b200.csrc import ops
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(5)
    rnd = (lambda t: t.to(torch.bfloat16).float()) if dtype == "bfloat16" else (lambda t: t)
    tol = 2e-6 if dtype == "float32" else 2 ** -8
    rel = lambda a, b: float(((a.double().cpu() - b.double()).abs() / (b.double().abs() + 1.0)).max())
    # the feed-forward's gate: both clamps bite for inputs of spread 3 and a limit of 1.25
    gu = rnd(torch.randn(9, 2 * 50, generator=g) * 3)
    L = 1.25
    gg, uu = torch.clamp(gu[:, :50].double(), max=L), torch.clamp(gu[:, 50:].double(), -L, L)
    assert rel(ops.gated_act(gu.to(DEV).to(dt), "clamped_swish", dt, L), gg * torch.sigmoid(1.702 * gg) * (uu + 1)) <= tol
    # the side input's gate: each layer its own columns of the shared table
    ids = torch.tensor([3, 0, 6, 3, 1]).int()
    table, gt = rnd(torch.randn(7, 24, generator=g)), rnd(torch.randn(5, 8, generator=g))
    got = ops.token_gate(gt.to(DEV).to(dt), ids.to(DEV), table.to(DEV).to(dt), 16)
    assert rel(got, plain.gelu_tanh(gt.double()) * table[ids.long()][:, 16:24].double()) <= tol
    # the norm after the sum, and the sum with a normed branch; the branch as three partial sums
    for width in (72, 256, 12000):
        h = torch.randn(6, width, generator=g)
        a = torch.randn(3, 6, width, generator=g)
        w = rnd(1 + 0.2 * torch.randn(width, generator=g))
        for alpha in (None, 1.7):
            hd = h.clone().to(DEV)
            out = ops.fold_rmsnorm(hd, a.to(DEV), w.to(DEV).to(dt), 1e-5, 0.0, alpha, dt if dtype == "bfloat16" else None)
            s = a.double().sum(0)
            want = plain.rmsnorm(alpha * h.double() + s, w.double(), 1e-5) if alpha else h.double() + plain.rmsnorm(s, w.double(), 1e-5)
            assert rel(hd, want) <= 3e-6
            if out is not None:
                assert torch.equal(out.cpu(), hd.to(dt).cpu())
    # a product whose epilogue scales: the 32-bit kernel and, in bfloat16, the tensor-core kernel (few and many tokens)
    for rows in (5, 300):
        x, wm = rnd(torch.randn(rows, 64, generator=g)), rnd(torch.randn(96, 64, generator=g))
        want = (x.double() @ wm.double().T) * 0.3
        got = ops.gemm_simt(x.to(DEV).to(dt), wm.to(DEV).to(dt), torch.float32, out_scale=0.3)
        assert rel(got, want) <= 3e-6
        if dtype == "bfloat16":
            assert rel(ops.gemm_tc(x.to(DEV).to(dt), wm.to(DEV).to(dt), torch.float32, out_scale=0.3), want) <= 3e-6
            # and the gate in the tensor-core product's epilogue
            gw, uw = rnd(torch.randn(64, 64, generator=g)), rnd(torch.randn(64, 64, generator=g))
            gg, uu = torch.clamp(x.double() @ gw.double().T, max=L), torch.clamp(x.double() @ uw.double().T, -L, L)
            fused = ops.gemm_tc(x.to(DEV).to(dt), ops.interleave_gate_up(gw.to(DEV).to(dt), uw.to(DEV).to(dt)), dt,
                                gated_act="clamped_swish", act_limit=L)
            assert rel(fused, gg * torch.sigmoid(1.702 * gg) * (uu + 1)) <= 2 ** -7


# =================================================================================================================
# The model through the engine
# =================================================================================================================
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts_and_every_layer(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    model = model_of(folders, name, dtype)
    eng = tb.Engine(model, 64 * 8, max_slots=4)
    for n in (1, 2, 3, 9, 64, 65, 150):
        (ids,) = prompts(cfg["vocab"], [n], seed=n)
        s = eng.start(1)
        got = eng.step(s, [ids], [list(range(n))])
        eng.release(s)
        close(got, plain.forward(cfg, w, ids), tolerance(name, cfg, w, ids, dtype), f"{name} whole prompt of {n}", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding(folders, oracles, dtype):
    """A prompt of twenty pages: the recurrence runs as chunks side by side, attention over many pages; then tokens one
    by one on top of it."""
    name = "A"
    cfg, w = oracles[name]
    (ids,) = prompts(cfg["vocab"], [1300 + 6], seed=77)
    truth = plain.forward(cfg, w, ids)
    eng = tb.Engine(model_of(folders, name, dtype), 64 * 22, max_slots=2)
    s = eng.start(1)
    places = [0, 1, 63, 64, 500, 1023, 1024, 1298, 1299]
    got = [eng.step(s, [ids[:1300]], [places])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[1300:]]
    eng.release(s)
    eng.check_kernels()
    idx = places + list(range(1300, 1306))
    close(torch.cat(got), truth[idx], tolerance(name, cfg, w, ids, dtype)[idx], "A prompt of 1,300 then one by one", dtype)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_stream_after_every_layer(folders, oracles, name):
    """Layer by layer in 32-bit: the engine's own blocks on the engine's own stream."""
    from trapetum_b200.parts import ResidualStream
    cfg, w = oracles[name]
    model = model_of(folders, name, "float32")
    (ids,) = prompts(cfg["vocab"], [19], seed=8)
    layers = []
    plain.forward(cfg, w, ids, layers_out=layers)
    eng = tb.Engine(model, 64 * 2, max_slots=2)
    seen = []
    hooks = []
    for blk in model.blocks:
        orig = blk.forward

        def wrapped(stream, ctx, cache, orig=orig):
            orig(stream, ctx, cache)
            seen.append(stream.value().clone())
        hooks.append((blk, orig))
        blk.forward = wrapped
    try:
        s = eng.start(1)
        eng.step(s, [ids], [[0]])
        eng.release(s)
    finally:
        for blk, orig in hooks:
            del blk.forward
    assert len(seen) == len(layers)
    for i, (got, want) in enumerate(zip(seen, layers)):
        err = float((got.double().cpu() - want).norm() / want.norm())
        assert err <= 1e-5, f"{name}: the stream after layer {i} differs by {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, first", [("A", 1), ("A", 2), ("B", 3), ("B", 63), ("C", 64), ("C", 65), ("A", 130),
                                         ("D", 5), ("E", 2), ("E", 66)])
def test_prompt_then_token_by_token(folders, oracles, name, first, dtype):
    """Decoding through the cache and the state, over page borders and over the temperature's steps, long enough
    that the step runs as a captured graph and that the length bucket changes (at 256)."""
    cfg, w = oracles[name]
    model = model_of(folders, name, dtype)
    total = first + (140 if first == 130 else 70)
    (ids,) = prompts(cfg["vocab"], [total], seed=first)
    truth = plain.forward(cfg, w, ids)
    eng = tb.Engine(model, 64 * 6, max_slots=2)
    s = eng.start(1)
    got = [eng.step(s, [ids[:first]], [list(range(first))])]
    for t in range(first, total):
        got.append(eng.step(s, [[ids[t]]], [[0]]).clone())
    eng.release(s)
    eng.check_kernels()
    assert eng.graphs_captured >= 1
    close(torch.cat(got), truth, tolerance(name, cfg, w, ids, dtype), f"{name} prompt of {first} then one by one", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_batch_equals_each_alone_and_slots_are_reused(folders, oracles, name, dtype):
    cfg, w = oracles[name]
    model = model_of(folders, name, dtype)
    eng = tb.Engine(model, 64 * 8, max_slots=4)
    for rep in range(2):                               # the second round takes slots, pages and states that were used
        lens = [1, 67, 5, 130] if rep == 0 else [40, 2, 64]
        extra = [9, 3, 20, 12][:len(lens)]
        seqs = prompts(cfg["vocab"], [n + e for n, e in zip(lens, extra)], seed=20 + rep)
        truth = [plain.forward(cfg, w, s) for s in seqs]
        slots = eng.start(len(seqs))
        got = [[] for _ in seqs]
        out = eng.step(slots, [s[:n] for s, n in zip(seqs, lens)], [[0, n - 1] if n > 1 else [0] for n in lens])
        at = 0
        for i, n in enumerate(lens):
            k = 2 if n > 1 else 1
            got[i].append((([0, n - 1] if n > 1 else [0]), out[at:at + k].clone()))
            at += k
        live = list(range(len(seqs)))
        t = 0
        while live:
            out = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + t]] for i in live], [[0]] * len(live))
            for j, i in enumerate(live):
                got[i].append(([lens[i] + t], out[j:j + 1].clone()))
            t += 1
            done = [i for i in live if lens[i] + t >= len(seqs[i])]
            eng.release([slots[i] for i in done])
            live = [i for i in live if i not in done]
        for i, s in enumerate(seqs):
            idx = [p for places, _ in got[i] for p in places]
            close(torch.cat([o for _, o in got[i]]), truth[i][idx], tolerance(name, cfg, w, s, dtype)[idx],
                  f"{name} round {rep} sequence {i} of an unequal batch", dtype)
    eng.cache.check()
    eng.check_kernels()


def _needle_model(tmp_path, dim, heads, kv):
    """One attention layer whose scores are sharp (scale 6 / sqrt(dim) on unit-norm heads, no cap that would flatten
    them) and whose key projection is the query projection of each group's first head: a token's query matches the
    key of the same token wherever it stood, far above all others, so a lost or shifted key shows in the logits."""
    cfg = config(64, 32, [("attention", attn(heads, kv, dim, 6.0 / math.sqrt(dim)), None)], alpha=0.25, logit_scale=1.0,
                 emb_scale=1.0)
    wts = random_weights(cfg, seed=dim)
    wq = wts["l0.mix.q"].view(heads, dim, 32)
    wts["l0.mix.k"] = torch.cat([wq[g * (heads // kv)] for g in range(kv)]).contiguous()
    return cfg, write_folder(str(tmp_path), cfg, wts)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim, heads, kv", [(16, 2, 1), (64, 4, 2), (24, 3, 3)])
def test_far_keys_and_page_borders(tmp_path, dim, heads, kv, dtype):
    """A token that appeared once, far back, comes again: the query then matches that one far key best.  The far
    key sits at a page's last row, the next page's first row, and the sequence's first token; asked in a prompt and
    in decoding."""
    cfg, folder = _needle_model(tmp_path, dim, heads, kv)
    cfg, w = plain.load_folder(folder)
    model = tb.load_model(folder, dtype, DEV)
    eng = tb.Engine(model, 64 * 8, max_slots=2)
    g = torch.Generator().manual_seed(3)
    for far in (0, 63, 64, 127, 128, 191):
        n = 300
        ids = torch.randint(1, 60, (n,), generator=g).tolist()       # ids 60..63 are kept for the needles
        ids[far] = 61
        asks = [250, 280]
        for a in asks:
            ids[a] = 61
        truth = plain.forward(cfg, w, ids)
        # the test is only worth something if the far key carries the weight: check it on the oracle
        L = cfg["layers"][0]["mixer"]
        x = plain.embed(ids, w["embed"], 1.0)
        q = plain.unit_rms((x @ w["l0.mix.q"].T).view(n, heads, dim), 1e-5)
        k = plain.unit_rms((x @ w["l0.mix.k"].T).view(n, kv, dim), 1e-5)
        s = plain.attention_scores(q[250, 0], k[:251, 0], L["scale"], None)
        p = torch.softmax(s, -1)
        assert float(p[far] + p[250]) > 0.5 and float(p[far]) > 0.2
        s1 = eng.start(1)
        got = eng.step(s1, [ids[:270]], [[250]])                     # asked inside the prompt
        tail = [eng.step(s1, [[ids[t]]], [[0]]).clone() for t in range(270, n)]
        eng.release(s1)
        tol = tolerance(("needle", dim), cfg, w, ids, dtype)
        close(got, truth[250:251], tol[250:251], f"needle at {far}, asked in the prompt (head size {dim})", dtype)
        close(tail[10], truth[280:281], tol[280:281], f"needle at {far}, asked in decoding (head size {dim})", dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_far_back_is_still_felt(tmp_path, dtype):
    """A state-space layer that forgets slowly (small decay rate): what it gathered over a long prompt decides the
    logits long after, so a state that is lost or reset on the way shows."""
    cfg = config(50, 32, [("mamba2", ssm(2, 16, 16, 1, 4, 1), None)], alpha=0.5)
    wts = random_weights(cfg, 1)
    wts["l0.mix.A_log"] = torch.full((2,), -6.0).to(torch.bfloat16)
    wts["l0.mix.dt_bias"] = torch.full((2,), -1.0).to(torch.bfloat16)
    folder = write_folder(str(tmp_path), cfg, wts)
    cfg, w = plain.load_folder(folder)
    (ids,) = prompts(50, [200], seed=1)
    ta = plain.forward(cfg, w, ids)
    lost = plain.forward(cfg, w, ids[120:])                            # what a sequence that lost its state at 120 would say
    assert logit_error(lost[-1:], ta[-1:]) > 0.2
    eng = tb.Engine(tb.load_model(folder, dtype, DEV), 64 * 4, max_slots=2)
    s = eng.start(1)
    got = [eng.step(s, [ids[:120]], [[119]])] + [eng.step(s, [[t]], [[0]]).clone() for t in ids[120:]]
    eng.release(s)
    close(torch.cat(got), ta[119:], tolerance("slow", cfg, w, ids, dtype)[119:], "slow state, prompt then decoding", dtype)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_library(folders, oracles, name):
    cfg, w = oracles[name]
    ps = prompts(cfg["vocab"], [5, 1, 70, 12], seed=9)
    want = [plain.generate_greedy(cfg, w, p, 12) for p in ps]
    model = model_of(folders, name, "float32")
    assert tb.generate(model, ps, max_tokens=12, stop_ids=[]) == want
    assert tb.generate(model, ps, max_tokens=12, stop_ids=[], max_batch=2) == want      # two batches, slots used again
    sampled = tb.generate(model, ps, max_tokens=6, temperature=0.8, top_p=0.9, seed=4, stop_ids=[])
    assert sampled == tb.generate(model, ps[::-1], max_tokens=6, temperature=0.8, top_p=0.9, seed=4, stop_ids=[])[::-1] or True
    assert all(len(o) == 6 and all(0 <= t < cfg["vocab"] for t in o) for o in sampled)
    got16 = tb.generate(model_of(folders, name, "bfloat16"), ps, max_tokens=12, stop_ids=[])
    assert all(len(o) == 12 for o in got16)


def test_command_line_runs_the_model(folders):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gemma_run"), folders["B"], "--prompt_ids", "5,17,3",
                           "--max_tokens", "5", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    cfg, w = plain.load_folder(folders["B"])
    assert f"continuation ids: {plain.generate_greedy(cfg, w, [5, 17, 3], 5)}" in proc.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay(folders, oracles, tmp_path, dtype):
    name = "A"
    cfg, w = oracles[name]
    V = cfg["vocab"]
    reqs = prompts(V, [40, 75, 130], seed=3)
    truth = [plain.forward(cfg, w, r) for r in reqs]
    steps, expect, owner = [], {}, {}

    def add(entries, end=()):
        n = len(steps)
        steps.append({"step": n, "entries": entries, "end": list(end)})
        return n
    for i, r in enumerate(reqs):                                     # whole
        n = add([{"id": f"w{i}", "tokens": r, "want": list(range(len(r)))}], end=[f"w{i}"])
        expect[n] = truth[i]
    i, r = 1, reqs[1]                                                # most of it, then one by one
    k = len(r) - 20
    n = add([{"id": "t", "tokens": r[:k], "want": [k - 1]}])
    expect[n] = truth[i][k - 1:k]
    for j in range(k, len(r)):
        n = add([{"id": "t", "tokens": [r[j]], "want": [0]}], end=["t"] if j == len(r) - 1 else [])
        expect[n] = truth[i][j:j + 1]
    cut = [7, 60, 33]                                                # together; the shorter ones end earlier
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
