"""Divanex without a GPU: the configuration reader, the spec, the tensor list, and the oracle against itself."""
import copy
import math

import pytest
import torch

import plain_divanex as plain
import trapetum_b200 as tb
from divanex_util import CFG_A, CFG_B, CFG_C, CONFIGS, prompts, random_weights
from trapetum_b200.config import ConfigError, load_config
from trapetum_b200.engine.model import tensor_specs_for_config


def test_every_size_and_constant_is_read_by_key():
    cfg, spec = load_config(copy.deepcopy(CFG_A))
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.postln_alpha, cfg.logit_scale, cfg.side_dim) == (200, 64, 3.0, 1.5, 0.5, 8)
    assert [L.type for L in cfg.layers] == ["mamba2", "attention", "attention"]
    assert cfg.layers[0].mlp.limit == 2.5 and cfg.layers[1].mlp is None
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.scale, a.softcap, a.q_temp_coef, a.q_temp_every) == (4, 2, 16, 0.9, 20.0, 0.3, 4)
    assert cfg.layers[2].mixer.softcap is None and cfg.layers[2].mixer.q_temp_every == 0
    m = cfg.layers[0].mixer
    assert (m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups) == (2, 16, 8, 2, 3, 2)
    assert [l.mixer.kind for l in spec.layers] == ["mamba2", "attention", "attention"]
    assert [l.feed_forward.kind for l in spec.layers] == ["gated_mlp", "none", "gated_mlp"]
    assert all(l.block.kind == "post_norm" and l.block.params["alpha"] == 1.5 for l in spec.layers)
    assert spec.layers[1].block.params["side"].params["first_col"] == 8
    assert spec.head.params["scale"] == 0.5 and spec.embedding.params["scale"] == 3.0
    _, spec_b = load_config(copy.deepcopy(CFG_B))
    assert all(l.block.params["side"] is None for l in spec_b.layers)


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "rwkv", "type"),
    (("layers", 1, "mixer", "heads"), None, "layers[1].mixer.heads"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "vdim"), 8, "vdim"),
    (("layers", 0, "mixer", "groups"), 3, "groups"),
    (("layers", 0, "mixer", "norm_groups"), 5, "norm_groups"),
    (("layers", 0, "mlp", "kind"), "experts", "mlp.kind"),
    (("layers", 0, "mlp", "limit"), None, "mlp.limit"),
    (("norm",), None, "norm"),
    (("vocab",), "many", "vocab"),
])
def test_errors_name_the_key(path, value, word):
    c = copy.deepcopy(CFG_A)
    d = c
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(c)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_list_is_what_the_oracle_reads(name):
    cfg = CONFIGS[name]
    specs = tensor_specs_for_config(copy.deepcopy(cfg))
    w = random_weights(cfg, 0)
    assert {k: tuple(v.shape) for k, v in specs.items()} == {k: tuple(v.shape) for k, v in w.items()}


def test_the_python_host_is_chosen_without_asking_the_native_library():
    assert tb._host(None, copy.deepcopy(CFG_A)) == "python"
    assert tb._host("auto", copy.deepcopy(CFG_B)) == "python"


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    d = tb.write_random_model(str(tmp_path / "m"), copy.deepcopy(CFG_B), seed=3, device="cpu")
    cfg, w = plain.load_folder(d)
    assert abs(float(w["l1.norm1"].mean()) - 1.0) < 0.1          # gains are drawn around 1
    logits = plain.forward(cfg, w, [1, 2, 3, 4])
    assert logits.shape == (4, 301) and torch.isfinite(logits).all()


# ---- the oracle against itself -------------------------------------------------------------------------------
def test_query_temperature_steps_at_multiples_of_every():
    f = plain.query_temperature(torch.arange(0, 13), 0.5, 4)
    want = [1.0] * 3 + [1 + 0.5 * math.log(2)] * 4 + [1 + 0.5 * math.log(3)] * 4 + [1 + 0.5 * math.log(4)] * 2
    assert torch.allclose(f, torch.tensor(want, dtype=f.dtype))


def test_conv_and_scan_carry_their_state():
    g = torch.Generator().manual_seed(1)
    u = torch.randn(9, 5, generator=g, dtype=torch.float64)
    wt, b = torch.randn(5, 3, generator=g, dtype=torch.float64), torch.randn(5, generator=g, dtype=torch.float64)
    whole = plain.causal_conv(u, wt, b, torch.zeros(2, 5, dtype=torch.float64))
    tail = plain.causal_conv(u[4:], wt, b, u[2:4])
    assert torch.allclose(whole[4:], tail)
    assert torch.allclose(whole[0], u[0] * wt[:, 2] + b)          # the last column is the current token's
    xs, Bm, Cm = (torch.randn(7, 2, 3, generator=g, dtype=torch.float64), torch.randn(7, 1, 4, generator=g, dtype=torch.float64),
                  torch.randn(7, 1, 4, generator=g, dtype=torch.float64))
    dt = torch.rand(7, 2, generator=g, dtype=torch.float64)
    A, D = torch.randn(2, generator=g, dtype=torch.float64), torch.randn(2, generator=g, dtype=torch.float64)
    S = torch.zeros(2, 4, 3, dtype=torch.float64)
    y = plain.ssm_scan(xs, Bm, Cm, dt, A, D, S, 1)
    S2 = torch.zeros(2, 4, 3, dtype=torch.float64)
    y2 = torch.cat([plain.ssm_scan(xs[:3], Bm[:3], Cm[:3], dt[:3], A, D, S2, 1),
                    plain.ssm_scan(xs[3:], Bm[3:], Cm[3:], dt[3:], A, D, S2, 1)])
    assert torch.allclose(y, y2) and torch.allclose(S, S2)
    # one step by hand: S = dt * B x^T, y = S^T C + D x
    S3 = torch.zeros(2, 4, 3, dtype=torch.float64)
    y3 = plain.ssm_scan(xs[:1], Bm[:1], Cm[:1], dt[:1], A, D, S3, 1)
    assert torch.allclose(y3[0, 1], dt[0, 1] * (Bm[0, 0] @ Cm[0, 0]) * xs[0, 1] + D[1] * xs[0, 1])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_oracle_whole_prompt_equals_token_by_token(name):
    cfg = CONFIGS[name]
    w = {k: v.double() for k, v in random_weights(cfg, 2).items()}
    (ids,) = prompts(cfg["vocab"], [21], seed=4)
    whole = plain.forward(cfg, w, ids)
    for first in (1, 2, 13):
        assert torch.allclose(whole, plain.forward_stepwise(cfg, w, ids, first), atol=1e-9, rtol=1e-9)


def test_dense_ff_clamps_both_branches():
    w = {"gate": torch.eye(3, dtype=torch.float64), "up": torch.eye(3, dtype=torch.float64), "down": torch.eye(3, dtype=torch.float64)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64)
    y = plain.dense_ff(h, w, "", 2.0)
    s = lambda g: g / (1 + math.exp(-1.702 * g))
    assert torch.allclose(y, torch.tensor([[s(2.0) * 3.0, s(-5.0) * (-2.0 + 1.0), s(0.5) * 1.5]], dtype=torch.float64))
