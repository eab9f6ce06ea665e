"""Lofirax without a GPU: the configuration reader, the spec and its schedule, the tensor list, and the oracle
against itself."""
import copy

import pytest
import torch

import plain_lofirax as plain
from lofirax_util import CFG_A, CFG_B, CFG_C, CONFIGS, RANKS, prompts, random_weights, write_folder
from trapetum_b200.config import ConfigError, load_config
from trapetum_b200.engine.model import tensor_specs_for_config


def test_every_size_and_constant_is_read_by_key():
    cfg, spec = load_config(copy.deepcopy(CFG_A))
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_eps, cfg.logit_softcap) == (200, 64, 3.0, 1e-5, 10.0)
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 2, 3)
    a = cfg.layers[0].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale, a.rot_dims, a.rot_base) == (2, 16, 8, 40, 40, 0.3, 8, 100.0)
    g = cfg.layers[1].mixer
    assert (g.heads, g.dim, g.vdim, g.tau, g.rank) == (3, 8, 16, 4.0, None)
    m = cfg.layers[0].mlp
    assert (m.experts, m.top, m.ff, m.groups, m.keep, m.shared_ff) == (6, 2, 32, 3, 2, 48)
    assert cfg.layers[1].mlp.ff == 96 and cfg.layers[2].mlp is None
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "gla", "gla"]
    assert [l.feed_forward.kind for l in spec.layers] == ["routed_experts", "gated_mlp", "none"]
    assert all(l.block.kind == "pre_norm" for l in spec.layers) and spec.layers[2].block.params["pre_ffn_norm"] is None
    assert spec.head.params["softcap"] == 10.0 and spec.final_norm.kind == "layernorm"
    b, spec_b = load_config(copy.deepcopy(CFG_B))
    assert b.loop is None and b.logit_softcap is None and b.layers[1].mixer.rot_dims == 8 and b.layers[0].mlp.groups == 1
    assert spec_b.layers[0].feed_forward.params["shared"] is None


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_schedule_names_every_layer_run_and_what_comes_before_it(name):
    cfg = CONFIGS[name]
    _, spec = load_config(copy.deepcopy(cfg))
    runs = plain.schedule(cfg)
    assert [e.layer for e in spec.schedule] == [i for i, _ in runs]
    assert all(e.cache_of is None for e in spec.schedule)                       # every pass has a cache of its own
    for e, (_, rep) in zip(spec.schedule, runs):
        if rep is None:
            assert e.before is None
        else:
            p = e.before.params
            assert e.before.kind == "pass_input" and p["row"] == rep and p["add_embedding"] == (rep > 0)
            assert p["rows"] == cfg["loop"]["times"] and p["table"] == "loop.step"


@pytest.mark.parametrize("path, value, word", [
    (("layers", 1, "type"), "rwkv", "type"),
    (("layers", 0, "mixer", "kv_rank"), None, "layers[0].mixer.kv_rank"),
    (("layers", 0, "mixer", "rot", "base"), None, "rot.base"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "tau"), 0.0, "tau"),
    (("layers", 0, "mlp", "kind"), "sparse", "mlp.kind"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 5, "groups"),
    (("layers", 0, "mlp", "expert"), None, "mlp.expert"),
    (("loop", "stop"), 7, "loop"),
    (("loop", "times"), 0, "loop"),
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


def test_kept_groups_must_hold_enough_experts():
    c = copy.deepcopy(CFG_A)
    c["layers"][0]["mlp"]["router"].update(top=3, groups={"count": 3, "keep": 1})
    with pytest.raises(ConfigError):
        load_config(c)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_tensor_list_is_the_files(name):
    cfg = CONFIGS[name]
    w = random_weights(cfg, 1, RANKS[name])
    specs = tensor_specs_for_config(copy.deepcopy(cfg))
    assert set(specs) == set(w)
    for k, s in specs.items():
        assert len(s.shape) == w[k].dim() and all(a < 0 or a == b for a, b in zip(s.shape, w[k].shape)), k
    free = [k for k, s in specs.items() if any(a < 0 for a in s.shape)]
    assert sorted(free) == sorted(f"l{i}.mix.{t}" for i, L in enumerate(cfg["layers"]) if L["type"] == "gla" for t in ("a1", "a2"))
    c = copy.deepcopy(cfg)
    for i, L in enumerate(c["layers"]):
        if L["type"] == "gla":
            L["mixer"]["rank"] = RANKS[name][i]                                  # given: the list is then exact
    assert all(tuple(s.shape) == tuple(w[k].shape) for k, s in tensor_specs_for_config(c).items())


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_agrees_with_itself_step_by_step(name):
    cfg = CONFIGS[name]
    w = {k: v.double() for k, v in random_weights(cfg, 2, RANKS[name]).items()}
    ids = prompts(cfg["vocab"], [23], seed=1)[0]
    whole = plain.forward(cfg, w, ids)
    for first in (1, 2, 9):
        assert torch.allclose(plain.forward_stepwise(cfg, w, ids, first), whole, atol=1e-9, rtol=1e-9)
    cap = cfg.get("logit_softcap")
    if cap:
        assert float(whole.abs().max()) < cap


def test_routing_in_the_plain_implementation():
    """Groups that are not kept are out even when their experts' choice scores are the largest of all negative ones."""
    t = {"router": torch.eye(6, dtype=torch.float64) * 0, "correction": torch.tensor([-3.0, -3.0, -0.9, -5.0, -1.0, -1.0], dtype=torch.float64)}
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    idx, wt = plain.route(torch.zeros(1, 6, dtype=torch.float64), r, t, "")
    assert sorted(idx[0].tolist()) == [4, 5]                   # group sums: -5, -4.9, -1; expert 2 alone does not save its group
    assert torch.allclose(wt.sum(-1), torch.ones(1, dtype=torch.float64))
    r["groups"]["keep"] = 2
    assert sorted(plain.route(torch.zeros(1, 6, dtype=torch.float64), r, t, "")[0][0].tolist()) == [2, 4]


def test_weight_files_decide_free_sizes_and_wrong_ones_are_reported(tmp_path):
    from trapetum_b200.weights.loader import WeightError, load_tensors
    cfg = CFG_B
    w = random_weights(cfg, 3, RANKS["B"])
    folder = write_folder(str(tmp_path / "ok"), cfg, w)
    specs = tensor_specs_for_config(copy.deepcopy(cfg))
    got = load_tensors(folder, specs, torch.float32, "cpu")
    assert got["l0.mix.a1"].shape[0] == RANKS["B"][0]
    bad = dict(w)
    bad["l0.mix.a1"] = w["l0.mix.a1"][:, :-1].contiguous()
    del bad["final.norm.b"]
    with pytest.raises(WeightError) as e:
        load_tensors(write_folder(str(tmp_path / "bad"), cfg, bad), specs, torch.float32, "cpu")
    assert "l0.mix.a1" in str(e.value) and "final.norm.b" in str(e.value)
