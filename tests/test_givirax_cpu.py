"""Givirax without a GPU: the configuration reader, the model as data (run list, caches, tensor names), the cache
managers' kept first pages, and that the test models are sharp enough for a mask that is one token off to show."""
import copy
import random

import pytest
import torch

import givirax_models as gm
import plain_givirax as plain
from cppvllm_b200.cache.manager import CacheManager, GroupConfig
from cppvllm_b200.config.givirax_config import GiviraxConfig
from cppvllm_b200.config.model_config import ConfigError
from cppvllm_b200.config.registry import resolve_architecture
from cppvllm_b200.parts.base import CacheSpec, Runtime, Workspace
from cppvllm_b200.parts.model import CausalLM


def build(cfg):
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    cpu = torch.device("cpu")
    return spec, CausalLM(spec, Runtime(cpu, torch.float32, Workspace(cpu, 0)))


def test_configuration_is_read_from_the_file_alone():
    c = GiviraxConfig.from_dict(gm.GV_A)
    assert (c.vocab, c.width, c.max_positions, c.embedding_scale, c.norm_eps) == (97, 48, 160, 2.5, 1e-5)
    assert (c.loop_start, c.loop_stop, c.loop_times) == (1, 3, 3) and c.has_loop
    assert [l.mlp.kind if l.mlp else None for l in c.layers] == ["dense", "moe", None]
    assert (c.layers[1].mlp.experts, c.layers[1].mlp.top, c.layers[1].mlp.ff) == (5, 2, 24)
    m = c.layers[0].mixer
    assert (m.heads, m.kv_heads, m.dim, m.window, m.keep_first, m.scale) == (3, 1, 16, 9, 2, 0.3)
    assert not GiviraxConfig.from_dict(gm.GV_B).has_loop
    assert resolve_architecture(gm.GV_B).name == "Givirax"
    for breaker in (lambda d: d.pop("vocab"), lambda d: d["layers"][0].update(type="conv"),
                    lambda d: d["layers"][1]["mlp"].update(kind="glu"), lambda d: d["layers"][0]["mixer"].update(vdim=8),
                    lambda d: d["layers"][0]["mixer"].update(kv_heads=2), lambda d: d["loop"].update(stop=7),
                    lambda d: d["layers"][1]["mlp"]["router"].update(top=6), lambda d: d["norm"].pop("eps")):
        bad = copy.deepcopy(gm.GV_A)
        breaker(bad)
        with pytest.raises(ConfigError):
            GiviraxConfig.from_dict(bad)


def test_run_list_caches_and_tensor_names():
    spec, model = build(gm.GV_A)
    order = [(e.layer, e.input, e.input_index) for e in model.run_order]
    assert order == [(0, None, 0), (1, "loop", 0), (2, None, 0), (1, "loop", 1), (2, None, 0), (1, "loop", 2), (2, None, 0)]
    assert len({e.cache for e in model.run_order}) == 7                  # every pass has a cache of its own
    assert set(model.cache_units().values()) == {CacheSpec.keys_only(1, 16, 9, 2)}
    names = set(model.weight_specs())
    assert {"embed", "pos", "loop.step", "l0.norm1", "l0.mix.q", "l0.mix.k", "l0.mix.o", "l0.mlp.up", "l0.mlp.down",
            "l1.mlp.router", "l1.mlp.router.b", "l1.mlp.e4.gate", "l1.mlp.e0.down", "final.norm", "head"} <= names
    assert not any(n.startswith("l2.mlp") or n.endswith(".v") for n in names)
    assert model.weight_specs()["loop.step"].shape == (3, 48) and model.weight_specs()["l1.mlp.e2.up"].shape == (24, 48)
    spec_b, model_b = build(gm.GV_B)
    assert spec_b.inputs == {} and [e.input for e in model_b.run_order] == [None] * 3
    assert len(set(model_b.cache_units().values())) == 3                 # three shapes of cache: three groups of pages
    assert spec.residual_dtype == "float32"


def managers(groups, page, slots, width):
    out = [CacheManager(groups, page, slots)]
    try:
        from cppvllm_b200.cache.native import NativeCacheManager
        out.append(NativeCacheManager(groups, page, slots, width))
    except Exception as e:                                               # no compiler on this machine
        pytest.skip(f"the C++ cache manager could not be built: {e}")
    return out


def test_kept_first_pages_stay_while_the_window_gives_the_others_back():
    for m in managers([GroupConfig(12, window=10, keep_first=5), GroupConfig(12, window=10)], 4, 2, 40):
        m.admit("r")
        m.reserve("r", 30)
        m.advance("r", 30)
        kept, plain_window = [list(t) for t in m.lease("r").tables]
        # the next token (position 30) reads 21..30: pages 5.. ; positions 0..4 are kept: pages 0 and 1 stay
        assert [p >= 0 for p in kept] == [True, True, False, False, False, True, True, True]
        assert [p >= 0 for p in plain_window] == [False] * 5 + [True] * 3
        m.reserve("r", 31)
        m.advance("r", 31)
        assert list(m.lease("r").tables[0])[:2] == kept[:2]
        m.check_invariants()
        m.release("r")
        assert m.num_free_pages(0) == 12 and m.num_free_pages(1) == 12


def test_both_managers_agree_on_random_histories_with_kept_pages():
    rng = random.Random(3)
    groups = [GroupConfig(20, window=11, keep_first=6), GroupConfig(20, window=5, keep_first=1), GroupConfig(20)]
    py, nat = managers(groups, 4, 4, 32)
    live = {}
    for step in range(300):
        if live and rng.random() < 0.15:
            rid = rng.choice(list(live))
            py.release(rid), nat.release(rid)
            del live[rid]
        elif len(live) < 4 and rng.random() < 0.3:
            rid = f"r{step}"
            py.admit(rid), nat.admit(rid)
            live[rid] = 0
        elif live:
            rid = rng.choice(list(live))
            upto = live[rid] + rng.choice([1, 1, 2, 7, 13])
            if upto > 120 or not py.can_reserve(rid, upto):
                assert upto > 120 or not nat.can_reserve(rid, upto)
                continue
            py.reserve(rid, upto), nat.reserve(rid, upto)
            py.advance(rid, upto), nat.advance(rid, upto)
            live[rid] = upto
        for rid in live:
            for g in range(3):
                assert list(py.lease(rid).tables[g]) == [int(x) for x in nat.lease(rid).tables[g]]
        for g in range(3):
            assert py.num_free_pages(g) == nat.num_free_pages(g)
    py.check_invariants(), nat.check_invariants()


def test_plain_mechanisms_one_by_one():
    torch.manual_seed(0)
    x = torch.randn(5, 8, dtype=torch.float64)
    w = torch.rand(8, dtype=torch.float64) + 0.5
    n = plain.rms_norm(x, w, 1e-3)
    assert torch.allclose(n / w * torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3), x)
    vis = plain.visible(12, 4, 2)
    assert vis[11].tolist() == [True, True] + [False] * 6 + [True] * 4       # two kept, then the last four
    assert vis[3].tolist() == [True] * 4 + [False] * 8 and plain.visible(5, 0, 0)[4].all()
    z = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
    chosen, weights = plain.route(torch.eye(3, dtype=torch.float64), torch.tensor([[1.0, 0, 0], [1.0, 0, 0], [0, 2.0, 0], [0, 0, 0.5]],
                                  dtype=torch.float64), torch.tensor([0.0, 0.0, 0.0, 0.1], dtype=torch.float64), 2)
    assert chosen == [[0, 1], [2, 3], [3, 0]]                               # equal logits: the lower index first
    assert torch.allclose(weights[0], torch.tensor([0.5, 0.5], dtype=torch.float64))
    # attention with unit keys (which are the values too)
    k = torch.eye(6, dtype=torch.float64)
    n6 = torch.eye(6, dtype=torch.float64)
    y = plain.attention(n6, torch.zeros(6, 6, dtype=torch.float64), torch.eye(6, dtype=torch.float64), torch.eye(6, dtype=torch.float64),
                        1, 1, 6, 1.0, 3, 0)
    assert torch.allclose(y[5], (k[3] + k[4] + k[5]) / 3)                   # zero queries: the mean of the visible keys


@pytest.mark.parametrize("name", ["gv_a", "gv_c"])
def test_the_test_models_show_a_mask_that_is_one_token_off(tmp_path, name):
    """The sharpened weights make the logits move by a twentieth of their size or more when the window is one token longer
    or the kept first tokens one fewer: thousands of times the float32 tolerance of the engine tests, so a fault of that
    kind cannot hide in it."""
    cfg = gm.config(name)
    d = gm.write_model(str(tmp_path / name), cfg, gm.SETUPS[name][1])
    toks = gm.random_tokens(cfg["vocab"], 100, 1)
    w = plain.read_weights(d)
    ref = plain.forward(d, toks, w, cfg)
    scale = float(ref.abs().max())
    for key, delta in (("size", 1), ("keep_first", -1)):
        other = copy.deepcopy(cfg)
        for layer in other["layers"]:
            layer["mixer"]["mask"][key] += delta
        moved = float((plain.forward(d, toks, w, other) - ref).abs().max()) / scale
        assert moved > 0.05, (key, moved)
