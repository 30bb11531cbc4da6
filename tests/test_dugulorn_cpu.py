"""Dugulorn without a GPU: the configuration reader and its refusals, the model as data (tensor names, cache units, state
sizes, the run list of a layer that reads another layer's cache), the loader's sizes left to the checkpoint, and the plain
implementation checked against closed forms and against what the test models are meant to show."""
import copy
import math

import pytest
import torch

import dugulorn_models as dm
import plain_dugulorn as plain
from cppvllm_b200.config.dugulorn_config import ChannelDeltaConfig, DugulornConfig, LatentAttentionConfig, LightningConfig
from cppvllm_b200.config.model_config import ConfigError
from cppvllm_b200.config.registry import resolve_architecture
from cppvllm_b200.parts.base import Runtime, Workspace
from cppvllm_b200.parts.model import CausalLM


def _model(cfg_dict):
    arch = resolve_architecture(cfg_dict)
    spec = arch.build_spec(arch.parse_config(cfg_dict))
    cpu = torch.device("cpu")
    return CausalLM(spec, Runtime(cpu, torch.float32, Workspace(cpu, 0), max_positions=64)), spec


def test_the_configuration_is_read_layer_by_layer():
    cfg = DugulornConfig.from_dict(dm.DG_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, len(cfg.layers)) == (97, 48, 1e-5, 4)
    a, b, c, d = (l.mixer for l in cfg.layers)
    assert isinstance(a, LatentAttentionConfig) and (a.heads, a.dim, a.rot_dim, a.vdim, a.q_rank, a.kv_rank, a.kv_from) == (3, 16, 8, 12, 24, 16, None)
    assert (a.rot.dims, a.rot.base, a.rot.factor, a.rot.original, a.rot.fast, a.rot.slow) == (8, 100.0, 3.0, 40.0, 8.0, 1.0)
    assert isinstance(b, LightningConfig) and b.decay == (0.9, 0.995) and cfg.layers[1].ff == 0
    assert c.kv_from == 0 and cfg.layers[2].ff == 56
    assert isinstance(d, ChannelDeltaConfig) and (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (4, 2, 12, 20, 3)
    plain_rot = DugulornConfig.from_dict(dm.DG_B).layers[1].mixer.rot
    assert (plain_rot.factor, plain_rot.original) == (1.0, 0.0)          # no stretching named: none applied


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="attention"), "not a mixer of this design"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "earlier latent_attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier latent_attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=32), "must equal that layer's"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decays"),
    (lambda c: c["layers"][3]["mixer"].update(kv_heads=3), "query/key heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rotated elements"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda c: c.pop("norm"), "norm.eps"),
])
def test_the_reader_refuses_what_does_not_fit(change, text):
    cfg = copy.deepcopy(dm.DG_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        DugulornConfig.from_dict(cfg)


def test_a_layer_that_reads_another_layers_cache_follows_a_layer_in_between_that_writes_none():
    cfg = copy.deepcopy(dm.DG_B)          # layers: delta, latent, lightning, latent reading layer 1
    model, spec = _model(cfg)
    order = [(e.layer, e.cache, e.writes_cache) for e in model.run_order]
    assert order[1][1:] == (1, True) and order[3][1:] == (1, False)
    units = model.cache_units()
    assert list(units) == [1] and units[1].entry_shape == (48 + 16,) and units[1].token_axis == 0
    states = model.state_specs()
    assert states[0].shape == (2 * 64 * 40 + 3 * (2 * 64 + 2 * 40),) and states[2].shape == (2 * 64 * 64,)
    assert states[1] is None and states[3] is None
    assert spec.residual_dtype == "float32" and spec.lm_head.names == {"weight": "embed"}


def test_tensor_names_and_shapes():
    model, _ = _model(dm.DG_A)
    ws = model.weight_specs()
    expect = {
        "embed": (97, 48), "embed.norm": (48,), "final.norm": (48,),
        "l0.mix.dq": (24, 48), "l0.mix.dq.norm": (24,), "l0.mix.uq": (3 * 24, 24), "l0.mix.dkv": (24, 48), "l0.mix.dkv.norm": (16,),
        "l0.mix.uk": (48, 16), "l0.mix.uv": (36, 16), "l0.mix.g": (3, 48), "l0.mix.o": (48, 36),
        "l0.mlp.up": (40, 48), "l0.mlp.up.b": (40,), "l0.mlp.down": (48, 40), "l0.mlp.down.b": (48,), "l0.norm1": (48,), "l0.norm2": (48,),
        "l1.mix.q": (20, 48), "l1.mix.k": (20, 48), "l1.mix.v": (14, 48), "l1.mix.g": (14, 48), "l1.mix.o": (48, 14), "l1.mix.norm": (14,),
        "l3.mix.q": (24, 48), "l3.mix.q.conv": (24, 3), "l3.mix.k.conv": (24, 3), "l3.mix.v": (80, 48), "l3.mix.v.conv": (80, 3),
        "l3.mix.b": (4, 48), "l3.mix.A_log": (4,), "l3.mix.norm": (20,), "l3.mix.a1": (6, 48), "l3.mix.a2": (48, 6),
        "l3.mix.dt_bias": (48,), "l3.mix.g1": (10, 48), "l3.mix.g2": (80, 10), "l3.mix.o": (48, 80),
    }
    for name, shape in expect.items():
        assert ws[name].shape == shape, name
    assert "l2.mix.dkv" not in ws and "l2.mix.dkv.norm" not in ws and "l2.mix.uk" in ws      # the reader of layer 0's cache
    assert "l1.norm2" not in ws and not any(n.startswith("l1.mlp") for n in ws)


def test_sizes_left_to_the_checkpoint(tmp_path):
    """The inner sizes of the delta mixer's low-rank projections are named by no configuration key: without the writer's
    optional keys the declaration leaves them open and the loader takes what the file holds."""
    from cppvllm_b200.weights.loader import WeightError, _shape_fits
    cfg = copy.deepcopy(dm.DG_A)
    del cfg["layers"][3]["mixer"]["a_rank"], cfg["layers"][3]["mixer"]["g_rank"]
    model, _ = _model(cfg)
    ws = model.weight_specs()
    assert ws["l3.mix.a1"].shape == (-1, 48) and ws["l3.mix.g2"].shape == (80, -1)
    assert _shape_fits((24, 48), (-1, 48)) and not _shape_fits((24, 47), (-1, 48)) and not _shape_fits((24,), (-1, 48))
    d = dm.write_model(str(tmp_path / "open"), cfg, 5)
    w = plain.read_weights(d)
    assert w["l3.mix.a1"].shape[0] == w["l3.mix.a2"].shape[1] > 0


def test_rotation_tables_equal_the_plain_frequencies():
    from cppvllm_b200.parts.base import build_part
    model, spec = _model(dm.DG_C)
    (name, part), = model.positions.items()
    rot = dm.DG_C["layers"][0]["mixer"]["rot"]
    freq, mag = plain.rotation_frequencies(rot)
    ang = torch.arange(64, dtype=torch.float64)[:, None] * freq[None, :]
    assert torch.allclose(part.cos.double(), torch.cos(ang) * mag, atol=1e-6) and torch.allclose(part.sin.double(), torch.sin(ang) * mag, atol=1e-6)
    assert mag == pytest.approx(0.1 * math.log(8.0) + 1.0) and freq[0] == pytest.approx(1.0)
    assert float(freq[-1]) == pytest.approx(5000.0 ** (-30 / 32) / 8.0)       # the slowest pair is fully stretched


# ---- the plain implementation against closed forms ------------------------------------------------------------------

def test_plain_rotation_keeps_lengths_and_depends_on_the_distance_only():
    rot = {"dims": 8, "base": 100.0}
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 12, generator=g, dtype=torch.float64), torch.randn(1, 12, generator=g, dtype=torch.float64)
    def dot(p, s):
        return float((plain.rotate(q, torch.tensor([p]), rot) * plain.rotate(k, torch.tensor([s]), rot)).sum())
    assert dot(9, 4) == pytest.approx(dot(25, 20)) and dot(9, 4) != pytest.approx(dot(9, 5))
    r = plain.rotate(q, torch.tensor([7]), rot)
    assert float(r.norm()) == pytest.approx(float(q.norm())) and torch.equal(r[:, 8:], q[:, 8:])      # the rest passes
    assert float(r[0, 0]) == pytest.approx(float(q[0, 0] * math.cos(7.0) - q[0, 1] * math.sin(7.0)))   # pair (0, 1), frequency 1


def test_plain_lightning_rule_is_a_decaying_sum():
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(9, 2, n, generator=g, dtype=torch.float64) for n in (5, 5, 3))
    o = plain.lightning_rule(q, k, v, [0.8, 1.0])
    for h, d in enumerate([0.8, 1.0]):
        for t in (0, 4, 8):
            ref = sum(d ** (t - s) * float(q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(o[t, h], ref)


def test_plain_delta_rule_overwrites_what_a_key_holds():
    """With no decay and beta = 1 the matrix maps a unit key to the last value written under it; with beta = 0 it keeps the old one."""
    k = torch.zeros(4, 1, 6, dtype=torch.float64)
    k[0, 0, 0] = k[1, 0, 1] = k[2, 0, 0] = k[3, 0, 0] = 1.0
    v = torch.arange(8, dtype=torch.float64).reshape(4, 1, 2) + 1.0
    ones = torch.ones(4, 1, 6, dtype=torch.float64)
    o = plain.delta_rule(k, k, v, ones, torch.tensor([[1.0], [1.0], [1.0], [0.0]], dtype=torch.float64))
    assert torch.allclose(o[2, 0], v[2, 0]) and torch.allclose(o[3, 0], v[2, 0]) and torch.allclose(o[1, 0], v[1, 0])
    half = plain.delta_rule(k, k, v, 0.5 * ones, torch.ones(4, 1, dtype=torch.float64))
    assert torch.allclose(half[2, 0], v[2, 0])                              # the read-out sees the current token's write


def test_plain_convolution_puts_its_last_tap_on_the_current_token():
    u = torch.arange(10, dtype=torch.float64).reshape(5, 2) + 1.0
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = plain.causal_conv(u, taps)
    assert torch.equal(y[:, 0], u[:, 0])
    assert torch.equal(y[:, 1], torch.tensor([0.0, 0.0, 2.0, 4.0, 6.0], dtype=torch.float64))       # two tokens back, zeros before the start


@pytest.fixture(scope="module")
def dg_dirs(tmp_path_factory):
    return dm.write_all(str(tmp_path_factory.mktemp("dugulorn")))


@pytest.mark.parametrize("name", ["dg_a", "dg_b", "dg_c", "dg_d"])
def test_the_test_models_show_a_lost_past(dg_dirs, name):
    """What an engine would compute after losing a cache page or a state slot: the sequence without its first tokens.  The
    last logits must then differ by far more than any tolerance the engine tests use, also when 150 tokens lie between."""
    d, vocab = dg_dirs[name], dm.config(name)["vocab"]
    toks = dm.random_tokens(vocab, 170, 3)
    full = plain.forward(d, toks)[-1]
    for drop, least in ((1, 2e-4), (20, 1e-2)):      # the engine tests' float32 tolerance is 2e-5
        cut = plain.forward(d, toks[drop:])[-1]
        assert float((full - cut).abs().max()) > least * float(full.abs().max()), (name, drop)


def test_greedy_generation_repeats_the_forward_pass(dg_dirs):
    d = dg_dirs["dg_a"]
    p = dm.random_tokens(97, 5, 1)
    out = plain.greedy_generate(d, p, 3)
    assert out[0] == int(plain.forward(d, p)[-1].argmax()) and out[1] == int(plain.forward(d, p + out[:1])[-1].argmax())
