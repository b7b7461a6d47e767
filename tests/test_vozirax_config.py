"""The Vozirax configuration, its tensors, its caches, and the plain implementation's own mechanisms, without a GPU."""
import copy
import math

import pytest
import torch

from plain import vozirax_plain as ZP
from vozirax_helpers import CONFIG_A, CONFIG_B, CONFIG_C, CONFIGS


def _spec(d):
    from transformers_neuronx_b200.config import config_from_dict
    arch, cfg = config_from_dict(copy.deepcopy(d))
    return arch, cfg, arch.build_spec(cfg)


def test_the_architecture_is_found_by_its_single_name_and_round_trips():
    from transformers_neuronx_b200.config import VoziraxConfig, config_from_dict
    arch, cfg, spec = _spec(CONFIG_A)
    assert arch.name == "Vozirax" and isinstance(cfg, VoziraxConfig)
    again = config_from_dict(cfg.to_dict())[1]
    assert again == cfg and again.to_dict()["layers"] == CONFIG_A["layers"]
    assert spec.vocab_size == 211 and spec.hidden_size == 72 and len(spec.layers) == 5
    assert all(l.block == "parallel_residual" and l.norm1.weight_offset == 1.0 and l.norm1.eps == 1e-4 for l in spec.layers)
    assert spec.head.final_norm.weight_offset == 1.0 and spec.head.logit_scale == 0.7
    assert spec.embedding.position.kind == "sinusoidal" and spec.embedding.position.dim == 72
    assert [(e.layer, e.cache) for e in spec.schedule] == [(i, i) for i in range(5)]


def test_tensor_names_and_shapes_follow_the_layers():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_A)
    t = {s.name: tuple(s.shape) for s in DecoderModel(spec).tensor_specs()}
    assert t["embed"] == (211, 72) and t["head"] == (211, 72) and t["final.norm"] == (72,)
    # attention: two maps a head in q and k, one gate a head, no biases
    assert t["l0.mix.q"] == (6 * 2 * 12, 72) and t["l0.mix.k"] == (2 * 2 * 12, 72) and t["l0.mix.v"] == (2 * 40, 72)
    assert t["l0.mix.g"] == (6, 72) and t["l0.mix.o"] == (72, 240) and t["l0.mix.q.norm"] == (12,) == t["l0.mix.k.norm"]
    assert all(t[f"l0.mix.{n}"] == (12,) for n in ("lq1", "lk1", "lq2", "lk2")) and "l0.mix.q.b" not in t
    assert all(t[f"l0.{n}"] == (72,) for n in ("norm1", "norm2", "ls1", "ls2"))
    # routed experts without gates, a correction per expert
    assert t["l0.mlp.router"] == (6, 72) and t["l0.mlp.correction"] == (6,) and "l0.mlp.e0.gate" not in t
    assert all(t[f"l0.mlp.e{j}.up"] == (20, 72) and t[f"l0.mlp.e{j}.down"] == (72, 20) for j in range(6)) and "l0.mlp.e6.up" not in t
    # the state-space layer: one input projection [z | x | B | C | dt], the convolution over x, B and C; no feed-forward
    assert t["l1.mix.in"] == (2 * 60 + 2 * 3 * 18 + 6, 72) and t["l1.mix.conv"] == (60 + 108, 5) and t["l1.mix.conv.b"] == (168,)
    assert t["l1.mix.dt_bias"] == t["l1.mix.A_log"] == t["l1.mix.D"] == (6,) and t["l1.mix.norm"] == (60,) and t["l1.mix.o"] == (72, 60)
    assert "l1.norm2" not in t and "l1.ls2" not in t and "l1.mlp.up" not in t and t["l1.ls1"] == (72,)
    # a reader has neither keys nor values, nor their norm
    assert "l2.mix.k" not in t and "l2.mix.v" not in t and "l2.mix.k.norm" not in t and t["l2.mix.q"] == (144, 72)
    assert t["l2.mlp.gate"] == (88, 72) == t["l2.mlp.up"] and t["l2.mlp.down"] == (72, 88)


def test_pages_and_state_of_every_layer():
    from transformers_neuronx_b200.cache.manager import FixedStateNeed, PagedKVNeed
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_A)
    needs = DecoderModel(spec).cache_needs()
    # both maps of a key side by side: rows of max(2 x 12, 40) -> 48 dims, on 2 key/value heads; the reader keeps nothing
    assert needs[(0, 0)] == PagedKVNeed(2, 48, None, None) and not any(k[0] == 2 for k in needs if isinstance(k, tuple))
    assert needs[(1, 0)] == FixedStateNeed((6, 10, 18), "float32") and needs[(1, 1)] == FixedStateNeed((4, 168), "activation")
    assert needs[(3, 0)] == FixedStateNeed((2, 24, 8), "float32") and needs[(3, 1)] == FixedStateNeed((1, 64), "activation")
    assert needs[(4, 0)] == PagedKVNeed(3, 48, None, None)
    _, _, spec_c = _spec(CONFIG_C)
    needs_c = DecoderModel(spec_c).cache_needs()
    assert (0, 1) not in needs_c and needs_c[(0, 0)] == FixedStateNeed((1, 50, 30), "float32")      # one tap: no past
    assert needs_c[(1, 0)] == PagedKVNeed(1, 112, None, None)


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].update(type="retnet"), "unknown layer type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "cannot share"),
    (lambda d: d["layers"][0]["mixer"].update(scale=0.0), "scale"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mixer"].update(q_temp={"coef": 1.0, "every": 0}), "every"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=1), "no keys and values"),
    (lambda d: d["layers"][4]["mixer"].update(kv_from=2), "no keys and values"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=24), "differs"),
    (lambda d: d["layers"][1]["mixer"].update(groups=4), "groups"),
    (lambda d: d["layers"][1]["mixer"].update(norm_groups=7), "equal parts"),
    (lambda d: d["layers"][1]["mixer"].update(conv=0), "conv"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "not a choice"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=1), "fewer than"),
    (lambda d: d["layers"][0]["mlp"].update(kind="switch"), "kind"),
    (lambda d: d.update(logit_scale="big"), "logit_scale"),
    (lambda d: d["norm"].update(eps=0.0), "eps")])
def test_a_configuration_that_cannot_be_run_is_refused_by_name(edit, word):
    from transformers_neuronx_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(CONFIG_A)
    edit(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_a_mechanism_whose_key_is_absent_is_not_there():
    d = copy.deepcopy(CONFIG_A)
    d.pop("logit_scale")
    d["layers"][3]["mixer"].pop("groups"); d["layers"][3]["mixer"].pop("norm_groups")
    d["layers"][4]["mixer"].pop("kv_heads")
    d["layers"][3]["mlp"]["router"].pop("scale")
    _, cfg, spec = _spec(d)
    assert spec.head.logit_scale == 1.0 and spec.layers[3].mixer.groups == 1 and spec.layers[3].mixer.norm_groups == 1
    assert spec.layers[4].mixer.n_kv_heads == 3 and spec.layers[3].feed_forward.weight_scale == 1.0
    assert spec.layers[1].feed_forward is None and spec.layers[4].mixer.temp_every == 0 and spec.layers[3].feed_forward.n_groups == 1


def test_sizes_the_kernels_do_not_take_are_refused_when_the_model_is_built():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    d = copy.deepcopy(CONFIG_A)
    d["layers"][1]["mixer"].update(state=300)
    with pytest.raises(ValueError, match="state size"):
        DecoderModel(_spec(d)[2])
    d = copy.deepcopy(CONFIG_A)
    d["layers"][1]["mixer"].update(conv=9)
    with pytest.raises(ValueError, match="taps"):
        DecoderModel(_spec(d)[2])


def test_all_configurations_build():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    for d in CONFIGS.values():
        model = DecoderModel(_spec(d)[2])
        assert model.graph_safe and "ssd" in model.libraries() and "diff_attention" in model.libraries()


def test_plain_sinusoid_interleaves_sine_and_cosine():
    s = ZP.sinusoid([0, 3], 6)
    assert s[0].tolist() == [0.0, 1.0, 0.0, 1.0, 0.0, 1.0]
    w = [1.0, 10000.0 ** (-2.0 / 6), 10000.0 ** (-4.0 / 6)]
    for i in range(3):
        assert abs(float(s[1, 2 * i]) - math.sin(3 * w[i])) < 1e-6 and abs(float(s[1, 2 * i + 1]) - math.cos(3 * w[i])) < 1e-6


def test_plain_convolution_puts_the_last_column_on_the_current_token():
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)           # taps: two back, one back, now
    y = ZP.causal_conv(u, w, torch.tensor([0.5], dtype=torch.float64), 3)
    assert y.reshape(-1).tolist() == [1.5, 12.5, 123.5]                 # zeros before the start


def test_plain_state_space_recurrence_is_the_closed_form_where_there_is_one():
    """One head, a state of one, one tap with weight one and no bias: y_t = C_t sum_s prod_(s<r<=t) a_r dt_s B_s x_s + D x_t."""
    T, W = 5, 4
    g = torch.Generator().manual_seed(1)
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    t = {"in": torch.randn(5, W, generator=g, dtype=torch.float64), "conv": torch.ones(3, 1, dtype=torch.float64),
         "conv.b": torch.zeros(3, dtype=torch.float64), "dt_bias": torch.tensor([0.3], dtype=torch.float64),
         "A_log": torch.tensor([-0.5], dtype=torch.float64), "D": torch.tensor([0.7], dtype=torch.float64),
         "norm": torch.ones(1, dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)}
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "norm_groups": 1, "conv": 1}
    u = h @ t["in"].T
    z, x, B, C = u[:, 0], ZP.silu(u[:, 1]), ZP.silu(u[:, 2]), ZP.silu(u[:, 3])
    dt = torch.log1p(torch.exp(u[:, 4] + 0.3))
    a = torch.exp(-math.exp(-0.5) * dt)
    want = []
    for i in range(T):
        s = sum(float(torch.prod(a[j + 1:i + 1])) * float(dt[j] * B[j] * x[j]) for j in range(i + 1))
        y = (float(C[i]) * s + 0.7 * float(x[i])) * float(ZP.silu(z[i]))
        want.append(y / math.sqrt(y * y + 1e-5))                        # a norm over one value keeps its sign
    got = ZP.ssd(h, t, "", m, 1e-5).reshape(-1)
    assert float((got - torch.tensor(want, dtype=torch.float64)).abs().max()) < 1e-12


def test_plain_routing_keeps_the_best_groups_and_weighs_by_the_uncorrected_scores():
    """Four experts in two groups, one kept, one expert a token.  The logits make expert 3 the best uncorrected score, but
    the correction lifts group 0's pair sum; the choice must come from group 0 although its choice scores are negative,
    and the weight is the chosen expert's sigmoid over itself, times the scale."""
    h = torch.eye(4, dtype=torch.float64)[:1]
    t = {"router": torch.tensor([[0.0], [-1.0], [-3.0], [2.0]], dtype=torch.float64).repeat(1, 4) * torch.eye(4, dtype=torch.float64)[0],
         "correction": torch.tensor([-0.9, -0.8, -2.0, -1.5], dtype=torch.float64)}
    r = {"experts": 4, "top": 1, "scale": 3.0, "groups": {"count": 2, "keep": 1}}
    (ids, w), = ZP.route(h, t, "", r)
    # choice scores: 0.5 - 0.9, 0.269 - 0.8, 0.047 - 2.0, 0.881 - 1.5: group sums -0.93 and -2.57
    assert ids == [0] and abs(float(w[0]) - 3.0) < 1e-9
    r["groups"]["keep"] = 2
    assert ZP.route(h, t, "", r)[0][0] == [0]                            # -0.4 beats -0.62 without the groups too
    t["correction"][3] = -1.2
    assert ZP.route(h, t, "", r)[0][0] == [3]
    r["groups"]["keep"] = 1
    assert ZP.route(h, t, "", r)[0][0] == [0]                            # group 1 (-0.32 - 1.95) still loses to group 0


def test_plain_differential_attention_of_one_token_is_its_value_normalised():
    """A single position: both softmaxes are 1, so o = (1 - lambda) v, whose norm removes the factor's size but keeps its sign."""
    g = torch.Generator().manual_seed(2)
    W, H, G, d, dv = 8, 2, 1, 4, 6
    t = {k: torch.randn(s, generator=g, dtype=torch.float64) for k, s in
         (("q", (H * 2 * d, W)), ("k", (G * 2 * d, W)), ("v", (G * dv, W)), ("g", (H, W)), ("o", (W, H * dv)), ("q.norm", (d,)),
          ("k.norm", (d,)), ("lq1", (d,)), ("lk1", (d,)), ("lq2", (d,)), ("lk2", (d,)))}
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.3, "diff": 0.25, "q_temp": {"coef": 0.5, "every": 3}}
    h = torch.randn(1, W, generator=g, dtype=torch.float64)
    lam = math.exp(float(t["lq1"] @ t["lk1"])) - math.exp(float(t["lq2"] @ t["lk2"])) + 0.25
    v = (t["v"] @ h[0])
    o = ZP.rms((1 - lam) * v, 1e-6) * 0.75
    gate = torch.sigmoid(t["g"] @ h[0])
    want = t["o"] @ torch.cat([o * gate[0], o * gate[1]])
    got, _ = ZP.differential_attention(h, t, "", m, 1e-6)
    assert float((got[0] - want).abs().max()) < 1e-12
