"""The Tutelix configuration, its tensors, its schedule and caches, and the plain implementation's own mechanisms,
without a GPU."""
import copy
import math

import pytest
import torch

from plain import tutelix_plain as TP
from tutelix_helpers import CONFIG_A, CONFIG_B, CONFIG_C, CONFIGS


def _spec(d):
    from transformers_neuronx_b200.config import config_from_dict
    arch, cfg = config_from_dict(copy.deepcopy(d))
    return arch, cfg, arch.build_spec(cfg)


def test_the_architecture_is_found_by_its_single_name_and_round_trips():
    from transformers_neuronx_b200.config import TutelixConfig, config_from_dict
    arch, cfg, spec = _spec(CONFIG_A)
    assert arch.name == "Tutelix" and isinstance(cfg, TutelixConfig)
    again = config_from_dict(cfg.to_dict())[1]
    assert again == cfg and again.to_dict()["layers"] == CONFIG_A["layers"] and again.to_dict()["loop"] == CONFIG_A["loop"]
    assert spec.vocab_size == 211 and spec.hidden_size == 72 and len(spec.layers) == 4
    assert spec.embedding.scale == 3.7 and all(l.block == "sandwich_norm" for l in spec.layers)
    assert all(l.norm1.weight_offset == 1.0 and l.norm1_post.weight_offset == 1.0 and l.norm1.eps == 1e-4 for l in spec.layers)
    assert spec.head.final_norm.weight_offset == 1.0


def test_a_looped_run_of_layers_is_walked_several_times_each_pass_with_a_cache_of_its_own():
    _, cfg, spec = _spec(CONFIG_A)
    assert cfg.layer_order() == [0, 1, 2, 1, 2, 1, 2, 3] == TP.layer_order(CONFIG_A)
    assert [e.layer for e in spec.schedule] == cfg.layer_order()
    assert len({e.cache for e in spec.schedule}) == 8                  # no two runs share a past
    _, cfg_b, spec_b = _spec(CONFIG_B)
    assert cfg_b.layer_order() == [0, 1, 2, 2, 3, 4] == TP.layer_order(CONFIG_B)
    _, cfg_c, _ = _spec(CONFIG_C)
    assert cfg_c.layer_order() == [0, 1, 2, 3]                          # no loop
    d = copy.deepcopy(CONFIG_C)
    d["loop"] = {"start": 0, "stop": 4, "times": 1}                     # a loop of one pass changes nothing
    assert _spec(d)[1].layer_order() == [0, 1, 2, 3]
    d["loop"] = {"start": 3, "stop": 4, "times": 3}                     # the last layer alone
    assert _spec(d)[1].layer_order() == [0, 1, 2, 3, 3, 3]
    d["loop"] = {"start": 2, "stop": 2, "times": 5}                     # an empty run
    assert _spec(d)[1].layer_order() == [0, 1, 2, 3]


def test_tensor_names_and_shapes_follow_the_layers():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_A)
    t = {s.name: tuple(s.shape) for s in DecoderModel(spec).tensor_specs()}
    assert t["embed"] == (211, 72) and t["head"] == (211, 72) and t["final.norm"] == (72,)
    # attention: biases on q and k, no value projection at all
    assert t["l0.mix.q"] == (144, 72) and t["l0.mix.q.b"] == (144,) and t["l0.mix.k"] == (48, 72) and t["l0.mix.k.b"] == (48,)
    assert t["l0.mix.o"] == (72, 144) and "l0.mix.v" not in t and "l0.mix.o.b" not in t
    assert all(t[f"l0.{n}"] == (72,) for n in ("norm1", "norm1b", "norm2", "norm2b"))
    assert t["l0.mlp.up"] == (88, 72) and t["l0.mlp.down"] == (72, 88) and "l0.mlp.up.b" not in t
    # latent attention: a latent wider than the heads; the rotated part rides on the down projection of keys/values
    assert t["l1.mix.dq"] == (28, 72) and t["l1.mix.dq.norm"] == (28,) and t["l1.mix.uq"] == (5 * 18, 28)
    assert t["l1.mix.dkv"] == (46, 72) and t["l1.mix.dkv.norm"] == (40,)
    assert t["l1.mix.uk"] == (60, 40) and t["l1.mix.uv"] == (100, 40) and t["l1.mix.o"] == (72, 100)
    assert "l1.norm2" not in t and "l1.norm2b" not in t and "l1.mlp.up" not in t     # no feed-forward: no norms around it
    # the recurrence: 6 heads on 2 query/key heads of 18, values of 10, five taps, inner sizes 7 and 12
    assert t["l2.mix.q"] == (36, 72) and t["l2.mix.k"] == (36, 72) and t["l2.mix.v"] == (60, 72)
    assert t["l2.mix.q.conv"] == (36, 5) and t["l2.mix.k.conv"] == (36, 5) and t["l2.mix.v.conv"] == (60, 5)
    assert t["l2.mix.b"] == (6, 72) and t["l2.mix.A_log"] == (6,) and t["l2.mix.dt_bias"] == (108,) and t["l2.mix.norm"] == (10,)
    assert t["l2.mix.a1"] == (7, 72) and t["l2.mix.a2"] == (108, 7) and t["l2.mix.g1"] == (12, 72) and t["l2.mix.g2"] == (60, 12)
    assert t["l2.mix.o"] == (72, 60) and "l2.mix.q.b" not in t
    # a looped layer's tensors exist once
    assert sum(1 for n in t if n.startswith("l1.")) == 10


def test_inner_sizes_of_the_low_rank_projections_may_be_left_to_the_stored_tensors():
    """Without decay_rank and gate_rank in the configuration the two halves' shapes are open in that dimension, and the
    mixer takes them from the tensors it is given."""
    from transformers_neuronx_b200.models.decoder import DecoderModel
    d = copy.deepcopy(CONFIG_C)
    for k in ("decay_rank", "gate_rank"):
        d["layers"][1]["mixer"].pop(k)
    _, _, spec = _spec(d)
    t = {s.name: tuple(s.shape) for s in DecoderModel(spec).tensor_specs()}
    assert t["l1.mix.a1"] == (-1, 100) and t["l1.mix.a2"] == (50, -1) and t["l1.mix.g1"] == (-1, 100) and t["l1.mix.g2"] == (30, -1)


def test_pages_and_state_of_every_run():
    from transformers_neuronx_b200.cache import FixedStateNeed, PagedKVNeed, group_needs
    from transformers_neuronx_b200.models.decoder import DecoderModel
    _, _, spec = _spec(CONFIG_A)
    needs = DecoderModel(spec).cache_needs()
    assert needs[0] == PagedKVNeed(2, 32, 21)                          # heads of 24 in rows of 32
    for run in (1, 3, 5):                                               # the latent (40) and the rotated part (6) in ONE head of 48
        assert needs[run] == PagedKVNeed(1, 48, 33)
    for run in (2, 4, 6):                                               # S per pass, and the convolutions' last four inputs
        assert needs[(run, 0)] == FixedStateNeed((6, 10, 18), "float32")
        assert needs[(run, 1)] == FixedStateNeed((4, 36 + 36 + 60), "activation")
    assert needs[7] == PagedKVNeed(1, 64, None)
    groups = group_needs(needs)
    assert [(g.window, g.cache_ids) for g in groups if g.paged] == [(21, [0]), (33, [1, 3, 5]), (None, [7])]
    _, _, spec_b = _spec(CONFIG_B)
    nb = DecoderModel(spec_b).cache_needs()
    assert nb[1] == PagedKVNeed(1, 64, 64) and nb[4] == PagedKVNeed(1, 128, None)
    assert nb[(5, 0)] == FixedStateNeed((4, 64, 32), "float32") and (5, 1) not in nb      # one tap keeps no inputs
    _, _, spec_c = _spec(CONFIG_C)
    assert DecoderModel(spec_c).cache_needs()[2] == PagedKVNeed(1, 32, 1)               # no rotated part: the latent alone


def test_pages_behind_a_window_go_back_to_the_pool():
    from transformers_neuronx_b200.cache import CacheManager, PagedKVNeed, group_needs
    cm = CacheManager(group_needs({0: PagedKVNeed(1, 16, 21)}), page_size=16, num_pages=4, max_slots=2)
    cm.add_request("a")
    cm.append("a", 36)                                   # positions 0..35; the next query (36) reads 16..36
    assert cm.release_behind_window("a") == 1 and cm.block_table("a")[0] == -1
    cm.append("a", 17)                                   # positions up to 52; the next query (53) reads 33..53
    assert cm.release_behind_window("a") == 1 and cm.block_table("a")[:2] == [-1, -1]
    cm.check()
    cm.free_request("a")
    assert cm.free_pages() == [4]


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].update(type="mamba"), "unknown layer type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "cannot share"),
    (lambda d: d["layers"][2]["mixer"].update(kv_heads=4), "cannot share"),
    (lambda d: d["layers"][0]["mixer"].update(vdim=32), "values are the keys"),
    (lambda d: d["layers"][0]["mixer"].update(rot={"dims": 26, "base": 9.0}), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"].update(rot={"dims": 7, "base": 9.0}), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].update(rot={"dims": 4, "base": 9.0}), "must equal rot_dim"),
    (lambda d: d["layers"][1]["mixer"].update(rot_dim=5), "rot_dim"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"].update(scale=0.0), "scale must be positive"),
    (lambda d: d["layers"][0]["mixer"].update(mask={"size": 0}), "size"),
    (lambda d: d["layers"][2]["mixer"].update(conv=0), "taps"),
    (lambda d: d["layers"][2]["mixer"].update(decay_rank=0), "decay_rank"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "kind must be 'dense'"),
    (lambda d: d["loop"].update(stop=5), "not a run"),
    (lambda d: d["loop"].update(start=3, stop=2), "not a run"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["embedding"].pop("scale"), "scale"),
    (lambda d: d.update(layers=[]), "at least one layer"),
])
def test_a_configuration_that_cannot_be_run_is_refused_by_name(edit, word):
    from transformers_neuronx_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(CONFIG_A)
    edit(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_sizes_the_kernels_do_not_take_are_refused_when_the_model_is_built():
    from transformers_neuronx_b200.models.decoder import DecoderModel
    d = copy.deepcopy(CONFIG_A)
    d["layers"][2]["mixer"].update(conv=9)
    with pytest.raises(ValueError, match="taps"):
        DecoderModel(_spec(d)[2])
    d = copy.deepcopy(CONFIG_A)
    d["layers"][1]["mixer"].update(kv_rank=770)
    with pytest.raises(ValueError, match="768 dims"):
        DecoderModel(_spec(d)[2])


def test_all_configurations_build():
    for d in CONFIGS.values():
        _, cfg, spec = _spec(d)
        assert len(spec.schedule) == len(cfg.layer_order())


# ---- the plain implementation's mechanisms against numbers worked out another way -------------------------
def test_plain_rotation_pairs():
    x = torch.arange(1, 9, dtype=torch.float64).view(1, 1, 8).repeat(2, 1, 1)
    y = TP.turn(x, [0, 3], 4, 100.0, True)                              # pairs (0, 1), (2, 3); dims 4.. pass unchanged
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, 0, 4:], x[1, 0, 4:])
    import numpy as np
    a0, a1 = 3.0, float(np.float32(3.0) * np.float32(100.0 ** -0.5))   # frequency and angle rounded to 32-bit
    want = [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
            3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1)]
    assert float((y[1, 0, :4] - torch.tensor(want, dtype=torch.float64)).abs().max()) < 1e-12
    z = TP.turn(x, [0, 3], 4, 100.0, False)                             # pairs (0, 2), (1, 3)
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)]
    assert float((z[1, 0, :4] - torch.tensor(want, dtype=torch.float64)).abs().max()) < 1e-12


def test_plain_window_counts_the_query_itself():
    w = TP.softmax_over_window(torch.zeros(6, 6, dtype=torch.float64), 3)
    assert w[5].tolist() == [0, 0, 0, 1 / 3, 1 / 3, 1 / 3] and w[1].tolist() == [0.5, 0.5, 0, 0, 0, 0]
    assert TP.softmax_over_window(torch.zeros(4, 4, dtype=torch.float64), 1)[3].tolist() == [0, 0, 0, 1]
    assert TP.softmax_over_window(torch.zeros(4, 4, dtype=torch.float64), None)[3].tolist() == [0.25] * 4


def test_plain_convolution_puts_the_last_column_on_the_current_token():
    u = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=torch.float64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)
    y = TP.short_conv_silu(u, w)
    pre = torch.tensor([1.0, 12.0, 123.0, 1230.0], dtype=torch.float64)
    assert float((y[:, 0] - pre * torch.sigmoid(pre)).abs().max()) < 1e-9


def test_plain_delta_rule_is_the_closed_form_where_there_is_one():
    """Orthonormal keys, beta 1, no decay: after the writes S^T k_i = v_i exactly (each write corrects its own key's
    read-out to its value); writing a key again with another value replaces the old one.  With a decay g on every row
    and beta 0 nothing is written and a first write fades as g^n."""
    d, dv = 4, 3
    k = torch.eye(d, dtype=torch.float64)[[0, 1, 2, 0]].view(4, 1, d)
    v = torch.tensor([[1.0, 2, 3], [4, 5, 6], [7, 8, 9], [-1, -2, -3]], dtype=torch.float64).view(4, 1, dv)
    q = torch.eye(d, dtype=torch.float64)[[0, 0, 1, 0]].view(4, 1, d)
    one, ones = torch.ones(4, 1, dtype=torch.float64), torch.ones(4, 1, d, dtype=torch.float64)
    o = TP.delta_recurrence(q, k, v, one, ones)
    assert o[:, 0].tolist() == [[1, 2, 3], [1, 2, 3], [4, 5, 6], [-1, -2, -3]]
    beta = torch.tensor([1.0, 0, 0, 0], dtype=torch.float64).view(4, 1)
    o = TP.delta_recurrence(q[[0, 0, 0, 0]], k, v, beta, ones * 0.5)
    assert float((o[:, 0, 0] - torch.tensor([0.5, 0.25, 0.125, 0.0625], dtype=torch.float64) * 2).abs().max()) < 1e-12
    # half a step: u = beta (v - S^T k) moves the read-out half of the way
    o = TP.delta_recurrence(q[[0, 0]], k[[0, 0]], v[[0, 0]], one[:2] * 0.5, ones[:2])
    assert o[:, 0].tolist() == [[0.5, 1.0, 1.5], [0.75, 1.5, 2.25]]
