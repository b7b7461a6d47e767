"""The Vozirax architecture as data: its configuration -> a ModelSpec naming parts, sizes, constants and tensors.

A decoder whose layers are listed one by one in the configuration.  A sinusoidal position vector is added to the
token's embedding.  Every layer runs its two sublayers side by side on the same stream, each behind a norm of its own
and with a learned scale per channel on its result:  x <- x + ls1 * mixer(norm1(x)) + ls2 * ff(norm2(x)),  RMS norms whose
stored weight w acts as 1 + w.  Two mixers:

  mamba2      a selective state-space recurrence (one decay per head and token) fed by projections of which x, B and C
              pass a short causal convolution and silu; gate, then a norm in equal parts of the inner width
  attention   differential attention: two softmax maps per head over the same values, subtracted; queries and keys
              normalised per head and map; a query temperature that grows with the logarithm of the position; an output
              gate per head; a layer may read an earlier layer's keys and values instead of projecting its own

The feed-forward is down(silu(gate h) * up h), or a mixture of experts down(relu(up h)^2) whose router adds a correction
to the sigmoid scores for the choice only and restricts the choice to the best groups of experts.  The head is a matrix
of its own behind a final norm; the logits are multiplied by a constant.

Tensor names: 'embed', 'final.norm', 'head', and for layer i the prefix 'l<i>.': 'norm1', 'norm2', 'ls1', 'ls2',
'mlp.gate|up|down' or 'mlp.router', 'mlp.correction', 'mlp.e<j>.up|down', and under 'mix.': in, conv, conv.b, dt_bias,
A_log, D, norm, o | q, k, v, q.norm, k.norm, lq1, lk1, lq2, lk2, g, o.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.vozirax_config import VoziraxConfig
from ..parts.spec import (DiffAttentionSpec, EmbeddingSpec, ExpertSpec, GatedFeedForwardSpec, HeadSpec, LayerSpec,
                          LinearSpec, ModelSpec, NormSpec, PositionSpec, RoutedFeedForwardSpec, ScheduleEntry, SSDSpec)

SINUSOID_BASE = 10000.0
RENORM_EPS = 1e-20             # the chosen experts' scores are divided by (their sum + 1e-20)
GROUP_TOP = 2                  # a group of experts is scored by the sum of its two largest choice scores


def _lin(name: str, n_in: int, n_out: int) -> LinearSpec:
    return LinearSpec(n_in, n_out, name, None)


def _ssd(p: str, W: int, m: dict, eps: float) -> SSDSpec:
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    return SSDSpec(kind="ssd", hidden=W, n_heads=H, v_dim=P, state=N, groups=G, norm_groups=m["norm_groups"],
                   conv_taps=int(m["conv"]), in_proj=_lin(p + ".in", W, 2 * inner + 2 * G * N + H),
                   out=_lin(p + ".o", inner, W), conv=p + ".conv", conv_bias=p + ".conv.b", dt_bias=p + ".dt_bias",
                   a_log=p + ".A_log", skip=p + ".D", out_norm=p + ".norm", norm_eps=eps, activation="silu")


def _attention(p: str, W: int, m: dict, eps: float) -> DiffAttentionSpec:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    own = m.get("kv_from") is None
    qt = m.get("q_temp")
    return DiffAttentionSpec(
        kind="diff_attention", hidden=W, n_heads=H, n_kv_heads=G, k_dim=d, v_dim=dv, scale=float(m["scale"]),
        diff=float(m["diff"]), out_mult=1.0 - float(m["diff"]), q=_lin(p + ".q", W, H * 2 * d),
        k=_lin(p + ".k", W, G * 2 * d) if own else None, v=_lin(p + ".v", W, G * dv) if own else None,
        gate=_lin(p + ".g", W, H), out=_lin(p + ".o", H * dv, W), q_norm=p + ".q.norm",
        k_norm=p + ".k.norm" if own else None, lambda_q1=p + ".lq1", lambda_k1=p + ".lk1", lambda_q2=p + ".lq2",
        lambda_k2=p + ".lk2", norm_eps=eps, temp_coef=float(qt["coef"]) if qt else 0.0,
        temp_every=int(qt["every"]) if qt else 0, kv_source=None if own else int(m["kv_from"]))


def _feed_forward(p: str, W: int, mlp: dict):
    if mlp["kind"] == "dense":
        F = mlp["ff"]
        return GatedFeedForwardSpec(kind="gated_dense", gate=_lin(p + ".gate", W, F), up=_lin(p + ".up", W, F),
                                    down=_lin(p + ".down", F, W), activation="silu")
    r, F = mlp["router"], mlp["expert"]["ff"]
    E = r["experts"]
    g = r.get("groups")
    return RoutedFeedForwardSpec(
        kind="routed_experts", hidden=W, ff=F, n_experts=E, top=r["top"], router=p + ".router",
        experts=tuple(ExpertSpec(None, f"{p}.e{j}.up", f"{p}.e{j}.down") for j in range(E)), scores="sigmoid",
        renormalize=True, weight_on_input=False, expert_form="relu2", correction=p + ".correction",
        n_groups=g["count"] if g else 1, keep_groups=g["keep"] if g else 1, group_top=GROUP_TOP, renorm_eps=RENORM_EPS,
        weight_scale=float(r["scale"]) if r.get("scale") is not None else 1.0)


def build_spec(cfg: VoziraxConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: NormSpec("rms_norm", W, eps, weight=name, weight_offset=1.0)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        mixer = (_ssd if layer["type"] == "mamba2" else _attention)(p + ".mix", W, layer["mixer"], eps)
        ff = n2 = s2 = None
        if layer.get("mlp") is not None:
            ff, n2, s2 = _feed_forward(p + ".mlp", W, layer["mlp"]), norm(p + ".norm2"), p + ".ls2"
        layers.append(LayerSpec(block="parallel_residual", norm1=norm(p + ".norm1"), mixer=mixer, norm2=n2,
                                feed_forward=ff, scale1=p + ".ls1", scale2=s2))
    # a layer's cache number is its index: a layer that reads another's keys and values names that layer
    return ModelSpec(hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
                     embedding=EmbeddingSpec(table="embed", vocab=cfg.vocab, dim=W,
                                             position=PositionSpec(kind="sinusoidal", dim=W, base=SINUSOID_BASE)),
                     layers=tuple(layers), schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
                     head=HeadSpec(weight="head", vocab=cfg.vocab, dim=W, final_norm=norm("final.norm"),
                                   logit_scale=float(cfg.logit_scale)))


register_architecture(Architecture(name="Vozirax", model_type="vozirax", config_class=VoziraxConfig,
                                   build_spec=build_spec))
