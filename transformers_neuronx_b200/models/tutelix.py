"""The Tutelix architecture as data: its configuration -> a ModelSpec naming parts, sizes, constants and tensors.

A decoder whose layers are listed one by one in the configuration.  The embedding's rows are multiplied by a constant.
Every sublayer has a norm before it and one behind it: x <- x + norm1b(mixer(norm1(x))), then
x <- x + norm2b(ff(norm2(x))), RMS norms whose stored weight w acts as 1 + w.  A run of layers may be looped: it is
walked several times in a row with the same weights, every pass with a cache of its own, which here is a schedule that
names those layers several times with different cache numbers.  Three mixers:

  attention         grouped key/value heads, q and k with biases, rotated in halves over the first rot.dims dims; the
                    values are the keys as projected (no value projection); sliding window
  latent_attention  queries through a normalised latent; keys and values expanded per head from one normalised latent,
                    plus one rotated key part (interleaved pairs) shared by all heads; sliding window; the pages hold
                    the latent and the rotated part only
  channel_delta     a recurrence with a decay per head and key channel and an error-correcting write, fed by
                    projections that pass a short causal convolution and silu; unit-norm q and k

The feed-forward is down(gelu(up h)) with the exact (erf) gelu and no biases.  The head is a matrix of its own behind
a final norm of the same kind.

Tensor names: 'embed', 'final.norm', 'head', and for layer i the prefix 'l<i>.': 'norm1', 'norm1b', 'norm2', 'norm2b',
'mlp.up|down', and under 'mix.': q, k (+ '.b'), o | dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o | q, k, v (+ '.conv'),
b, a1, a2, A_log, dt_bias, g1, g2, norm, o.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.tutelix_config import TutelixConfig
from ..parts.spec import (DeltaRuleSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LatentAttentionSpec, LayerSpec,
                          LinearSpec, ModelSpec, NormSpec, RotaryAttentionSpec, RotarySpec, ScheduleEntry)

UNIT_NORM_EPS = 1e-6           # q and k of the recurrence: x / sqrt(sum(x^2) + 1e-6)


def _lin(name: str, n_in: int, n_out: int, bias: bool = False) -> LinearSpec:
    return LinearSpec(n_in, n_out, name, name + ".b" if bias else None)


def _window(m: dict):
    return m["mask"]["size"] if m.get("mask") is not None else None


def _rot(m: dict, interleaved: bool):
    r = m.get("rot")
    if r is None or not r.get("dims"):
        return None
    return RotarySpec(int(r["dims"]), float(r["base"]), interleaved=interleaved)


def _attention(p: str, W: int, m: dict) -> RotaryAttentionSpec:
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    return RotaryAttentionSpec(kind="rotary_attention", hidden=W, n_heads=H, n_kv_heads=G, k_dim=d, v_dim=d,
                               scale=float(m["scale"]), q=_lin(p + ".q", W, H * d, True), k=_lin(p + ".k", W, G * d, True),
                               v=None, out=_lin(p + ".o", H * d, W), rotary=_rot(m, False), window=_window(m))


def _latent(p: str, W: int, m: dict, eps: float) -> LatentAttentionSpec:
    H, d, dr, dv, rq, rkv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
    return LatentAttentionSpec(kind="latent_attention", hidden=W, n_heads=H, k_dim=d, rot_dim=dr, v_dim=dv, q_rank=rq,
                               kv_rank=rkv, scale=float(m["scale"]), dq=_lin(p + ".dq", W, rq),
                               uq=_lin(p + ".uq", rq, H * (d + dr)), dkv=_lin(p + ".dkv", W, rkv + dr), uk=p + ".uk",
                               uv=p + ".uv", out=_lin(p + ".o", H * dv, W), q_norm=p + ".dq.norm",
                               kv_norm=p + ".dkv.norm", norm_eps=eps, rotary=_rot(m, True), window=_window(m))


def _delta(p: str, W: int, m: dict, eps: float) -> DeltaRuleSpec:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    ra, rg = int(m.get("decay_rank") or -1), int(m.get("gate_rank") or -1)     # -1: the stored tensors' inner size
    return DeltaRuleSpec(kind="delta_rule", hidden=W, n_heads=H, n_kv_heads=G, k_dim=d, v_dim=dv, conv_taps=int(m["conv"]),
                         q=_lin(p + ".q", W, G * d), k=_lin(p + ".k", W, G * d), v=_lin(p + ".v", W, H * dv),
                         beta=_lin(p + ".b", W, H), a1=_lin(p + ".a1", W, ra), a2=_lin(p + ".a2", ra, H * d),
                         g1=_lin(p + ".g1", W, rg), g2=_lin(p + ".g2", rg, H * dv), out=_lin(p + ".o", H * dv, W),
                         q_conv=p + ".q.conv", k_conv=p + ".k.conv", v_conv=p + ".v.conv", a_log=p + ".A_log",
                         dt_bias=p + ".dt_bias", out_norm=p + ".norm", norm_eps=eps, unit_eps=UNIT_NORM_EPS,
                         q_scale=float(d) ** -0.5, conv_activation="silu")


_MIXERS = {"attention": lambda p, W, m, eps: _attention(p, W, m), "latent_attention": _latent, "channel_delta": _delta}


def build_spec(cfg: TutelixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: NormSpec("rms_norm", W, eps, weight=name, weight_offset=1.0)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        ff = n2 = n2b = None
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            ff = DenseFeedForwardSpec(kind="dense", fc1=_lin(p + ".mlp.up", W, F), fc2=_lin(p + ".mlp.down", F, W),
                                      activation="gelu")
            n2, n2b = norm(p + ".norm2"), norm(p + ".norm2b")
        layers.append(LayerSpec(block="sandwich_norm", norm1=norm(p + ".norm1"),
                                mixer=_MIXERS[layer["type"]](p + ".mix", W, layer["mixer"], eps), norm2=n2,
                                feed_forward=ff, norm1_post=norm(p + ".norm1b"), norm2_post=n2b))
    # every run of a layer is a schedule entry with a cache of its own: a looped layer keeps one past per pass
    schedule = tuple(ScheduleEntry(layer, run) for run, layer in enumerate(cfg.layer_order()))
    return ModelSpec(hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
                     embedding=EmbeddingSpec(table="embed", vocab=cfg.vocab, dim=W, scale=float(cfg.embedding_scale)),
                     layers=tuple(layers), schedule=schedule,
                     head=HeadSpec(weight="head", vocab=cfg.vocab, dim=W, final_norm=norm("final.norm")))


register_architecture(Architecture(name="Tutelix", model_type="tutelix", config_class=TutelixConfig,
                                   build_spec=build_spec))
