"""The Vozirax decoder on the GPU against the plain implementation (tests/plain/vozirax_plain.py): every mechanism's
kernel alone, then whole models through the replay program's function (whole prompts, token by token, portions down
to two tokens, mixed batches with pages and slots used again), a far key made to stand out, decays that remember and
forget, long decoding, and greedy generation through the engine's own entry point and scheduler."""
import copy
import math
from types import SimpleNamespace

import pytest
import torch

from helpers import run_trace_inprocess
from plain import vozirax_plain as ZP
from vononex_helpers import TOLERANCE
from vozirax_helpers import (CONFIG_A, CONFIGS, VoziraxModel, attn, compare, cut_steps, dense, layer, mixed_steps, moe, ssm,
                             whole_steps)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
_models = {}


def _model(name, seed=5):
    if (name, seed) not in _models:
        _models[(name, seed)] = VoziraxModel(CONFIGS[name], seed=seed)
    return _models[(name, seed)]


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err <= tol, err


def _ctx(cuts, pad_rows=1):
    """cuts: per request (slot, first position, rows) -> the index arrays of a step, as the step function packs them,
    with a padded row and a padded request behind them."""
    req, pos, q_start, q_len, slots, row = [], [], [], [], [], 0
    for r, (slot, first, n) in enumerate(cuts):
        req += [r] * n
        pos += list(range(first, first + n))
        q_start.append(row); q_len.append(n); slots.append(slot)
        row += n
    return SimpleNamespace(token_request=_i32(req + [-1] * pad_rows), positions=_i32(pos + [0] * pad_rows),
                           q_start=_i32(q_start + [0]), q_len=_i32(q_len + [0]), state_slots=_i32(slots + [-1]),
                           decode_only=all(n == 1 for n in q_len))


# ---- each mechanism's kernel alone -----------------------------------------------------------------
@pytest.mark.parametrize("W", [72, 51, 2048])
def test_sinusoidal_positions_in_the_embedding_kernel(W):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    table = torch.randn(30, W, generator=g)
    ids, pos = [3, 29, 0, 7], [0, 1, 977, 40000]
    freq = torch.pow(torch.tensor(10000.0, dtype=F64), -2.0 * torch.arange((W + 1) // 2, dtype=F64) / W).float()
    x = torch.empty(4, W, device=DEV)
    ops.embed(table.to(DEV), None, _i32(ids), None, _i32(pos), 0, x, None, sin_freq=freq.to(DEV))
    want = table[ids].double() + ZP.sinusoid(pos, W)
    assert float((x.cpu().double() - want).abs().max()) <= 2e-6         # sine and cosine of a 32-bit angle, in 32-bit


@pytest.mark.parametrize("W, dtype", [(72, torch.float32), (50, torch.bfloat16), (2048, torch.bfloat16)])
def test_two_norms_of_one_row_and_two_scaled_results_into_the_stream(W, dtype):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    x = torch.randn(9, W, generator=g) * 3
    w1, w2 = torch.randn(W, generator=g) * 0.3, torch.randn(W, generator=g) * 0.3
    o1, o2 = torch.empty(9, W, device=DEV, dtype=dtype), torch.empty(9, W, device=DEV, dtype=dtype)
    ops.rms_norm_pair(x.to(DEV), w1.to(DEV), 1.0, 1e-4, o1, w2.to(DEV), 1.0, 1e-2, o2)
    tol = 1e-6 if dtype == torch.float32 else 5e-3
    _close(o1, ZP.rms(x.double(), 1e-4, 1.0 + w1.double()), tol)
    _close(o2, ZP.rms(x.double(), 1e-2, 1.0 + w2.double()), tol)
    only = torch.empty(9, W, device=DEV, dtype=dtype)
    ops.rms_norm_pair(x.to(DEV), None, 0.0, 1e-4, only)
    _close(only, ZP.rms(x.double(), 1e-4), tol)
    a, b = torch.randn(9, W, generator=g), torch.randn(9, W, generator=g)
    xs = x.to(DEV)
    ops.scaled_residual_add(xs, a.to(DEV), w1.to(DEV), b.to(DEV), w2.to(DEV))
    _close(xs, x.double() + a.double() * w1.double() + b.double() * w2.double(), 1e-6)
    ops.scaled_residual_add(xs, a.to(DEV))
    new = x.double() + a.double() * (w1.double() + 1.0) + b.double() * w2.double()
    _close(xs, new, 1e-6)
    # the kernel that closes a layer also forms the two norms of the layer that follows
    ops.scaled_residual_add(xs, b.to(DEV), w2.to(DEV), a.to(DEV), None, then=(w2.to(DEV), 1.0, 1e-3, o1, w1.to(DEV), 0.0, 1e-5, o2))
    new = new + b.double() * w2.double() + a.double()
    _close(xs, new, 1e-6)
    _close(o1, ZP.rms(new, 1e-3, 1.0 + w2.double()), tol)
    _close(o2, ZP.rms(new, 1e-5, w1.double()), tol)
    ops.scaled_residual_add(xs, a.to(DEV), then=(None, 0.0, 1e-5, only, None, 0.0, 0.0, None))
    _close(only, ZP.rms(new + a.double(), 1e-5), tol)


def _plain_maps(u, H, G, dk, dv, qn, kn, eps, temp, positions):
    """Queries, keys, values of differential attention from a row of projections, as the plain implementation forms them."""
    T = u.shape[0]
    q = ZP.rms(u[:, :2 * H * dk].double().reshape(T, H, 2, dk), eps, qn.double())
    k = ZP.rms(u[:, 2 * H * dk:2 * (H + G) * dk].double().reshape(T, G, 2, dk), eps, kn.double())
    v = u[:, 2 * (H + G) * dk:2 * (H + G) * dk + G * dv].double().reshape(T, G, dv)
    if temp is not None:
        for i, p in enumerate(positions):
            q[i] = q[i] * (1.0 + temp[0] * ZP.f32(math.log(float((p + 1) // temp[1] + 1))))
    return q, k, v


@pytest.mark.parametrize("H, G, dk, dv, temp, dtype", [
    (6, 2, 12, 40, (0.8, 7), torch.float32), (4, 2, 32, 80, (0.25, 96), torch.float32), (1, 1, 50, 30, None, torch.float32),
    (5, 5, 8, 20, (2.0, 1), torch.float32), (4, 2, 64, 128, (0.5, 3), torch.bfloat16)])
def test_queries_keys_and_values_of_the_two_maps(H, G, dk, dv, temp, dtype):
    """Norm per head and map, the temperature at positions around multiples of its period, the layout of one call of
    the attention kernels (a key row holds both maps, a query row its own map among zeros), a padded row left alone,
    and a reader that has queries only."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    D = -(-max(2 * dk, dv) // 16) * 16
    every = temp[1] if temp else 0
    pos = [0, 1, max(every - 2, 0), max(every - 1, 0), every, 2 * every + 5, 1000, 4095]
    T, width, col0 = len(pos), 2 * (H + G) * dk + G * dv + H, 3
    u = (torch.randn(T, width, generator=g) * 2).to(dtype)
    qn, kn = torch.randn(dk, generator=g), torch.randn(dk, generator=g)
    q, k, v = _plain_maps(u.float(), H, G, dk, dv, qn, kn, 1e-5, temp, pos)
    proj = torch.zeros(T + 1, col0 + width, dtype=dtype)
    proj[:T, col0:] = u
    ctx = SimpleNamespace(token_request=_i32([0] * T + [-1]), positions=_i32(pos + [0]))
    outs = [torch.full((T + 1, n), 9.0, device=DEV, dtype=dtype) for n in (2 * H * D, G * D, G * D)]
    ops.diff_qkv_prep(proj.to(DEV), col0, ctx.token_request, ctx.positions, qn.to(DEV), kn.to(DEV), 1e-5,
                      temp[0] if temp else 0.0, every, *outs, H, G, dk, dv, D)
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    qo, ko, vo = (o.float().cpu() for o in outs)
    for o in (qo, ko, vo):
        assert float((o[T] - 9.0).abs().max()) == 0.0
    qo = qo[:T].reshape(T, H, 2, D)
    for mp in range(2):
        _close(qo[:, :, mp, mp * dk:(mp + 1) * dk], q[:, :, mp], tol)
        rest = torch.cat([qo[:, :, mp, :mp * dk], qo[:, :, mp, (mp + 1) * dk:]], -1)
        assert float(rest.abs().max()) == 0.0
    ko = ko[:T].reshape(T, G, D)
    _close(ko[..., :2 * dk], k.reshape(T, G, 2 * dk), tol)
    vo = vo[:T].reshape(T, G, D)
    _close(vo[..., :dv], v, tol)
    assert float(ko[..., 2 * dk:].abs().max() if D > 2 * dk else 0.0) == 0.0 and float(vo[..., dv:].abs().max() if D > dv else 0.0) == 0.0
    only_q = torch.empty(T + 1, 2 * H * D, device=DEV, dtype=dtype)
    ops.diff_qkv_prep(proj.to(DEV), col0, ctx.token_request, ctx.positions, qn.to(DEV), None, 1e-5,
                      temp[0] if temp else 0.0, every, only_q, None, None, H, 0, dk, dv, D)
    assert torch.equal(only_q[:T].float().cpu().reshape(T, H, 2, D), qo)


@pytest.mark.parametrize("H, dv, D, dtype", [(6, 40, 48, torch.float32), (4, 128, 128, torch.bfloat16), (1, 30, 112, torch.float32)])
def test_the_two_maps_subtracted_normalised_and_gated(H, dv, D, dtype):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    T, lam, mult = 7, 0.37, 0.55
    att = torch.randn(T + 1, 2 * H * D, generator=g).to(dtype)
    gate = torch.randn(T + 1, H + 3, generator=g).to(dtype)
    a = att[:T].double().reshape(T, H, 2, D)[..., :dv]
    want = ZP.rms(a[:, :, 0] - lam * a[:, :, 1], 1e-5) * mult * torch.sigmoid(gate[:T, 2:2 + H].double())[..., None]
    out = torch.full((T + 1, H * dv + 8), 9.0, device=DEV, dtype=dtype)
    ops.diff_combine(att.to(DEV), gate.to(DEV)[:, 2:2 + H], _i32([0] * T + [-1]), lam, 1e-5, mult, 1.0, out[:, 8:], H, dv, D)
    _close(out[:T, 8:], want.reshape(T, H * dv), 2e-6 if dtype == torch.float32 else 5e-3)
    assert float((out[T].float() - 9.0).abs().max()) == 0.0 and float((out[:, :8].float() - 9.0).abs().max()) == 0.0


def _plain_ssd_inputs(u, w, b, a_log, dt_bias, H, P, G, N, taps):
    """x, B, C, dt and decay of a whole sequence from the projections' columns [x | B | C | dt]."""
    inner, gn = H * P, G * N
    xbc = ZP.silu(ZP.causal_conv(u[:, :inner + 2 * gn].double(), w.double(), b.double(), taps))
    dt = torch.nn.functional.softplus(u[:, inner + 2 * gn:].double() + dt_bias.double(), threshold=1e9)
    return xbc[:, :inner], xbc[:, inner:inner + gn], xbc[:, inner + gn:], dt, torch.exp(-torch.exp(a_log.double()) * dt)


CUTS = [(5, 1), (1, 2), (2, 0), (1, 1), (8, 17), (1, 1), (0, 1), (23, 18)]       # rows of two requests, step by step


@pytest.mark.parametrize("H, P, G, N, taps, dtype", [
    (6, 10, 3, 18, 5, torch.float32), (4, 64, 2, 128, 4, torch.float32), (1, 50, 1, 30, 1, torch.float32),
    (5, 20, 5, 12, 8, torch.float32), (8, 32, 1, 64, 3, torch.bfloat16), (4, 32, 1, 40, 4, torch.float32)])
def test_the_state_space_recurrence_across_cuts_and_slots(H, P, G, N, taps, dtype):
    """Two requests cut into unequal steps side by side (single tokens, pairs, a padded row, a request left out of a step):
    convolution with bias and silu, step sizes and decays, the recurrence with its decay per token and the keys and
    queries that groups of heads share, all against the plain recurrence over the whole sequences; the slots hold the
    last taps - 1 projected values afterwards, a slot nobody uses stays as it is, and a third request that takes a freed
    slot (zeroed, as the cache manager does on admission) must not see what was there."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    T, inner, gn = 41, H * P, G * N
    C, keep = inner + 2 * gn, taps - 1
    w, b = torch.randn(C, taps, generator=g) * 0.5, torch.randn(C, generator=g) * 0.3
    a_log, dt_bias = torch.randn(H, generator=g), torch.randn(H, generator=g)
    a_log[0] = -9.0                                                    # one head that forgets almost nothing
    state = torch.zeros(4, H, P, N, device=DEV)
    conv = torch.zeros(4, keep, C, device=DEV, dtype=dtype) if keep else None
    state[1].fill_(7.0)

    def run(seqs, slots, cuts_list):
        got = [torch.zeros(T, inner) for _ in seqs]
        at = [0] * len(seqs)
        for ns in cuts_list:
            reqs = [r for r, n in enumerate(ns) if n]
            cuts = [(slots[r], at[r], ns[r]) for r in reqs]
            ctx = _ctx(cuts)
            n_rows = sum(c[2] for c in cuts)
            proj = torch.zeros(n_rows + 1, 2 + inner + C + H, dtype=dtype)
            proj[:n_rows, 2 + inner:] = torch.cat([seqs[r][at[r]:at[r] + c[2]] for r, c in zip(reqs, cuts)])
            f = lambda n: torch.full((n_rows + 1, n), 9.0, device=DEV)
            x, bb, cc, dt, dec, y = f(inner), f(gn), f(gn), f(H), f(H), f(inner)
            ops.ssd_prep(proj.to(DEV), 2, w.t().contiguous().to(DEV), b.to(DEV), taps, conv, ctx, a_log.to(DEV),
                         dt_bias.to(DEV), "silu", x, bb, cc, dt, dec, H, P, G, N)
            ops.retention_scan(cc, bb, x, None, state, ctx.q_start, ctx.q_len, ctx.state_slots, y, H, N, P,
                               most_tokens=1 if ctx.decode_only else n_rows, decay_tok=dec, kscale_tok=dt, qk_heads=G)
            assert float((x[n_rows] - 9.0).abs().max()) == 0.0 and float((y[n_rows] - 9.0).abs().max()) == 0.0
            row = 0
            for r, (_, first, n) in zip(reqs, cuts):
                got[r][first:first + n] = y[row:row + n].cpu()
                row += n; at[r] += n
        return got

    def plain(u):
        x, bb, cc, dt, dec = _plain_ssd_inputs(u.float(), w, b, a_log, dt_bias, H, P, G, N, taps)
        y = torch.zeros(T, H, P, dtype=F64)
        for h in range(H):
            gi, S = h // (H // G), torch.zeros(N, P, dtype=F64)
            for t in range(T):
                S = dec[t, h] * S + dt[t, h] * torch.outer(bb[t, gi * N:(gi + 1) * N], x[t, h * P:(h + 1) * P])
                y[t, h] = S.T @ cc[t, gi * N:(gi + 1) * N]
        return y.reshape(T, inner)

    seqs = [(torch.randn(T, C + H, generator=g)).to(dtype) for _ in range(3)]
    got = run(seqs[:2], [2, 0], CUTS)
    tol = 2e-5
    for r in range(2):
        _close(got[r], plain(seqs[r]), tol)
    assert float((state[1] - 7.0).abs().max()) == 0.0
    if keep:
        _close(conv[2].float(), seqs[0][T - keep:, :C].double(), 0.0)   # the request's last projected values, oldest first
    state[2].zero_()
    if keep:
        conv[2].zero_()
    got = run([seqs[2]], [2], [(3,), (1,), (1,), (30,), (2,), (1,), (1,), (1,), (1,)])
    _close(got[0], plain(seqs[2]), tol)


@pytest.mark.parametrize("lanes, stage", [(0, 0), (0, 8), (0, 2), (16, 0), (16, 4)])
def test_the_scan_does_not_depend_on_how_its_tokens_are_staged(lanes, stage):
    """Stages of 32, 8 or 2 tokens and a column's rows over 8 or 16 lanes (the kernel chooses by the number of blocks; a
    hook imposes them): the state is the same bit for bit, the outputs to the order of a sum."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    H, P, G, N, T = 4, 32, 2, 128, 75
    c, b = torch.randn(T, G * N, generator=g).to(DEV), torch.randn(T, G * N, generator=g).to(DEV)
    x, dt = torch.randn(T, H * P, generator=g).to(DEV), torch.rand(T, H, generator=g).to(DEV)
    dec = (torch.rand(T, H, generator=g) * 0.3 + 0.7).to(DEV)
    ctx = _ctx([(1, 0, T)], pad_rows=0)

    def run():
        state, y = torch.zeros(2, H, P, N, device=DEV), torch.empty(T, H * P, device=DEV)
        ops.retention_scan(c, b, x, None, state, ctx.q_start, ctx.q_len, ctx.state_slots, y, H, N, P, most_tokens=T,
                           decay_tok=dec, kscale_tok=dt, qk_heads=G)
        return state, y
    want_state, want_y = run()
    ops.retention_scan_force(lanes, stage)
    try:
        state, y = run()
    finally:
        ops.retention_scan_force(0, 0)
    assert torch.equal(state, want_state)
    _close(y, want_y.cpu(), 0.0 if lanes == 0 else 2e-6)


@pytest.mark.parametrize("inner, P, parts, dtype", [(60, 10, 3, torch.float32), (256, 64, 1, torch.bfloat16), (256, 32, 8, torch.float32),
                                                    (50, 50, 5, torch.float32)])
def test_the_gate_comes_before_the_norm_in_parts(inner, P, parts, dtype):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    T = 6
    y, x = torch.randn(T + 1, inner, generator=g), torch.randn(T + 1, inner, generator=g)
    z = torch.randn(T + 1, inner + 5, generator=g).to(dtype)
    skip, w = torch.randn(inner // P, generator=g), torch.randn(inner, generator=g)
    v = (y[:T].double() + skip.double().repeat_interleave(P) * x[:T].double()) * ZP.silu(z[:T, 5:].double())
    want = ZP.rms(v.reshape(T, parts, inner // parts), 1e-5).reshape(T, inner) * w.double()
    out = torch.full((T + 1, inner), 9.0, device=DEV, dtype=dtype)
    ops.ssd_gate_norm(y.to(DEV), x.to(DEV), skip.to(DEV), z.to(DEV)[:, 5:], _i32([0] * T + [-1]), w.to(DEV), 1e-5, "silu", out,
                      P, parts)
    _close(out[:T], want, 2e-6 if dtype == torch.float32 else 5e-3)
    assert float((out[T].float() - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("E, top, groups, W", [(8, 3, (4, 3), 64), (6, 3, (3, 2), 72), (12, 4, (2, 1), 40), (5, 1, None, 33),
                                               (1, 1, None, 16), (16, 6, (16, 7), 48), (64, 8, (8, 4), 128)])
def test_routing_with_a_correction_and_groups(E, top, groups, W):
    """Choice scores are sigmoid + correction, also where they are negative (an expert of a dropped group must not win
    against them); a group counts by its two largest; the weights are the uncorrected scores, normalised and scaled."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(7)
    N = 40
    h = torch.randn(N, W, generator=g)
    router = torch.randn(E, W, generator=g) * 0.4
    corr = torch.randn(E, generator=g) * 0.5 - 1.2                      # most choice scores are negative
    r = {"experts": E, "top": top, "scale": 1.75}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    want = ZP.route(h.double(), {"router": router.double(), "correction": corr.double()}, "", r)
    ids = torch.empty(N + 1, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(N + 1, top, device=DEV)
    hp = torch.cat([h, torch.zeros(1, W)]).to(DEV)
    ops.moe_route(hp, router.to(DEV), _i32([0] * N + [-1]), ids, wts, top, renormalize=True, correction=corr.to(DEV),
                  n_groups=groups[0] if groups else 1, keep_groups=groups[1] if groups else 1, group_top=2, renorm_eps=1e-20,
                  weight_scale=1.75)
    assert ids[N].tolist() == [-1] * top
    for n, (e_want, w_want) in enumerate(want):
        assert ids[n].tolist() == e_want, (n, ids[n].tolist(), e_want)
        _close(wts[n], w_want, 2e-6)


@pytest.mark.parametrize("N, E, top, W, F, dtype", [(5, 4, 2, 72, 20, torch.float32), (40, 8, 2, 256, 96, torch.bfloat16),
                                                   (300, 8, 3, 128, 192, torch.bfloat16), (3, 5, 5, 50, 36, torch.float32)])
def test_experts_without_a_gate(N, E, top, W, F, dtype):
    """down(relu(up x)^2) with the weight on the output, in the form that streams the matrices and (16-bit) in the
    grouped tensor-core form."""
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(8)
    h = torch.randn(N, W, generator=g).to(dtype)
    up, down = (torch.randn(E, F, W, generator=g) * 0.2).to(dtype), (torch.randn(E, W, F, generator=g) * 0.2).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(N)]).to(torch.int32)
    wts = torch.rand(N, top, generator=g) + 0.1
    want = torch.zeros(N, W, dtype=F64)
    for n in range(N):
        for e, wt in zip(ids[n].tolist(), wts[n].tolist()):
            want[n] += wt * (down[e].double() @ torch.relu(up[e].double() @ h[n].double()) ** 2)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    out = torch.full((N, W), 1.0, device=DEV)
    y = torch.empty(N * top, F, device=DEV, dtype=dtype)
    ops.moe_experts(h.to(DEV), up.to(DEV), down.to(DEV), ids.to(DEV), wts.to(DEV), y, out, math.inf, -math.inf, math.inf, 1.0,
                    0.0, weight_on_input=False, accumulate=True, form="relu2")
    _close(out, want + 1.0, tol)
    if dtype != torch.float32:
        ctx = StepContext(torch.device(DEV), dtype)
        out = torch.empty(N, W, device=DEV)
        ops.moe_grouped(ctx, h.to(DEV), up.to(DEV), down.to(DEV), ids.to(DEV), wts.to(DEV), out, math.inf, -math.inf, math.inf,
                        1.0, 0.0, weight_on_input=False, accumulate=False, form="relu2")
        _close(out, want, tol)


# ---- whole models through the replay program's function -------------------------------------------
LENGTHS = {"A": [1, 2, 17, 45, 130], "B": [3, 140, 300], "C": [3, 70, 41]}
# The rows' median error in bfloat16: A is narrow (72) and routes 3 of 6 experts, so a rounding now and then picks another
# expert for a token; B and C stay under the bound of the other designs' tests.  The 32-bit engine holds every row to 3e-5.
BF16_MEDIAN = {"A": 7e-2, "B": TOLERANCE["bfloat16"], "C": TOLERANCE["bfloat16"]}


def _tol(name, dtype):
    return BF16_MEDIAN[name] if dtype == "bfloat16" else None


def _requests(m, lengths, seed=100):
    return {f"r{i}": m.random_ids(n, seed=seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_stream_after_every_layer(name):
    """The residual stream after each layer against the plain one: the first wrong layer names the mechanism."""
    from transformers_neuronx_b200.engine.loading import load_model
    from transformers_neuronx_b200.engine.step import StepEntry, StepRunner
    m = _model(name)
    ids = m.random_ids(70, 11)
    want = m.plain_hidden(ids)                                          # [layers, T, width]
    model, _ = load_model(m.folder, "float32", verbose=False)
    runner = StepRunner(model, page_size=16, num_pages=8, max_slots=2, max_model_len=128, use_cuda_graphs=False)
    runner.add_request("a")
    with model.tap_hidden_states() as taps:
        runner.step([StepEntry("a", ids, [len(ids) - 1])])
        torch.cuda.synchronize()
        for run in range(want.shape[0]):
            _close(taps[f"entry{run}"][:len(ids)], want[run], 2e-5)
    runner.finish("a")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts(name, dtype):
    m = _model(name)
    reqs = _requests(m, LENGTHS[name])
    steps = whole_steps(reqs)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype, tol=_tol(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_prefix_then_token_by_token(name, dtype):
    """Decoding through the pages and the states: the last 70 tokens one by one (the temperature's period passes several
    times among them), the decode steps replayed from a captured graph."""
    m = _model(name)
    reqs = _requests(m, [n for n in LENGTHS[name] if n > 71])
    steps = cut_steps(reqs, [1000], tail=70)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype, tol=_tol(name, dtype))


@pytest.mark.parametrize("name", ["A", "C"])
def test_from_the_first_token_on_one_by_one(name):
    """The first positions: zeros before the start of the convolution, a state that starts at zero, a softmax over one key."""
    m = _model(name)
    reqs = _requests(m, [50])
    steps = cut_steps(reqs, [1])
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_changing_size_down_to_two_tokens(name, dtype):
    """Portions shorter than the convolution (2 and 3 tokens under 5 taps), portions that end one before, at and one
    behind a page's border, and a long one."""
    m = _model(name)
    reqs = _requests(m, LENGTHS[name][-2:])
    steps = cut_steps(reqs, [2, 33, 3, 16, 2, 17, 64, 5, 15, 130], tail=3)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype, tol=_tol(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype):
    """More requests than the replay program has slots: a finished request's slot (recurrent state and the convolution's
    last inputs) and its pages go to the next request, and the pool holds no more than the live requests need."""
    m = _model(name)
    lengths = [90, 7, 33, 150, 12, 64, 5, 49, 2, 120, 31] if name == "A" else [150, 20, 70, 9, 200, 40, 33, 129, 18]
    reqs = _requests(m, lengths, seed=300)
    steps = mixed_steps(reqs, [9, 2, 31, 16, 5, 64, 3])
    most = sorted(-(-n // 64) * 64 for n in lengths)[-4:]
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, sum(most)), dtype, tol=_tol(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_no_fast_path_takes(dtype):
    m = _model("C")
    reqs = _requests(m, LENGTHS["C"], seed=600)
    for steps in (whole_steps(reqs), mixed_steps(reqs, [7, 2, 19, 33], decode_tail=12)):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 4), dtype)


def test_logits_do_not_depend_on_the_cut_or_the_batch_beyond_rounding():
    m = _model("A")
    reqs = _requests(m, [130, 45], seed=500)
    runs = []
    for steps in (whole_steps(reqs), cut_steps(reqs, [2, 16, 17, 1, 31]), mixed_steps(reqs, [15, 2, 40], decode_tail=20)):
        res = run_trace_inprocess(m.folder, "float32", steps, 64 * 4)
        at, out = {r: 0 for r in reqs}, {}
        for s in steps:
            row = 0
            for e in s["entries"]:
                for w in e["want"]:
                    out[(e["id"], at[e["id"]] + w)] = torch.from_numpy(res[s["step"]][row].copy()); row += 1
                at[e["id"]] += len(e["tokens"])
        runs.append(out)
    for other in runs[1:]:
        for key, lg in other.items():
            assert float((lg - runs[0][key]).abs().max()) <= 2e-5 * float(runs[0][key].abs().max()), key


# ---- a key far away, decays that remember and forget -----------------------------------------------
def _one(kind, mixer, mlp=None, width=64, vocab=97):
    return {"architecture": "Vozirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 1.5, "init_std": 0.3,
            "layers": [layer(kind, mixer, mlp)]}


def _edge_steps(reqs):
    return (whole_steps(reqs), cut_steps(reqs, [48, 47, 2, 49, 16, 15, 1, 64], tail=57),
            mixed_steps(reqs, [31, 2, 48, 17], decode_tail=51))


def test_a_sharp_softmax_finds_the_same_key_among_hundreds():
    """A scale of 8 on normalised queries and keys makes both maps nearly one-hot over up to 300 visible keys, so every
    row reads single values from anywhere in the sequence: across pages, hundreds of tokens back, and, decoded, far
    behind the portion they came in with.  A page, a map or a key/value head that is off picks another value."""
    m = VoziraxModel(_one("attention", attn(4, 2, 16, 24, 8.0, 0.4, temp=(0.5, 64))), seed=22)
    reqs = {"a": m.random_ids(300, 1), "b": m.random_ids(77, 2)}
    for steps in _edge_steps(reqs):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 7), "float32", tol=2e-4)
    # the maps do decide the rows: with the two maps' keys swapped the logits differ wholesale
    other = copy.deepcopy(m.plain_tensors)
    k = other["l0.mix.k"].reshape(2, 2, 16, -1)
    other["l0.mix.k"] = k.flip(1).reshape(64, -1).contiguous()
    plain = m.plain_logits(reqs["a"])
    off = (ZP.forward(m.cfg_dict, other, reqs["a"]).float() - plain).abs().amax(-1) / plain.abs().amax(-1)
    assert int((off > 0.05).sum()) >= 100


def test_a_reader_uses_its_sources_keys_under_its_own_queries():
    """Two layers, the second reading the first one's keys and values with sharp maps of its own: what it reads is what
    the first layer's pages hold (normalised keys), in prompts, decoded tokens and mixed batches."""
    cfg = _one("attention", attn(4, 2, 16, 24, 0.3, 0.4))
    cfg["layers"].append(layer("attention", attn(4, 2, 16, 24, 7.0, 0.7, temp=(1.0, 16), kv_from=0), dense(40)))
    m = VoziraxModel(cfg, seed=24)
    reqs = {"a": m.random_ids(200, 1), "b": m.random_ids(61, 2)}
    for steps in _edge_steps(reqs):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 6), "float32", tol=2e-4)


def test_a_slow_decay_remembers_the_first_tokens_and_a_fast_one_forgets():
    """A rate of e^-12 keeps what the first tokens wrote in the state for the whole prompt (head 0), a rate of e^3 with a
    large step wipes it within a token (head 1); the rest as drawn."""
    def rates(t):
        a, b = t["l0.mix.A_log"].clone(), t["l0.mix.dt_bias"].clone()
        a[0], a[1], b[1] = -12.0, 3.0, 2.0
        t["l0.mix.A_log"], t["l0.mix.dt_bias"] = a, b
    m = VoziraxModel(_one("mamba2", ssm(4, 24, 16, 2, 2, 3)), seed=23, edit=rates)
    reqs = {"a": m.random_ids(260, 3)}
    for steps in (whole_steps(reqs), cut_steps(reqs, [2, 50, 1, 17], tail=30)):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 5), "float32")


def test_long_decoding():
    m = _model("A")
    reqs = _requests(m, [260], seed=700)
    steps = cut_steps(reqs, [4], tail=250)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 5), "float32")


# ---- the engine's own entry point ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    m = _model("B")
    model, typed = load_model(m.folder, dtype, verbose=False)
    eng = LLMEngine(model, EngineConfig(dtype=dtype, max_num_seqs=3, max_batch_tokens=48, max_portion=20, max_tokens=640,
                                        max_model_len=256))
    prompts = [m.random_ids(n, 900 + n) for n in (37, 5, 70, 18)]
    outs = eng.generate(prompts, 12, stop_on_eos=False)
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        logits = m.plain_logits(list(prompt) + list(out))
        for i, tok in enumerate(out):
            lg = logits[len(prompt) - 1 + i]
            if tok != int(lg.argmax()):                      # a tie that rounding may decide either way
                assert float(lg.max() - lg[tok]) / float(lg.abs().max()) <= 2 * TOLERANCE[dtype], (i, tok)
    eng.runner.cache.check()
    assert eng.runner.cache.slots.num_free == 3


def test_the_entry_point_class_and_the_command_line(tmp_path):
    """config.json picks the entry-point class; greedy `sample` equals the plain argmax, teacher-forced; the demo
    command line writes a folder of random weights from a config.json and samples from it."""
    import json
    import os
    import subprocess
    import sys
    from transformers_neuronx_b200 import NeuronAutoModelForCausalLM, VoziraxForSampling
    m = _model("A")
    model = NeuronAutoModelForCausalLM.from_pretrained(m.folder, batch_size=2, amp="f32", n_positions=64)
    assert isinstance(model, VoziraxForSampling)
    model.to_neuron()
    prompts = torch.tensor([m.random_ids(9, 41), m.random_ids(9, 42)])
    seq = model.sample(prompts, sequence_length=20, top_k=1)
    assert tuple(seq.shape) == (2, 20) and torch.equal(seq[:, :9], prompts)
    for row in seq.tolist():
        logits = m.plain_logits(row)
        for i in range(9, 20):
            lg = logits[i - 1]
            if row[i] != int(lg.argmax()):
                assert float(lg.max() - lg[row[i]]) / float(lg.abs().max()) <= 1e-4
                break
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    demo = os.path.join(root, "bin", "vozirax_demo")
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIG_A))
    folder = tmp_path / "model"
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "save", str(folder), "--random", "--config", str(cfg)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "run", str(folder), "--batch_size", "2", "--n_positions", "24",
                        "--top_k", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "generated_sequence=" in r.stdout, r.stderr
