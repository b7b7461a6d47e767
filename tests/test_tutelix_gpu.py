"""The Tutelix decoder on the GPU against the plain implementation (tests/plain/tutelix_plain.py): every mechanism's
kernel alone, then whole models through the replay program's function (whole prompts, token by token, portions down
to two tokens, mixed batches with pages and slots used again), keys at the edges of windows made to stand out, a
memory written far back and read much later, long decoding, and greedy generation through the engine's own entry
point and scheduler."""
import copy
from types import SimpleNamespace

import pytest
import torch

from helpers import run_trace_inprocess
from plain import tutelix_plain as TP
from tutelix_helpers import (CONFIG_A, CONFIGS, TutelixModel, attention, compare, cut_steps, delta, latent, layer,
                             mixed_steps, whole_steps)
from vononex_helpers import TOLERANCE

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
_models = {}


def _model(name, seed=5):
    if (name, seed) not in _models:
        _models[(name, seed)] = TutelixModel(CONFIGS[name], seed=seed)
    return _models[(name, seed)]


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err <= tol, err


def _step_arrays(cuts):
    """cuts: per request (slot, first position, rows) -> the index arrays of a step, as the step function packs them."""
    req, pos, q_start, q_len, slots, row = [], [], [], [], [], 0
    for r, (slot, first, n) in enumerate(cuts):
        req += [r] * n
        pos += list(range(first, first + n))
        q_start.append(row); q_len.append(n); slots.append(slot)
        row += n
    return req, pos, q_start, q_len, slots


def _ctx(cuts, pad_rows=1):
    req, pos, q_start, q_len, slots = _step_arrays(cuts)
    return SimpleNamespace(token_request=_i32(req + [-1] * pad_rows), positions=_i32(pos + [0] * pad_rows),
                           q_start=_i32(q_start + [0]), q_len=_i32(q_len + [0]), state_slots=_i32(slots + [-1]),
                           decode_only=all(n == 1 for n in q_len))


# ---- each mechanism's kernel alone -----------------------------------------------------------------
@pytest.mark.parametrize("W", [72, 50, 2048])
def test_the_norm_behind_a_sublayer_and_the_norm_before_the_next_in_one_kernel(W):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    x, d = torch.randn(5, W, generator=g), torch.randn(5, W, generator=g) * 30
    w, w2 = torch.randn(W, generator=g) * 0.3, torch.randn(W, generator=g) * 0.3       # stored around zero: they act as 1 + w
    new = x.double() + TP.rms(d.double(), 1e-3, 1.0 + w.double())
    nxt = TP.rms(new, 1e-5, 1.0 + w2.double())
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 5e-3)):
        xs, out = x.to(DEV), torch.empty(5, W, device=DEV, dtype=dtype)
        ops.rms_norm_add(xs, 1.0, d.to(DEV), w.to(DEV), 1e-3, out_f32=xs, out_act=out, weight_offset=1.0,
                         then=(w2.to(DEV), 1.0, 1e-5))
        _close(xs, new, 1e-6)                                  # the stream in place, 32-bit in either engine
        _close(out, nxt, tol)                                  # the next sublayer's input
        xs = x.to(DEV)
        ops.rms_norm_add(xs, 1.0, d.to(DEV), w.to(DEV), 1e-3, out_f32=xs, out_act=out, weight_offset=1.0)
        _close(out, new, tol)                                  # without a follower: the row's copy


@pytest.mark.parametrize("rq, rkv, dr, inter, dtype", [
    (28, 40, 6, True, torch.float32), (72, 48, 16, True, torch.float32), (9, 22, 0, True, torch.float32),
    (48, 96, 32, True, torch.bfloat16), (33, 17, 10, False, torch.float32), (16, 250, 6, True, torch.float32)])
@pytest.mark.parametrize("col0", [0, 3])
def test_the_latents_are_normalised_and_the_shared_key_part_is_turned(rq, rkv, dr, inter, dtype, col0):
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.rotary import inverse_frequencies
    g = torch.Generator().manual_seed(2)
    pos = [0, 1, 2, 77, 78, 300, 5, 6]
    N, D = len(pos), -(-(rkv + dr) // 16) * 16
    proj = (torch.randn(N + 1, col0 + rq + rkv + dr + 2, generator=g) * 3).to(dtype)
    gq, gkv = torch.rand(rq, generator=g) + 0.5, torch.rand(rkv, generator=g) + 0.5
    p = proj[:N, col0:].double()
    cq = TP.rms(p[:, :rq], 1e-4, gq.double())
    c = TP.rms(p[:, rq:rq + rkv], 1e-4, gkv.double())
    r = TP.turn(p[:, rq + rkv:rq + rkv + dr].reshape(N, 1, dr), pos, dr, 777.0, inter)[:, 0] if dr else p[:, :0]
    cq_o, k_o, v_o = (torch.full((N + 1, n), 9.0, device=DEV, dtype=dtype) for n in (rq, D, D))
    ops.latent_prep(proj.to(DEV), col0, _i32([0, 0, 0, 1, 1, 2, 3, 3, -1]), _i32(pos + [0]), gq.to(DEV), gkv.to(DEV), 1e-4,
                    inverse_frequencies(dr, 777.0, DEV) if dr else None, inter, cq_o, k_o, v_o, rq, rkv, dr)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    _close(cq_o[:N], cq, tol)
    _close(k_o[:N, :rkv], c, tol)
    _close(v_o[:N, :rkv], c, tol)
    if dr:
        _close(k_o[:N, rkv:rkv + dr], r, max(tol, 3e-5))      # angles are 32-bit products of position and frequency
    assert float(k_o[:N, rkv + dr:].float().abs().max() if D > rkv + dr else 0.0) == 0.0       # the rows' padding
    assert float(v_o[:N, rkv:].float().abs().max() if D > rkv else 0.0) == 0.0                  # values have no turned part
    for o in (cq_o, k_o, v_o):
        assert float((o[N].float() - 9.0).abs().max()) == 0.0                                   # the padded row is left alone


@pytest.mark.parametrize("H, d, dr, dv, rkv, dtype", [
    (5, 12, 6, 20, 40, torch.float32), (6, 64, 16, 32, 48, torch.bfloat16), (3, 10, 0, 14, 22, torch.float32),
    (4, 32, 32, 96, 96, torch.bfloat16), (1, 7, 2, 3, 5, torch.float32), (2, 128, 64, 128, 192, torch.float32)])
@pytest.mark.parametrize("N", [1, 7, 150])
def test_scores_and_values_through_the_latent_equal_those_of_expanded_heads(H, d, dr, dv, rkv, dtype, N):
    """The part keeps one row [c | turned r | 0] per position and moves the per-head matrices to the queries' and the
    output's side.  Here: q' = [W_uk,h^T q_h | turned q_rot,h | 0] against the key row gives the expanded heads'
    scores, and W_uv,h applied to a weighted sum of latents gives the weighted sum of expanded values."""
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.rotary import inverse_frequencies
    g = torch.Generator().manual_seed(3)
    D = -(-(rkv + dr) // 16) * 16
    q = torch.randn(N + 1, H * (d + dr), generator=g).to(dtype)
    uk = (torch.randn(H * d, rkv, generator=g) * rkv ** -0.5).to(dtype)
    uv = (torch.randn(H * dv, rkv, generator=g) * rkv ** -0.5).to(dtype)
    c = torch.randn(N, rkv, generator=g).to(dtype)                      # one latent and one turned part per position
    r = torch.randn(N, dr, generator=g).to(dtype)
    pos = [(37 * n) % 128 for n in range(N)]
    req = _i32([0] * N + [-1])
    qa = torch.full((N + 1, H * D), 9.0, device=DEV, dtype=dtype)
    tail = dict(positions=_i32(pos + [0]), inv_freq=inverse_frequencies(dr, 500.0, DEV) if dr else None, rot_dims=dr,
                interleaved=True, pad_to=D) if D > rkv else {}
    ops.headwise_product(q.to(DEV), d + dr, uk.view(H, d, rkv).contiguous().to(DEV), qa, D, req, H, d, rkv, **tail)
    qh = q[:N].double().view(N, H, d + dr)
    q_rot = TP.turn(qh[:, :, d:], pos, dr, 500.0, True) if dr else qh[:, :, d:]
    k_plain = (c.double() @ uk.double().T).view(N, H, d)                # the expanded heads' unrotated keys
    want = torch.einsum("nhd,mhd->hnm", qh[:, :, :d], k_plain) + torch.einsum("nhr,mr->hnm", q_rot, r.double())
    key_row = torch.cat([c.double(), r.double(), torch.zeros(N, D - rkv - dr, dtype=F64)], 1)
    got = torch.einsum("nhD,mD->hnm", qa[:N].double().cpu().view(N, H, D), key_row)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())
    assert float(qa[:N].float().view(N, H, D)[:, :, rkv + dr:].abs().max() if D > rkv + dr else 0.0) == 0.0
    assert float((qa[N].float() - 9.0).abs().max()) == 0.0
    # the output's side: a head's slice of D dims holds a weighted sum of key rows' first rkv dims
    att = torch.randn(N + 1, H * D, generator=g).to(dtype)
    out = torch.full((N + 1, H * dv), 9.0, device=DEV, dtype=dtype)
    ops.headwise_product(att.to(DEV), D, uv.view(H, dv, rkv).transpose(1, 2).contiguous().to(DEV), out, dv, req, H, rkv, dv)
    want = torch.einsum("nhr,hvr->nhv", att[:N].double().view(N, H, D)[:, :, :rkv], uv.double().view(H, dv, rkv))
    assert float((out[:N].double().cpu().view(N, H, dv) - want).abs().max()) <= tol * float(want.abs().max())
    assert float((out[N].float() - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("H, x_head, k, n_out, out_head", [(16, 160, 128, 96, 128), (6, 80, 64, 48, 64), (4, 64, 32, 96, 128),
                                                          (3, 128, 96, 128, 128), (2, 256, 192, 40, 48), (1, 64, 64, 8, 8)])
@pytest.mark.parametrize("N", [64, 150, 300])
def test_the_per_head_products_of_all_heads_in_one_tensor_core_launch(H, x_head, k, n_out, out_head, N):
    """Head h multiplies ITS columns of x with ITS matrix and writes ITS columns of out; what lies between a head's
    n_out and out_head columns stays as it was.  Every head's inputs are scaled differently (by 1, 2, 4, ...), so a
    head that read a neighbour's columns or matrix is off by a factor."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    x = torch.randn(N, H, x_head, generator=g) * (2.0 ** torch.arange(H)).view(1, H, 1)
    w = torch.randn(H, n_out, k, generator=g) * k ** -0.5
    x, w = x.to(torch.bfloat16), w.to(torch.bfloat16)
    out = torch.full((N, H * out_head), 9.0, device=DEV, dtype=torch.bfloat16)
    xs, ws = x.view(N, H * x_head).to(DEV), w.to(DEV)
    assert ops.gemm_tc_batched_supported(xs, x_head, ws, out, out_head)
    ops.gemm_tc_batched(xs, x_head, ws, out, out_head)
    want = torch.einsum("nhi,hci->nhc", x.double()[:, :, :k], w.double())
    got = out.double().cpu().view(N, H, out_head)
    for h in range(H):
        assert float((got[:, h, :n_out] - want[:, h]).abs().max()) <= 1e-2 * float(want[:, h].abs().max()), h
    assert float((got[:, :, n_out:] - 9.0).abs().max() if out_head > n_out else 0.0) == 0.0
    # sizes it refuses: a head pitch that is no multiple of 8, k whose last block of 64 would leave the head
    assert not ops.gemm_tc_batched_supported(xs, x_head - 4, ws, out, out_head)
    if k % 64:
        assert not ops.gemm_tc_batched_supported(xs, k, ws, out, out_head)


def _plain_delta_inputs(u, a, blog, w, a_log, dt_bias, H, G, dk, dv):
    """The recurrence's inputs of one whole request from its projections (u: q, k, v side by side), in 64-bit."""
    T = u.shape[0]
    y = TP.short_conv_silu(u.double(), w.double())
    q = TP.unit(y[:, :G * dk].view(T, G, dk)) * dk ** -0.5
    k = TP.unit(y[:, G * dk:2 * G * dk].view(T, G, dk))
    v = y[:, 2 * G * dk:].view(T, H, dv)
    beta = torch.sigmoid(blog.double())
    step = torch.nn.functional.softplus(a.double() + dt_bias.double()).view(T, H, dk)
    return q, k, v, beta, torch.exp(-torch.exp(a_log.double())[None, :, None] * step)


CUTS = [(5, 1), (1, 2), (2, 0), (1, 1), (8, 17), (1, 1), (0, 1), (23, 18)]       # rows of two requests, step by step


@pytest.mark.parametrize("H, G, dk, dv, taps, dtype", [
    (6, 2, 18, 10, 5, torch.float32), (2, 2, 128, 64, 4, torch.float32), (4, 2, 32, 64, 1, torch.float32),
    (1, 1, 50, 30, 2, torch.float32), (4, 1, 64, 48, 8, torch.bfloat16), (3, 3, 256, 8, 3, torch.float32)])
@pytest.mark.parametrize("col0", [0, 5])
def test_what_enters_the_recurrence_across_cuts(H, G, dk, dv, taps, dtype, col0):
    """Two requests cut into unequal steps side by side (single tokens, pairs, a padded row, a request left out of a
    step): convolution and silu, unit vectors, write strengths and decays equal those of the whole sequences, and the
    slots hold the last taps - 1 projected values afterwards.  A slot nobody uses stays as it is."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    T, C = 41, 2 * G * dk + H * dv
    u = torch.randn(2, T, C, generator=g).to(dtype)
    blog = torch.randn(2, T, H, generator=g).to(dtype)
    a = torch.randn(2, T, H * dk, generator=g) * 3                    # the decays' logits are 32-bit in either engine
    w = torch.randn(C, taps, generator=g) * 0.5
    a_log, dt_bias = torch.randn(H, generator=g), torch.randn(H * dk, generator=g)
    want = [_plain_delta_inputs(u[r], a[r], blog[r], w, a_log, dt_bias, H, G, dk, dv) for r in range(2)]
    keep, b_off = taps - 1, col0 + C + 2
    state = torch.zeros(4, keep, C, device=DEV, dtype=dtype) if keep else None
    if keep:
        state[1].fill_(7.0)
    widths = (G * dk, G * dk, H * dv, H, H * dk)
    got = [[torch.zeros(T, n) for n in widths] for _ in range(2)]
    at = [0, 0]
    for n0, n1 in CUTS:
        reqs = [r for r, n in enumerate((n0, n1)) if n]
        cuts = [((2, 0)[r], at[r], (n0, n1)[r]) for r in reqs]
        ctx = _ctx(cuts)
        N = sum(c[2] for c in cuts)
        proj = torch.zeros(N + 1, b_off + H + 1, dtype=dtype)
        proj[:N, col0:col0 + C] = torch.cat([u[r, at[r]:at[r] + c[2]] for r, c in zip(reqs, cuts)])
        proj[:N, b_off:b_off + H] = torch.cat([blog[r, at[r]:at[r] + c[2]] for r, c in zip(reqs, cuts)])
        a_rows = torch.cat([a[r, at[r]:at[r] + c[2]] for r, c in zip(reqs, cuts)] + [torch.zeros(1, H * dk)])
        outs = [torch.full((N + 1, n), 9.0, device=DEV) for n in widths]
        ops.delta_prep(proj.to(DEV), col0, b_off, a_rows.to(DEV), w.t().contiguous().to(DEV), taps, state, ctx,
                       a_log.to(DEV), dt_bias.to(DEV), 1e-6, dk ** -0.5, "silu", *outs, H, G, dk, dv)
        for o in outs:
            assert float((o[N] - 9.0).abs().max()) == 0.0           # the padded row is left alone
        row = 0
        for r, (_, first, n) in zip(reqs, cuts):
            for j, o in enumerate(outs):
                got[r][j][first:first + n] = o[row:row + n].cpu()
            row += n; at[r] += n
    tol = 5e-6 if dtype == torch.float32 else 2e-5                     # the inputs are rounded, the arithmetic is 32-bit
    for r in range(2):
        for j in range(5):
            _close(got[r][j], want[r][j].reshape(T, -1), tol)
    if keep:
        assert float((state[1].float() - 7.0).abs().max()) == 0.0
        _close(state[2].float(), u[0, T - keep:].double(), 0.0)        # the request's last projected values, oldest first
        _close(state[0].float(), u[1, T - keep:].double(), 0.0)


@pytest.mark.parametrize("H, G, dk, dv", [(6, 2, 18, 10), (2, 2, 128, 64), (4, 2, 32, 64), (1, 1, 50, 30), (3, 1, 256, 8),
                                          (2, 1, 16, 200), (5, 5, 7, 3)])
def test_the_recurrence_across_cuts_and_slots(H, G, dk, dv):
    """The scan over two requests cut as above, against the plain recurrence over the whole sequences; then a third
    request takes a freed slot (zeroed, as the cache manager does on admission) and must not see what was there."""
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    T = 41

    def draw():
        q = TP.unit(torch.randn(T, G, dk, generator=g).double()) * dk ** -0.5
        k = TP.unit(torch.randn(T, G, dk, generator=g).double())
        v = torch.randn(T, H, dv, generator=g).double()
        beta = torch.rand(T, H, generator=g).double()
        decay = torch.rand(T, H, dk, generator=g).double() ** 0.2     # mostly near one, some rows fade fast
        return q, k, v, beta, decay
    seqs = [draw(), draw(), draw()]
    want = [TP.delta_recurrence(*s) for s in seqs]
    state = torch.zeros(4, H, dv, dk, device=DEV)
    state[1].fill_(7.0)
    got = [torch.zeros(T, H * dv) for _ in range(3)]

    def run(pairs):
        """pairs: (sequence, slot, first row, rows) of a step."""
        ctx = _ctx([(slot, first, n) for _, slot, first, n in pairs])
        N = sum(p[3] for p in pairs)
        rows = [torch.cat([seqs[s][j][first:first + n].reshape(n, -1) for s, _, first, n in pairs] +
                          [torch.full((1, seqs[0][j][0].numel()), 3.0, dtype=F64)]).float().to(DEV) for j in range(5)]
        out = torch.full((N + 1, H * dv), 9.0, device=DEV)
        ops.delta_scan(*rows, state, ctx.q_start, ctx.q_len, ctx.state_slots, out, H, G, dk, dv)
        assert float((out[N] - 9.0).abs().max()) == 0.0
        row = 0
        for s, _, first, n in pairs:
            got[s][first:first + n] = out[row:row + n].cpu(); row += n

    at = [0, 0]
    for n0, n1 in CUTS:
        run([(r, (2, 0)[r], at[r], n) for r, n in enumerate((n0, n1)) if n])
        at[0] += n0; at[1] += n1
    for r in range(2):
        _close(got[r], want[r].reshape(T, -1), 2e-5)
    assert float((state[1] - 7.0).abs().max()) == 0.0                # a slot nobody uses
    # S itself, stored [head, value dim, key dim]: S^T k for any k is what the plain state would read
    q, k, v, beta, decay = seqs[0]
    probe = torch.zeros_like(q); probe[-1] = 1.0
    state[2].zero_()                                                  # the third request takes the first one's slot
    for first, n in ((0, 2), (2, 1), (3, 38)):
        run([(2, 2, first, n)])
    _close(got[2], want[2].reshape(T, -1), 2e-5)


def test_a_value_written_long_ago_is_read_back_exactly():
    """No decay, full write strength, orthonormal keys: a value is read back many tokens and steps later bit for bit
    (sums of exact zeros) until its key is written again; a rewritten key returns its latest value, v_old + (v_new -
    v_old) in 32-bit."""
    from transformers_neuronx_b200.kernels import ops
    H, G, dk, dv, T = 2, 1, 64, 32, 200
    eye = torch.eye(dk)
    k = eye[[t % 60 for t in range(T)]].view(T, 1, dk)                 # keys 0..59 in turn; 60..63 never written
    v = torch.randn(T, H, dv, generator=torch.Generator().manual_seed(6))
    q = eye[[0] * (T - 1) + [59]].view(T, 1, dk)
    beta, decay = torch.ones(T, H), torch.ones(T, H, dk)
    state = torch.zeros(1, H, dv, dk, device=DEV)
    outs, at = [], 0
    for n in [3, 1, 1, 2, 40, 1, 1, 1, 97, 2] + [1] * 51:
        ctx = _ctx([(0, at, n)], pad_rows=0)
        rows = [x[at:at + n].reshape(n, -1).to(DEV) for x in (q, k, v, beta, decay)]
        out = torch.empty(n, H * dv, device=DEV)
        ops.delta_scan(*rows, state, ctx.q_start, ctx.q_len, ctx.state_slots, out, H, G, dk, dv)
        outs.append(out.cpu()); at += n
    o = torch.cat(outs).view(T, H, dv)
    for t in range(T - 1):                                             # key 0's latest value: written at 0, 60, 120, 180
        if t < 60:
            assert torch.equal(o[t], v[0]), t
        else:
            assert float((o[t] - v[t - t % 60]).abs().max()) <= 1e-6, t
    assert float((o[T - 1] - v[179]).abs().max()) <= 1e-6              # key 59, written at 59, 119, 179
    assert float(state[0, :, :, 60:].abs().max()) == 0.0


@pytest.mark.parametrize("H, dv, dtype", [(6, 10, torch.float32), (2, 64, torch.bfloat16), (1, 30, torch.float32),
                                         (4, 128, torch.bfloat16)])
def test_the_read_out_is_normalised_per_head_and_gated_by_a_sigmoid(H, dv, dtype):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(7)
    N = 9
    o = torch.randn(N + 1, H * dv, generator=g) * 5
    gate = torch.randn(N + 1, H * dv, generator=g).to(dtype)
    w = torch.rand(dv, generator=g) + 0.5
    out = torch.full((N + 1, H * dv), 9.0, device=DEV, dtype=dtype)
    ops.headwise_gated_rms_norm(o.to(DEV), gate.to(DEV), _i32([0] * N + [-1]), w.to(DEV), 1e-4, 1.0, out, H, dv,
                                gate_activation="sigmoid")
    want = TP.rms(o[:N].double().view(N, H, dv), 1e-4, w.double()) * torch.sigmoid(gate[:N].double().view(N, H, dv))
    _close(out[:N], want.reshape(N, -1), 3e-6 if dtype == torch.float32 else 8e-3)
    assert float((out[N].float() - 9.0).abs().max()) == 0.0


# ---- whole models through the replay function ------------------------------------------------------
LENGTHS = {"A": [1, 2, 17, 45, 130], "B": [3, 140, 300]}
# The rows' median error in bfloat16.  A walks eight layer runs of width 72 (twelve sublayers, each normalised to unit size
# before it joins the stream, so each one's rounding arrives in full): measured medians 3.8e-2 to 4.9e-2 under every cut
# alike, where B and C (wider, fewer runs) stay under the 3e-2 of the other designs' tests.  The 32-bit engine holds every
# row of all three to 3e-5.
BF16_MEDIAN = {"A": 7e-2, "B": TOLERANCE["bfloat16"], "C": TOLERANCE["bfloat16"]}


def _tol(name, dtype):
    return BF16_MEDIAN[name] if dtype == "bfloat16" else None


def _requests(m, lengths, seed=100):
    return {f"r{i}": m.random_ids(n, seed=seed + i) for i, n in enumerate(lengths)}


def test_the_stream_after_every_layer_run():
    """The residual stream after each run of a layer (a looped layer counts every pass) against the plain one: the
    first wrong run names the mechanism."""
    from transformers_neuronx_b200.engine import load_model
    from transformers_neuronx_b200.engine.step import StepEntry, StepRunner
    m = _model("A")
    ids = m.random_ids(70, 11)
    want = m.plain_hidden(ids)                                          # [runs, T, width]
    model, _ = load_model(m.folder, "float32", verbose=False)
    runner = StepRunner(model, page_size=16, num_pages=8, max_slots=2, max_model_len=128, use_cuda_graphs=False)
    runner.add_request("a")
    with model.tap_hidden_states() as taps:
        runner.step([StepEntry("a", ids, [len(ids) - 1])])
        torch.cuda.synchronize()
        assert want.shape[0] == 8 and "entry8" not in taps               # 1 + 3 passes over 2 layers + 1
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
    """Decoding through the pages and the states: the last 70 tokens one by one, so that every window (21, 33, 48 and
    64 positions) passes over decoded tokens only, and the decode steps are replayed from a captured graph."""
    m = _model(name)
    reqs = _requests(m, [n for n in LENGTHS[name] if n > 71])
    steps = cut_steps(reqs, [1000], tail=70)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype, tol=_tol(name, dtype))


def test_from_the_first_token_on_one_by_one():
    """The first positions: zeros before the start of the convolution, a state that starts at zero, windows that are
    not full yet."""
    m = _model("A")
    reqs = _requests(m, [50])
    steps = cut_steps(reqs, [1])
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_changing_size_down_to_two_tokens(name, dtype):
    """Portions shorter than the convolution (2 and 3 tokens under 5 taps), portions that end one before, at and one
    behind a page's border, and one longer than every window."""
    m = _model(name)
    reqs = _requests(m, LENGTHS[name][-2:])
    steps = cut_steps(reqs, [2, 33, 3, 16, 2, 17, 64, 5, 15, 130], tail=3)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype, tol=_tol(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype):
    """More requests than the replay program has slots: a finished request's slot (recurrent state and the
    convolution's last inputs, of every pass of a looped layer) and its pages go to the next request, and the pool
    holds no more than the live requests need."""
    m = _model(name)
    lengths = [90, 7, 33, 150, 12, 64, 5, 49, 2, 120, 31] if name == "A" else [150, 20, 70, 9, 200, 40, 33, 129, 18]
    reqs = _requests(m, lengths, seed=300)
    steps = mixed_steps(reqs, [9, 2, 31, 16, 5, 64, 3])
    most = sorted(-(-n // 64) * 64 for n in lengths)[-4:]
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, sum(most)), dtype, tol=_tol(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_no_fast_path_takes(dtype):
    m = _model("C")
    reqs = _requests(m, [3, 70, 41], seed=600)
    for steps in (whole_steps(reqs), mixed_steps(reqs, [7, 2, 19, 33], decode_tail=12)):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 4), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rows_wider_than_the_16_bit_attention_kernels_take(dtype):
    """A latent and heads of more than 256 dims a position run on the CUDA-core attention kernel in either engine."""
    m = _model("D")
    reqs = _requests(m, [75, 4, 52], seed=700)
    for steps in (whole_steps(reqs), mixed_steps(reqs, [9, 2, 31], decode_tail=40)):
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


# ---- keys at the edges of windows and far away, made to stand out ----------------------------------
def _one(kind, mixer, width=64, vocab=97, ff=None):
    return {"architecture": "Tutelix", "vocab": vocab, "width": width, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5},
            "init_std": 0.3, "layers": [layer(kind, mixer, ff)]}


def _edge_steps(reqs, window):
    """Whole prompts; portions that end right at, one before and one behind a multiple of the window, then tokens one by
    one over more than a window; and a mixed batch."""
    return (whole_steps(reqs), cut_steps(reqs, [window, window - 1, 2, window + 1, 16, 15, 1, 64], tail=window + 9),
            mixed_steps(reqs, [31, 2, window, 17], decode_tail=window + 3))


@pytest.mark.parametrize("window", [21, 32, 1])
def test_a_marked_key_is_seen_up_to_the_windows_edge_and_not_behind_it(window):
    """Token 7 is the mark: every query head carries, through its bias, the direction of the mark's key on the
    unrotated dims, 25 times over, so a query puts nearly all its weight on a mark wherever one is visible.  The marks
    sit 20 to 40 positions apart: a query at distance window - 1 from the last mark reads it, the next one must not,
    and a window that is one token off changes that row's logits wholesale.  The values are the keys, so what is read
    is the mark's own key."""
    cfg = _one("attention", attention(4, 2, 32, 1.0, window, 16, 1000.0))

    def mark(t):
        h = TP.rms(t["embed"][7].double() * 4.0, 1e-5, 1.0 + t["l0.norm1"].double())
        k = (t["l0.mix.k"].double() @ h + t["l0.mix.k.b"].double()).view(2, 32)
        k[:, :16] = 0.0                                                   # the rotated dims carry nothing of it
        qb = (25.0 * k / k.norm(dim=-1, keepdim=True) / k.norm(dim=-1, keepdim=True)).repeat_interleave(2, dim=0)
        t["l0.mix.q.b"] = qb.reshape(-1).to(torch.bfloat16)
    m = TutelixModel(cfg, seed=21, edit=mark)
    g = torch.Generator().manual_seed(4)
    ids, at = [t if t != 7 else 8 for t in m.random_ids(300, 1)], 3
    while at < 300:
        ids[at] = 7
        at += int(torch.randint(20, 41, (1,), generator=g))
    reqs = {"a": ids, "b": [t if t != 7 else 9 for t in m.random_ids(77, 2)]}
    reqs["b"][5] = 7
    for steps in _edge_steps(reqs, max(window, 4)):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 7), "float32", tol=2e-4)
    # the mark does decide the rows: without the window's edge (a window of one more) the logits differ wholesale
    wider = copy.deepcopy(cfg)
    wider["layers"][0]["mixer"]["mask"]["size"] = window + 1
    other = TP.forward_logits(ids, m.plain_tensors, wider).float()
    plain = m.plain_logits(ids)
    assert float((other - plain).abs().max()) > 0.2 * float(plain.abs().max())


@pytest.mark.parametrize("window", [33, 16, None])
def test_a_sharp_softmax_through_the_latents_finds_the_same_key(window):
    """A scale of 6 makes every head's softmax nearly one-hot over the visible keys: for one query in `window` the
    chosen key is the last one visible, for another the best key is the first one hidden.  A window, a page, a latent
    or a rotation that is off picks another value."""
    m = TutelixModel(_one("latent_attention", latent(4, 16, 8, 24, 20, 28, 6.0, window, 300.0)), seed=22)
    reqs = {"a": m.random_ids(300, 1), "b": m.random_ids(77, 2)}
    for steps in _edge_steps(reqs, window or 48):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 7), "float32", tol=2e-4)
    if window:
        wider = copy.deepcopy(m.cfg_dict)
        wider["layers"][0]["mixer"]["mask"]["size"] = window + 1
        plain = m.plain_logits(reqs["a"])
        off = (TP.forward_logits(reqs["a"], m.plain_tensors, wider).float() - plain).abs().amax(-1) / plain.abs().amax(-1)
        assert int((off > 0.05).sum()) >= 5                              # rows whose best key is the first hidden one


def test_a_slow_decay_remembers_the_first_tokens_and_a_fast_one_forgets():
    """Rates of e^-12 keep what the first tokens wrote in the state for the whole prompt (head 0), rates of e^3 wipe
    it within a token (head 1); the rest as drawn."""
    def rates(t):
        a = t["l0.mix.A_log"].clone()
        a[0], a[1] = -12.0, 3.0
        t["l0.mix.A_log"] = a
    m = TutelixModel(_one("channel_delta", delta(4, 2, 16, 24, 3, 6, 5)), seed=23, edit=rates)
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
    from transformers_neuronx_b200 import NeuronAutoModelForCausalLM, TutelixForSampling
    m = _model("A")
    model = NeuronAutoModelForCausalLM.from_pretrained(m.folder, batch_size=2, amp="f32", n_positions=64)
    assert isinstance(model, TutelixForSampling)
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
    demo = os.path.join(root, "bin", "tutelix_demo")
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIG_A))
    folder = tmp_path / "model"
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "save", str(folder), "--random", "--config", str(cfg)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "run", str(folder), "--batch_size", "2", "--n_positions", "24",
                        "--top_k", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "generated_sequence=" in r.stdout, r.stderr
