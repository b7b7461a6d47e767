"""A plain, slow implementation of the Tutelix decoder in 64-bit: the oracle of the tests.

One function per mechanism, loops over tokens where a loop says it most directly, whole sequences only (no cache,
no state, no batches): the engine's answers under any cut of a request must equal these.  It shares no code with
the package.

  embedding      x_t = E[token_t] * s_emb
  layer          x <- x + n1b(mixer(n1(x)));  x <- x + n2b(ff(n2(x)))     with n(y) = rms(y) * (1 + w)
  order          layers[0 .. start), then layers[start .. stop) `times` times in a row (the same weights, but every
                 pass is a mixer application of its own with its own past), then layers[stop ..)
  mixers         `windowed_attention` (values are the unrotated keys), `latent_attention` (queries and keys/values
                 through low-rank latents, one rotated key part shared by the heads), `gated_delta` (a recurrence
                 with a decay per key channel and an error-correcting write)
  feed-forward   down(gelu(up h)), the exact (erf) gelu
  head           n_final(x), then the output matrix
"""
import math

import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def turn(x, positions, dims, base, interleaved):
    """x [T, heads, d]: the first `dims` dims of every head turned by position * base^(-2i/dims); pair i is
    (2i, 2i + 1) when interleaved, else (i, i + dims/2).  The design forms positions and angles in 32-bit: the
    frequency and the product are rounded to 32-bit here as well (at position 180 an angle's 32-bit rounding alone moves
    the logits by 4e-5), sine and cosine of that angle are 64-bit."""
    y = x.clone()
    f32 = lambda z: float(torch.tensor(z, dtype=torch.float32))
    freq = [f32(base ** (-2.0 * i / dims)) for i in range(dims // 2)]
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a_ = f32(float(p) * freq[i])
            c, s = math.cos(a_), math.sin(a_)
            ia, ib = (2 * i, 2 * i + 1) if interleaved else (i, i + dims // 2)
            u, v = x[t, :, ia], x[t, :, ib]
            y[t, :, ia] = u * c - v * s
            y[t, :, ib] = v * c + u * s
    return y


def softmax_over_window(scores, window):
    """scores [T, T] (query, key): softmax over the keys j with 0 <= i - j < window (window None: all j <= i)."""
    T = scores.shape[0]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = (j <= i) if window is None else (j <= i) & (i - j < window)
    return torch.softmax(scores.masked_fill(~see, -math.inf), -1)


def _window(m):
    return m["mask"]["size"] if m.get("mask") else None


def windowed_attention(h, t, p, m):
    T, H, G, d = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    pos = list(range(T))
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(T, G, d)
    v = k                                                      # the values are the keys as projected
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = turn(q, pos, rot["dims"], float(rot["base"]), False)
        k = turn(k, pos, rot["dims"], float(rot["base"]), False)
    out = torch.zeros(T, H, d, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        w = softmax_over_window((q[:, hd] @ k[:, g].T) * float(m["scale"]), _window(m))
        out[:, hd] = w @ v[:, g]
    return out.reshape(T, H * d) @ t[p + "o"].T


def latent_attention(h, t, p, m, eps):
    T, H, d, dr, dv, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = list(range(T))
    base = float(m["rot"]["base"])
    cq = rms(h @ t[p + "dq"].T, eps, t[p + "dq.norm"])
    q = (cq @ t[p + "uq"].T).view(T, H, d + dr)
    q_plain, q_rot = q[:, :, :d], turn(q[:, :, d:], pos, dr, base, True)
    ckv = h @ t[p + "dkv"].T
    c = rms(ckv[:, :rank], eps, t[p + "dkv.norm"])
    k_rot = turn(ckv[:, rank:].view(T, 1, dr), pos, dr, base, True)[:, 0]
    k_plain = (c @ t[p + "uk"].T).view(T, H, d)
    v = (c @ t[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * float(m["scale"])
        out[:, hd] = softmax_over_window(s, _window(m)) @ v[:, hd]
    return out.reshape(T, H * dv) @ t[p + "o"].T


def short_conv_silu(u, w):
    """u [T, C], w [C, taps]: y_t = silu(sum_j w[:, j] u_(t - taps + 1 + j)), zeros before the first position."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for tt in range(T):
        for j in range(taps):
            src = tt - taps + 1 + j
            if src >= 0:
                y[tt] += w[:, j] * u[src]
    return y * torch.sigmoid(y)


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_recurrence(q, k, v, beta, decay):
    """q, k [T, G, d], v [T, H, dv], beta [T, H], decay [T, H, d] -> o [T, H, dv].  Per head, with S of d x dv from zero:
    S <- decay_t * S (row i by decay_t[i]); u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t."""
    T, H, dv, G, d = v.shape[0], v.shape[1], v.shape[2], k.shape[1], k.shape[2]
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for tt in range(T):
            S = decay[tt, hd][:, None] * S
            u = beta[tt, hd] * (v[tt, hd] - S.T @ k[tt, g])
            S = S + torch.outer(k[tt, g], u)
            o[tt, hd] = S.T @ q[tt, g]
    return o


def gated_delta(h, t, p, m, eps):
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit(short_conv_silu(h @ t[p + "q"].T, t[p + "q.conv"]).view(T, G, d)) * d ** -0.5
    k = unit(short_conv_silu(h @ t[p + "k"].T, t[p + "k.conv"]).view(T, G, d))
    v = short_conv_silu(h @ t[p + "v"].T, t[p + "v.conv"]).view(T, H, dv)
    beta = torch.sigmoid(h @ t[p + "b"].T)                                           # [T, H]
    rate = torch.exp(t[p + "A_log"])[None, :, None]                                  # per head
    step = torch.nn.functional.softplus((h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "dt_bias"]).view(T, H, d)
    decay = torch.exp(-rate * step)                                                  # [T, H, d]
    gate = torch.sigmoid((h @ t[p + "g1"].T) @ t[p + "g2"].T).view(T, H, dv)
    o = rms(delta_recurrence(q, k, v, beta, decay), eps, t[p + "norm"]) * gate
    return o.reshape(T, H * dv) @ t[p + "o"].T


def feed_forward(h, t, p):
    z = h @ t[p + "up"].T
    return (0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))) @ t[p + "down"].T


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward_hidden(ids, tensors, cfg):
    """The residual stream after every layer run, [runs, T, width], and the logits [T, vocab]."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    norm = lambda y, name: rms(y, eps, 1.0 + t[name])
    x = t["embed"][list(ids)] * float(cfg["embedding"]["scale"])
    after = []
    for i in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        hin = norm(x, p + "norm1")
        kind = layer["type"]
        if kind == "attention":
            y = windowed_attention(hin, t, p + "mix.", layer["mixer"])
        elif kind == "latent_attention":
            y = latent_attention(hin, t, p + "mix.", layer["mixer"], eps)
        elif kind == "channel_delta":
            y = gated_delta(hin, t, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(kind)
        x = x + norm(y, p + "norm1b")
        if layer.get("mlp") is not None:
            x = x + norm(feed_forward(norm(x, p + "norm2"), t, p + "mlp."), p + "norm2b")
        after.append(x.clone())
    return torch.stack(after), norm(x, "final.norm") @ t["head"].T


def forward_logits(ids, tensors, cfg):
    return forward_hidden(ids, tensors, cfg)[1]
