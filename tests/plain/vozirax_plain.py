"""A plain, slow implementation of the Vozirax decoder in 64-bit: the oracle of the tests.

One function per mechanism, loops over tokens where a loop says it most directly, whole sequences only (no cache,
no state, no batches): the engine's answers under any cut of a request must equal these.  It shares no code with
the package.

  embedding      x_t = E[token_t] + s(t),  s(t)[2i] = sin(t w_i), s(t)[2i + 1] = cos(t w_i), w_i = 10000^(-2i / width)
  layer          x <- x + ls1 * mixer(n1(x)) + ls2 * ff(n2(x)),  both sublayers read the same x;  n(y) = rms(y) * (1 + w)
  mixers         `ssd` (a selective state-space recurrence with one decay per head and token),
                 `differential_attention` (two softmax maps over the same values, subtracted)
  feed-forward   down(silu(gate h) * up h), or a mixture of experts down(relu(up h)^2) with grouped, corrected routing
  head           n_final(x), then the output matrix, times a constant
"""
import math

import torch

F64 = torch.float64


def f32(z):
    return float(torch.tensor(z, dtype=torch.float32))


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def sinusoid(positions, width):
    """[T, width]: entry 2i = sin(p w_i), entry 2i + 1 = cos(p w_i), w_i = 10000^(-2i / width).  The design forms
    positions and angles in 32-bit, so the frequency and the product are rounded to 32-bit here too; sine and cosine of
    that angle are 64-bit."""
    out = torch.zeros(len(positions), width, dtype=F64)
    for t, p in enumerate(positions):
        for i in range((width + 1) // 2):
            a = f32(float(p) * f32(10000.0 ** (-2.0 * i / width)))
            out[t, 2 * i] = math.sin(a)
            if 2 * i + 1 < width:
                out[t, 2 * i + 1] = math.cos(a)
    return out


def causal_conv(u, w, b, taps):
    """u [T, C], w [C, taps] (last column weighs the current token), b [C] or None: zeros before the start."""
    T = u.shape[0]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
        if b is not None:
            y[t] += b
    return y


def ssd(h, t, p, m, eps):
    """h [T, W].  The in-projection's rows are [z | x | B | C | dt]; x, B, C pass the convolution and silu together."""
    T, H, P, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ t[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, t[p + "conv"], t[p + "conv.b"], m["conv"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + t[p + "dt_bias"], threshold=1e9)
    A = -torch.exp(t[p + "A_log"])
    y = torch.zeros(T, H, P, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for i in range(T):
            S = torch.exp(A[hd] * dt[i, hd]) * S + dt[i, hd] * torch.outer(B[i, g], x[i, hd])
            y[i, hd] = S.T @ C[i, g] + t[p + "D"][hd] * x[i, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * t[p + "norm"]
    return y @ t[p + "o"].T


def differential_attention(h, t, p, m, eps, kv=None):
    """Returns (output, (k, v)) so that a later layer can read this layer's normalised keys and its values.
    `kv`: an earlier layer's pair, used instead of projections of this layer's own."""
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ t[p + "q"].T).reshape(T, H, 2, d), eps, t[p + "q.norm"])
    if kv is None:
        k = rms((h @ t[p + "k"].T).reshape(T, G, 2, d), eps, t[p + "k.norm"])
        v = (h @ t[p + "v"].T).reshape(T, G, dv)
    else:
        k, v = kv
    temp = m.get("q_temp")
    if temp is not None:
        for i in range(T):
            q[i] = q[i] * (1.0 + temp["coef"] * f32(math.log(float((i + 1) // temp["every"] + 1))))
    lam = (math.exp(float((t[p + "lq1"] * t[p + "lk1"]).sum())) - math.exp(float((t[p + "lq2"] * t[p + "lk2"]).sum()))
           + m["diff"])
    gate = torch.sigmoid(h @ t[p + "g"].T)                        # [T, H]
    see = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * m["scale"]
            a.append(torch.softmax(s.masked_fill(~see, -math.inf), -1) @ v[:, g])
        o = rms(a[0] - lam * a[1], eps) * (1.0 - m["diff"])
        out[:, hd] = o * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv) @ t[p + "o"].T, (k, v)


def gated_feed_forward(h, t, p):
    return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def route(h, t, p, r):
    """[(experts, weights)] per token.  Choice scores are sigmoid + correction; only experts of the `keep` groups whose
    two largest choice scores sum highest can be chosen; the weights are the chosen experts' uncorrected scores,
    normalised and scaled."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ t[p + "router"].T)
    choice = s + t[p + "correction"]
    out = []
    for i in range(h.shape[0]):
        c = choice[i].clone()
        grp = r.get("groups")
        if grp is not None:
            size = E // grp["count"]
            gs = [float(torch.topk(c[j * size:(j + 1) * size], min(2, size)).values.sum()) for j in range(grp["count"])]
            kept = sorted(range(grp["count"]), key=lambda j: (-gs[j], j))[:grp["keep"]]
            for j in range(grp["count"]):
                if j not in kept:
                    c[j * size:(j + 1) * size] = -math.inf
        ids = sorted(range(E), key=lambda e: (-float(c[e]), e))[:top]
        w = torch.stack([s[i, e] for e in ids])
        out.append((ids, w / (w.sum() + 1e-20) * r["scale"]))
    return out


def expert_feed_forward(h, t, p, r):
    y = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F64)
    for i, (ids, w) in enumerate(route(h, t, p, r)):
        for e, we in zip(ids, w):
            a = torch.relu(t[p + f"e{e}.up"] @ h[i]) ** 2
            y[i] += we * (t[p + f"e{e}.down"] @ a)
    return y


def forward(config, tensors, tokens, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer with keep_layers)."""
    t = {k: v.to(F64) for k, v in tensors.items() if v.is_floating_point()}
    W, eps = config["width"], config["norm"]["eps"]
    T = len(tokens)
    x = t["embed"][torch.tensor(tokens)] + sinusoid(range(T), W)
    kept, stream = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h1 = rms(x, eps, 1.0 + t[p + "norm1"])
        if layer["type"] == "mamba2":
            mix = ssd(h1, t, p + "mix.", m, eps)
        else:
            mix, kept[i] = differential_attention(h1, t, p + "mix.", m, eps,
                                                  kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        delta = mix * t[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = rms(x, eps, 1.0 + t[p + "norm2"])
            ff = (gated_feed_forward(h2, t, p + "mlp.") if mlp["kind"] == "dense"
                  else expert_feed_forward(h2, t, p + "mlp.", mlp["router"]))
            delta = delta + ff * t[p + "ls2"]
        x = x + delta
        stream.append(x.clone())
    logits = (rms(x, eps, 1.0 + t["final.norm"]) @ t["head"].T) * config["logit_scale"]
    return (logits, stream) if keep_layers else logits
