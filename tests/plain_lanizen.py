"""A plain, slow restatement of the Lanizen decoder for tests: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the package.  Weights come as a ``{name: tensor}`` mapping and the configuration as
the dictionary config.json holds.

Notation: T tokens, W the model's width, S residual streams, H heads; ``h`` is a sub-layer's input ``[T, W]``.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def rms_normalise(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layer norm: the stored weight lies around zero, the factor is 1 + w."""
    return rms_normalise(x, eps) * (1.0 + f64(w))


def plain_norm(x, w, eps):
    return rms_normalise(x, eps) * f64(w)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x, taps):
    """x [T, C], taps [C, K]: y[t, c] = sum_j taps[c, j] x[t - (K - 1 - j), c], zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=F), x], 0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(K):
        y += padded[j:j + T] * f64(taps[:, j])[None, :]
    return y


def delta_rule(q, k, v, g, beta):
    """One head, token by token.  q, k [T, D]; v [T, V]; g, beta [T].  S [D, V] starts at zero:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, D = q.shape
    V = v.shape[1]
    S = torch.zeros(D, V, dtype=F)
    out = torch.zeros(T, V, dtype=F)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, p, m, eps):
    """The gated delta-rule mixer.  ``w``: weights, ``p``: the layer's prefix with '.mix', ``m``: its sizes."""
    T = h.shape[0]
    H, KH, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    def conv(x, name):                       # a mixer without taps has no convolution
        return causal_conv(x, w[name]) if m.get("conv") is not None else x
    q = silu(conv(h @ f64(w[p + ".q"]).T, p + ".q.conv")).view(T, KH, D)
    k = silu(conv(h @ f64(w[p + ".k"]).T, p + ".k.conv")).view(T, KH, D)
    v = silu(conv(h @ f64(w[p + ".v"]).T, p + ".v.conv")).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ f64(w[p + ".b"]).T)                                   # [T, H]
    g = torch.exp(-torch.exp(f64(w[p + ".A_log"]))[None, :] * softplus(h @ f64(w[p + ".a"]).T + f64(w[p + ".dt_bias"])[None, :]))
    gate = silu(h @ f64(w[p + ".g"]).T).view(T, H, V)
    rep = H // KH
    heads = []
    for i in range(H):
        o = delta_rule(q[:, i // rep], k[:, i // rep], v[:, i], g[:, i], beta[:, i])
        heads.append(plain_norm(o, w[p + ".norm"], eps) * gate[:, i])
    return torch.cat(heads, -1) @ f64(w[p + ".o"]).T


def rotate_interleaved(x, positions, dims, base):
    """Pairs (2i, 2i+1) of the first ``dims`` elements of the last axis are turned by position * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=F)
    ang = f64(positions)[:, None] * torch.pow(torch.tensor(base, dtype=F), -2.0 * i / dims)[None, :]   # [T, dims/2]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_of(h, w, p, m, eps, positions):
    """What a latent-attention layer caches per token: the normed latent [T, R] and the rotated shared key part [T, P]."""
    R, P = m["kv_rank"], m["rot_dim"]
    ckv = h @ f64(w[p + ".dkv"]).T
    c = plain_norm(ckv[:, :R], w[p + ".dkv.norm"], eps)
    kr = ckv[:, R:R + P]
    if m.get("rot") is not None:
        kr = rotate_interleaved(kr, positions, m["rot"]["dims"], m["rot"]["base"])
    return c, kr


def sink_softmax_attention(scores, visible, sink):
    """scores [T, T], visible a boolean mask; the denominator also holds exp(sink).  Returns the weights [T, T]."""
    s = scores.masked_fill(~visible, -math.inf)
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))


def latent_attention_mixer(h, w, p, m, eps, positions, latent):
    """``latent``: (c, rotated key part) of this layer or of the layer it reads them from."""
    T = h.shape[0]
    H, D, P, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = latent
    cq = plain_norm(h @ f64(w[p + ".dq"]).T, w[p + ".dq.norm"], eps)
    q = (cq @ f64(w[p + ".uq"]).T).view(T, H, D + P)
    qn, qr = q[..., :D], q[..., D:]
    if m.get("rot") is not None:
        qr = rotate_interleaved(qr, positions, m["rot"]["dims"], m["rot"]["base"])
    kn = (c @ f64(w[p + ".uk"]).T).view(T, H, D)
    val = (c @ f64(w[p + ".uv"]).T).view(T, H, V)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if m.get("mask") is not None:
        visible = visible & (i - j < m["mask"]["size"])
    sink = f64(w[p + ".sink"]) if (p + ".sink") in w else None
    heads = []
    for a in range(H):
        scores = (qn[:, a] @ kn[:, a].T + qr[:, a] @ kr.T) * m["scale"]
        if sink is not None:
            weights = sink_softmax_attention(scores, visible, sink[a])
        else:
            weights = torch.softmax(scores.masked_fill(~visible, -math.inf), -1)
        heads.append(weights @ val[:, a])
    out = torch.cat(heads, -1) * torch.sigmoid(h @ f64(w[p + ".g"]).T)
    return out @ f64(w[p + ".o"]).T


def dense_feed_forward(h, w, p):
    """W_down relu(W_up h)^2."""
    z = torch.relu(h @ f64(w[p + ".up"]).T)
    return (z * z) @ f64(w[p + ".down"]).T


def hyper_read(X, w_in):
    """X [S, T, W] -> the sub-layer's input sum_s in[s] X_s."""
    return torch.einsum("s,stw->tw", f64(w_in), X)


def hyper_write(X, y, w_mix, w_out):
    """X_t <- sum_s mix[s, t] X_s + out[t] y, all streams from the old ones."""
    return torch.einsum("st,sxw->txw", f64(w_mix), X) + f64(w_out)[:, None, None] * y[None]


def forward(config, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (float64); with ``return_layers`` also the residual (the sum of the
    streams) after every layer."""
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)] * config.get("embedding", {}).get("scale", 1.0)
    S = config.get("streams")
    X = x[None].repeat(S, 1, 1) if S is not None else None
    latents = {}
    after = []
    for n, layer in enumerate(config["layers"]):
        p, m = f"l{n}", layer["mixer"]

        def sublayer(q, fn, x=None):
            nonlocal X
            if X is None:
                return fn(offset_norm(x, w[f"{p}.norm{q}"], eps))
            y = fn(offset_norm(hyper_read(X, w[f"{p}.hc{q}.in"]), w[f"{p}.norm{q}"], eps))
            X = hyper_write(X, y, w[f"{p}.hc{q}.mix"], w[f"{p}.hc{q}.out"])
            return None

        def mixer(hh):
            if layer["type"] == "delta":
                return delta_mixer(hh, w, p + ".mix", m, eps)
            if m.get("kv_from") is None:
                latents[n] = latent_of(hh, w, p + ".mix", m, eps, positions)
            return latent_attention_mixer(hh, w, p + ".mix", m, eps, positions, latents[m.get("kv_from", n) if m.get("kv_from") is not None else n])

        y = sublayer(1, mixer, x)
        if X is None:
            x = x + y
        if layer.get("mlp") is not None:
            y = sublayer(2, lambda hh: dense_feed_forward(hh, w, p + ".mlp"), x)
            if X is None:
                x = x + y
        after.append(X.sum(0) if X is not None else x.clone())
    x = X.sum(0) if X is not None else x
    logits = offset_norm(x, w["final.norm"], eps) @ f64(w["head"]).T
    return (logits, torch.stack(after)) if return_layers else logits
