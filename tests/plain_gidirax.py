"""A plain, slow restatement of the Gidirax decoder for tests: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the package.  Weights come as a ``{name: tensor}`` mapping and the configuration as
the dictionary config.json holds.

Notation: T tokens, W the model's width, H heads; ``h`` is a sub-layer's input ``[T, W]``; a layer is
x <- x + LN(mixer(x)); x <- x + LN(ff(x)) with the norm on the sub-layer's output.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, var = mean of squared deviations; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * f64(w)


def rms_normalise(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(x, taps, bias=None):
    """x [T, C], taps [C, K]: y[t, c] = sum_j taps[c, j] x[t - (K - 1 - j), c] (+ bias[c]), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=F), x], 0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(K):
        y += padded[j:j + T] * f64(taps[:, j])[None, :]
    if bias is not None:
        y = y + f64(bias)[None, :]
    return y


# ---- the state-space mixer ------------------------------------------------------------------------------------------

def ssm_scan(x, B, C, dt, a, D):
    """One head.  x [T, P]; B, C [T, N]; dt [T]; a = exp(A_log) > 0; D a number.  S [N, P] from zero:
    S <- exp(-a dt) S + dt B x^T;  y = S^T C + D x."""
    T, P = x.shape
    S = torch.zeros(B.shape[1], P, dtype=F)
    y = torch.zeros(T, P, dtype=F)
    for t in range(T):
        S = torch.exp(-a * dt[t]) * S + dt[t] * torch.outer(B[t], x[t])
        y[t] = S.T @ C[t] + D * x[t]
    return y


def mamba2_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, P, N = m["heads"], m["vdim"], m["state"]
    G, NG = m.get("groups") or 1, m.get("norm_groups") or 1
    inner = H * P
    proj = h @ f64(w[p + ".in"]).T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    if m.get("conv") is not None:                                 # a mixer without taps has no convolution
        xbc = causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"])
    xbc = silu(xbc)
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + f64(w[p + ".dt_bias"])[None, :])
    a = torch.exp(f64(w[p + ".A_log"]))
    D = f64(w[p + ".D"])
    y = torch.zeros(T, H, P, dtype=F)
    for i in range(H):
        g = i // (H // G)
        y[:, i] = ssm_scan(x[:, i], B[:, g], C[:, g], dt[:, i], a[i], D[i])
    y = y.reshape(T, inner) * silu(z)                              # the gate comes before the norm
    y = rms_normalise(y.view(T, NG, inner // NG), eps).reshape(T, inner) * f64(w[p + ".norm"])[None, :]
    return y @ f64(w[p + ".o"]).T


# ---- attention over a window with kept first tokens -------------------------------------------------------------------

def rotate_interleaved(x, dims, base):
    """x [T, heads, dim]: pairs (2i, 2i+1) of the first ``dims`` elements turn by p * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.clone()
    if dims == 0:
        return out
    i = torch.arange(dims // 2, dtype=F)
    ang = torch.arange(T, dtype=F)[:, None] * torch.pow(torch.tensor(base, dtype=F), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, size, keep_first):
    """mask[i, j]: j <= i and (i - j < size or j < keep_first); size None: every earlier token."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    near = (i - j < size) if size is not None else torch.ones(T, T, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def window_attention_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, V = m.get("kv_heads") or H, m.get("vdim") or D
    def branch(name, heads, size):
        x = h @ f64(w[f"{p}.{name}"]).T
        if m.get("conv") is not None:
            x = causal_conv(x, w[f"{p}.{name}.conv"])
        return x.view(T, heads, size)
    q, k, v = branch("q", H, D), branch("k", G, D), branch("v", G, V)
    q = rms_normalise(q, eps) * f64(w[p + ".q.norm"])
    k = rms_normalise(k, eps) * f64(w[p + ".k.norm"])
    rot = m.get("rot")
    if rot is not None:
        q = rotate_interleaved(q, rot["dims"], rot["base"])
        k = rotate_interleaved(k, rot["dims"], rot["base"])
    mask = m.get("mask") or {}
    see = visible(T, mask.get("size"), mask.get("keep_first") or 0)
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(H):
        g = i // (H // G)
        s = (q[:, i] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~see, -math.inf)
        out[:, i] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * V) @ f64(w[p + ".o"]).T


# ---- the gated linear recurrent unit -----------------------------------------------------------------------------------

def gated_linear_recurrence(a, b):
    """S_t = a_t S_(t-1) + b_t elementwise, from S = 0."""
    S = torch.zeros(a.shape[1], dtype=F)
    out = torch.zeros_like(a)
    for t in range(a.shape[0]):
        S = a[t] * S + b[t]
        out[t] = S
    return out


def recurrent_block_mixer(h, w, p, m, eps):
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ f64(w[p + ".y"]).T + f64(w[p + ".y.b"])[None, :])
    u = h @ f64(w[p + ".x"]).T + f64(w[p + ".x.b"])[None, :]
    if m.get("conv") is not None:
        u = causal_conv(u, w[p + ".conv"], w[p + ".conv.b"])
    ub = u.view(T, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, f64(w[p + ".ra"])) + f64(w[p + ".ra.b"])[None]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, f64(w[p + ".ri"])) + f64(w[p + ".ri.b"])[None]).reshape(T, width)
    log_a = -8.0 * r * softplus(f64(w[p + ".lam"]))[None, :]
    a = torch.exp(log_a)
    S = gated_linear_recurrence(a, torch.sqrt(1.0 - a * a) * i * u)
    return (S * y) @ f64(w[p + ".o"]).T


def parallel_mixer(h, w, p, m, eps):
    left = window_attention_mixer(h, w, p + ".left", m["left"], eps)
    right = recurrent_block_mixer(h, w, p + ".right", m["right"], eps)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


# ---- the delta rule with a decay per key channel -----------------------------------------------------------------------

def channel_delta_rule(q, k, v, g, beta):
    """One head.  q, k, g [T, D]; v [T, V]; beta [T].  S [D, V] from zero:
    S <- g[:, None] S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=F)
    out = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, KH, D, V = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    def branch(name, heads, size):
        x = h @ f64(w[f"{p}.{name}"]).T
        if m.get("conv") is not None:
            x = causal_conv(x, w[f"{p}.{name}.conv"])
        return silu(x).view(T, heads, size)
    q, k, v = branch("q", KH, D), branch("k", KH, D), branch("v", H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ f64(w[p + ".b"]).T)
    pre = (h @ f64(w[p + ".a1"]).T) @ f64(w[p + ".a2"]).T + f64(w[p + ".dt_bias"])[None, :]
    g = torch.exp(-torch.exp(f64(w[p + ".A_log"]))[None, :, None] * softplus(pre).view(T, H, D))
    o = torch.zeros(T, H, V, dtype=F)
    for i in range(H):
        j = i // (H // KH)
        o[:, i] = channel_delta_rule(q[:, j], k[:, j], v[:, i], g[:, i], beta[:, i])
    o = rms_normalise(o, eps) * f64(w[p + ".norm"])[None, None, :]
    gate = torch.sigmoid((h @ f64(w[p + ".g1"]).T) @ f64(w[p + ".g2"]).T).view(T, H, V)
    return (o * gate).reshape(T, H * V) @ f64(w[p + ".o"]).T


# ---- routed experts ---------------------------------------------------------------------------------------------------

def route(scores, top, count, keep):
    """scores [T, E] -> chosen [T, top] (indices) among the experts of the ``keep`` groups (of ``count`` equal groups of
    neighbours) whose largest score is highest."""
    T, E = scores.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    if count is not None and count > 1 and keep < count:
        best = scores.view(T, count, E // count).max(-1).values
        kept = best.topk(keep, -1).indices
        group_ok = torch.zeros(T, count, dtype=torch.bool)
        group_ok.scatter_(1, kept, True)
        allowed = group_ok[:, :, None].expand(T, count, E // count).reshape(T, E)
    return scores.masked_fill(~allowed, -1.0).topk(top, -1).indices


def expert(h, w, p):
    return (silu(h @ f64(w[p + ".gate"]).T) * (h @ f64(w[p + ".up"]).T)) @ f64(w[p + ".down"]).T


def moe_feed_forward(h, w, p, mlp):
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {}
    s = torch.softmax(h @ f64(w[p + ".router"]).T, -1)
    chosen = route(s, top, groups.get("count"), groups.get("keep", 1))
    out = torch.zeros_like(h)
    for e in range(E):
        rows = (chosen == e).any(-1)
        if rows.any():
            out[rows] += s[rows, e][:, None] * expert(h[rows], w, f"{p}.e{e}")
    return out


# ---- the model ----------------------------------------------------------------------------------------------------------

MIXERS = {"mamba2": mamba2_mixer, "parallel": parallel_mixer, "channel_delta": channel_delta_mixer}


def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out`` (a list) receives the residual after every layer."""
    eps = config["norm"]["eps"]
    x = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        x = x + layer_norm(MIXERS[layer["type"]](x, w, p + ".mix", layer["mixer"], eps), w[p + ".norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(moe_feed_forward(x, w, p + ".mlp", layer["mlp"]), w[p + ".norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ f64(w["embed"]).T
