"""A plain, slow statement of the Gigusun decoder: the tests' oracle.

One function per mechanism, in float64 torch on the CPU, token by token where a
recurrence is involved. It shares no code with the engine: weights come as a dict
of tensors under the checkpoint's names, sizes from the configuration dict.

Notation: h is a layer's normed input [T, C] of ONE sequence whose first token has
position 0; W x means ``x @ W.T`` for a stored [out, in] matrix.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    """x over the root of (the mean of its squares plus eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(tokens, w, eps):
    x = w["embed"][tokens] + w["pos"][: len(tokens)]
    return norm_one_plus(x, w["embed.norm"], eps)


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def attention(h, w, p, m, eps):
    """Windowed softmax attention with kept first tokens, a capped score, a logarithmic distance
    penalty, a value-less sink of score 0 in the denominator and a sigmoid gate per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, V)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = norm_plain(k, w[p + "k.norm"], eps)
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, H]
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    cap, scale = m["softcap"], m["scale"]
    r1, r2 = w[p + "r1"], w[p + "r2"]
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep)]
        jt = torch.tensor(js)
        dist = (i - jt).to(F)
        for a in range(H):
            g = a // (H // G)
            s = (k[jt, g] @ q[i, a]) * scale
            s = cap * torch.tanh(s / cap)
            s = s - r1[a] * torch.log1p(r2[a] * dist)
            e = torch.exp(s)
            prob = e / (1.0 + e.sum())
            out[i, a] = prob @ v[jt, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].T


def gla(h, w, p, m, eps):
    """Gated linear attention: a decay per key channel, S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, D)
    S = torch.zeros(H, D, V, dtype=F)
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = norm_plain(o, w[p + "norm"], eps).reshape(T, H * V)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def causal_conv(x, taps):
    """x [T, C], taps [C, L] whose last column weighs the current token; zeros before the start."""
    T, C = x.shape
    L = taps.shape[1]
    padded = torch.cat([torch.zeros(L - 1, C, dtype=F), x])
    y = torch.zeros(T, C, dtype=F)
    for j in range(L):
        y = y + padded[j : j + T] * taps[:, j]
    return y


def delta(h, w, p, m, eps):
    """Gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)  # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    S = torch.zeros(H, D, V, dtype=F)
    o = torch.zeros(T, H, V, dtype=F)
    rep = H // G
    for t in range(T):
        for a in range(H):
            kk, qq = k[t, a // rep], q[t, a // rep]
            S[a] = decay[t, a] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ kk)
            S[a] = S[a] + kk[:, None] * u[None, :]
            o[t, a] = S[a].T @ qq
    o = rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * V) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def polynorm_ff(h, w, p, eps):
    """W_down act(W_up h) with act(z) = a N(z) + b N(z^2) + c N(z^3) + e, N the division by a row's root mean square."""
    z = h @ w[p + "up"].T
    a, b, c, e = w[p + "act"]
    act = a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z ** 3, eps) + e
    return act @ w[p + "down"].T


MIXERS = {"attention": attention, "gla": gla, "delta": delta}


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); optionally the residual stream after every layer."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = embed(torch.as_tensor(tokens, dtype=torch.long), w, eps)
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](norm_one_plus(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + polynorm_ff(norm_one_plus(x, w[p + "norm2"], eps), w, p + "mlp.", eps)
        layers.append(x)
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits
