"""A plain, slow statement of the Girelix decoder: the tests' oracle.

One function per mechanism, in float64 torch on the CPU, token by token where a
recurrence is involved. It shares no code with the engine: weights come as a dict
of tensors under the checkpoint's names, sizes from the configuration dict.

Notation: x is the residual stream [T, C] of ONE sequence whose first token has
position 0, h its normed copy; W y means ``y @ W.T`` for a stored [out, in] matrix.
"""

from __future__ import annotations

import torch

F = torch.float64


def rms(y, eps):
    """y over the root of (the mean of its squares plus eps), along the last axis."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(y, dims, base, first_position=0):
    """Rotary positions on the first ``dims`` channels of every head of y [T, heads, D]: channel 2i turns with
    channel 2i + 1 by the angle position * base^(-2i / dims); the other channels pass."""
    T = y.shape[0]
    out = y.clone()
    pos = torch.arange(first_position, first_position + T, dtype=F)
    for i in range(dims // 2):
        a = pos * float(base) ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = y[:, :, 2 * i], y[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def sink_attention(h, w, p, m):
    """Causal softmax attention whose values are the keys as projected (before the rotation) and whose denominator
    holds one more term exp(sink) per head, without a key or a value."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = k
    rot = m["rot"]
    q, k = rotate_pairs(q, rot["dims"], rot["base"]), rotate_pairs(k, rot["dims"], rot["base"])
    out = torch.zeros(T, H, D, dtype=F)
    for i in range(T):
        for a in range(H):
            g = a // (H // G)
            s = (k[: i + 1, g] @ q[i, a]) * m["scale"]
            e = torch.exp(s)
            out[i, a] = (e / (e.sum() + torch.exp(w[p + "sink"][a]))) @ v[: i + 1, g]
    return out.reshape(T, H * D) @ w[p + "o"].T


def decayed_linear_attention(h, w, p, m, eps, state=None):
    """Linear attention with one fixed decay per head: S <- decay S + k v^T, o = S^T q on silu'd q, k, v; the heads'
    outputs are normed together, gated by sigmoid(W_g h) and projected. Returns (result, the states after)."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, D)
    k = silu(h @ w[p + "k"].T).reshape(T, H, D)
    v = silu(h @ w[p + "v"].T).reshape(T, H, V)
    S = torch.zeros(H, D, V, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        for a in range(H):
            S[a] = float(m["decay"][a]) * S[a] + torch.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    y = rms(o.reshape(T, H * V), eps) * w[p + "norm"]
    y = y * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T, S


def two_mixers(h, w, p, m, eps):
    left = sink_attention(h, w, p + "left.", m["left"])
    right, _ = decayed_linear_attention(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def route(h, w, p, r, margins=None):
    """For every token the chosen router outputs and their weights: softmax over all router outputs; the choice is
    by score plus correction among the outputs of the best groups; the weights are the plain scores, normalised.
    ``margins``, a list, receives per token how far the choice was from going another way (the smaller of the gap
    between the last kept and the first dropped group and the gap between the last chosen and the first unchosen
    output): a test in reduced precision cannot hold a token whose margin is of rounding's size."""
    n = r["experts"] + r["identity"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    size = n // count
    chosen, weights = [], []
    for t in range(h.shape[0]):
        best = choice[t].reshape(count, size).max(dim=-1).values
        groups = torch.topk(best, keep).indices.tolist()
        masked = torch.full((n,), float("-inf"), dtype=F)
        for g in groups:
            masked[g * size : (g + 1) * size] = choice[t, g * size : (g + 1) * size]
        idx = torch.topk(masked, r["top"]).indices
        if margins is not None:
            ordered = torch.sort(masked, descending=True).values
            gap = float(ordered[r["top"] - 1] - ordered[r["top"]]) if r["top"] < n else float("inf")
            if keep < count:
                groups_sorted = torch.sort(best, descending=True).values
                gap = min(gap, float(groups_sorted[keep - 1] - groups_sorted[keep]))
            margins.append(gap)
        chosen.append(idx)
        weights.append(s[t, idx] / (s[t, idx].sum() + 1e-20))
    return torch.stack(chosen), torch.stack(weights)


def expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixture(h, w, p, f, margins=None):
    """The weighted sum of the chosen experts' outputs; a router output past the real experts is an expert that
    returns its input."""
    r = f["router"]
    chosen, weights = route(h, w, p, r, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            out[t] += g * (h[t] if e >= r["experts"] else expert(h[t : t + 1], w, f"{p}e{e}.")[0])
    return out


def layer(x, w, i, entry, cfg, margins=None):
    """x + m * (ls1 * mixer(h) + ls2 * ff(h)) with ONE norm h that both sublayers read."""
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = rms(x, eps) * w[p + "norm1"]
    total = w[p + "ls1"] * two_mixers(h, w, p + "mix.", entry["mixer"], eps)
    if entry.get("mlp") is not None:
        total = total + w[p + "ls2"] * mixture(h, w, p + "mlp.", entry["mlp"], margins)
    return x + cfg["residual_mult"] * total


def forward(tokens, w, cfg, trace=None, margins=None):
    """Logits [T, vocab] of one sequence; ``trace``, a list, receives the residual stream after every layer, and
    ``margins``, a list, one list per routed layer of the tokens' routing margins (see ``route``)."""
    w = {k: v.to(F) for k, v in w.items()}
    x = w["embed"][torch.as_tensor(tokens)]
    for i, entry in enumerate(cfg["layers"]):
        here = [] if margins is not None and entry.get("mlp") is not None else None
        x = layer(x, w, i, entry, cfg, here)
        if here is not None:
            margins.append(here)
        if trace is not None:
            trace.append(x.clone())
    x = rms(x, cfg["norm"]["eps"]) * w["final.norm"]
    return x @ w["head"].T
