"""Plain, slow Turevik forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Turevik tests.  It shares no code with the product package: it takes the
configuration as a plain ``dict`` (the keys of config.json) and the weights as a ``dict`` of
numpy arrays keyed by tensor name, and computes everything in float64 except the rotary angle,
which is the float32 product of position and frequency (a 64-bit angle would differ from every
32-bit engine by more than rounding at large positions).

Notation: D model width, T tokens of one sequence; a layer is
    x <- x + post1(mixer(shift(pre1(x))))          x <- x + post2(ff(pre2(x)))
with all four norms of the form n(x) = x / sqrt(mean(x^2) + eps) * (1 + w).
"""
from __future__ import annotations

import numpy as np


def _same(x):
    return x


def bf16_round(x):
    """Nearest bfloat16 (ties to even) of every element, returned as float64."""
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    bits = x32.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return unit_rms(x, eps) * w


def token_shift(h, mu, before=None):
    """Row t becomes h[t] + (h[t-1] - h[t]) * mu; row 0 mixes with `before` (zeros for a new sequence)."""
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    if before is not None:
        prev[0] = before
    return h + (prev - h) * mu


def rotate_interleaved(v, positions, base, dims):
    """v [T, ..., n]: dimensions (2i, 2i+1), i < dims/2, are turned by positions * base^(-2i/dims)."""
    out = np.array(v, dtype=np.float64, copy=True)
    i = np.arange(dims // 2, dtype=np.float64)
    freq = (base ** (-2.0 * i / dims)).astype(np.float32)
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32).astype(np.float64)
    shape = [len(positions)] + [1] * (v.ndim - 2) + [dims // 2]
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_cache_rows(h, W, p, m, eps, positions, rnd=_same):
    """What a latent-attention layer with a down-projection of its own keeps per token: the normed
    latent [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    R, r = m["kv_rank"], m["rot_dim"]
    d = rnd(h) @ rnd(W[p + "dkv"]).T
    c = plain_norm(d[:, :R], W[p + "dkv.norm"], eps)
    kr = rotate_interleaved(d[:, R:R + r], positions, m["rot"]["base"], m["rot"]["dims"])
    return rnd(c), rnd(kr)


def latent_attention(h, W, p, m, positions, c, kr, rnd=_same):
    """Causal attention of every row of h over the latents c and shared rotated keys kr (one row per
    position 0..T-1), every head with its own up-projections, a sink in the softmax's denominator."""
    T = h.shape[0]
    H, dn, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (rnd(h) @ rnd(W[p + "q"]).T).reshape(T, H, dn + r)
    qn = q[..., :dn]
    qr = rotate_interleaved(q[..., dn:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = (rnd(c) @ rnd(W[p + "uk"]).T).reshape(-1, H, dn)
    v = (rnd(c) @ rnd(W[p + "uv"]).T).reshape(-1, H, dv)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        s = (rnd(qn[:, hh]) @ rnd(kn[:, hh]).T + rnd(qr[:, hh]) @ rnd(kr).T) * m["scale"]
        for t in range(T):
            n = int(positions[t]) + 1
            row = s[t, :n]
            top = max(row.max(), W[p + "sink"][hh])
            e = np.exp(row - top)
            den = e.sum() + np.exp(W[p + "sink"][hh] - top)
            out[t, hh] = (e / den) @ v[:n, hh]
    return rnd(out.reshape(T, H * dv)) @ rnd(W[p + "o"]).T


def mingru(h, W, p, state=None, rnd=_same):
    """Recurrence whose gate and candidate are computed from the input rows alone; returns (output, last state)."""
    z = sigmoid(rnd(h) @ rnd(W[p + "z"]).T + W[p + "z.b"])
    u = rnd(h) @ rnd(W[p + "x"]).T + W[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    g = silu(rnd(h) @ rnd(W[p + "g"]).T)
    S = np.zeros(z.shape[1]) if state is None else np.array(state, dtype=np.float64)
    ys = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        ys[t] = S * g[t]
    return rnd(ys) @ rnd(W[p + "o"]).T, S


def gated_ff(h, W, p, act, rnd=_same):
    a = act(rnd(h) @ rnd(W[p + "gate"]).T) * (rnd(h) @ rnd(W[p + "up"]).T)
    return rnd(a) @ rnd(W[p + "down"]).T


def dense_ff(h, W, p, rnd=_same):
    return gated_ff(h, W, p, gelu_tanh, rnd)


def route(h, W, p, top):
    """Scores of every expert and, per row, its `top` highest-scoring experts (lowest index first on ties)."""
    s = sigmoid(h @ W[p + "router"].T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return s, order


def moe_ff(h, W, p, mlp, rnd=_same):
    top = mlp["router"]["top"]
    s, chosen = route(rnd(h), W, p, top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t]:
            out[t] += gated_ff(s[t, e] * h[t:t + 1], W, f"{p}e{e}.", silu, rnd)[0]
    if mlp.get("shared") is not None:
        gate = sigmoid(rnd(h) @ rnd(W[p + "shared.sg"]).T)
        out += gate * gated_ff(h, W, p + "shared.", silu, rnd)
    return out


def forward(cfg: dict, W: dict, tokens, rnd=_same, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    tokens = list(tokens)
    T = len(tokens)
    pos = np.arange(T)
    x = np.asarray(W["embed"], dtype=np.float64)[tokens]
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        h = token_shift(offset_norm(x, W[L + "norm1"], eps), W[L + "shift"])
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_cache_rows(h, W, L + "mix.", m, eps, pos, rnd)
                src = i
            y = latent_attention(h, W, L + "mix.", m, pos, *kept[src], rnd=rnd)
        elif layer["type"] == "mingru":
            y, _ = mingru(h, W, L + "mix.", rnd=rnd)
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, W[L + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = offset_norm(x, W[L + "norm2"], eps)
            y = dense_ff(h, W, L + "mlp.", rnd) if mlp["kind"] == "dense" else moe_ff(h, W, L + "mlp.", mlp, rnd)
            x = x + offset_norm(y, W[L + "norm2b"], eps)
        after.append(x.copy())
    logits = rnd(offset_norm(x, W["final.norm"], eps)) @ rnd(np.asarray(W["embed"], dtype=np.float64)).T
    return (logits, np.stack(after)) if return_layers else logits


def attend_latent(qa, rows, sink, scale, n_keys):
    """One row's heads over cached rows [c | kr] directly in the latent space: qa [H, R + r], rows [n, R + r];
    returns [H, R + r] = sum_j p_j rows_j (the first R columns are the heads' latent sums) with p the softmax of (qa . rows_j) * scale over j < n_keys and the head's sink."""
    s = (qa @ rows[:n_keys].T) * scale                      # [H, n]
    top = np.maximum(s.max(axis=1), sink)
    e = np.exp(s - top[:, None])
    den = e.sum(axis=1) + np.exp(sink - top)
    return (e / den[:, None]) @ rows[:n_keys]
