"""Plain, slow Porarax forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Porarax tests.  It shares no code with the product package: it takes the configuration as a plain
``dict`` (the keys of config.json) and the weights as a ``dict`` of numpy arrays keyed by tensor name, and computes
everything in float64 except the rotary angle, which is the float32 product of position and frequency.  Keys and values
are BUILT per head and per token (the engine never builds the latent layers' keys), the delta rule walks token by token,
and every expert is applied to its tokens one at a time.

Notation: D model width, T tokens of one sequence.  A layer is  h = n(x);  x <- mixer(h) + ff(h) + x  with
n(x) = x / sqrt(mean(x^2) + eps) * w.  `rnd` models a bfloat16 engine: it is applied where such an engine must round
(inputs of matrix products, cached rows); the identity gives exact arithmetic.
"""
from __future__ import annotations

import numpy as np

SWISH_ALPHA = 1.702
UNIT_EPS = 1e-6


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


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def softmax_rows(s):
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


# ---- latent attention over a sliding window --------------------------------------------------------------------
def latent_rows(h, W, p, eps):
    """The cached latent of every token: the normed down-projection, [T, R]."""
    return unit_rms(h @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]


def latent_attention(h, W, p, m, c, eps, rnd=_same):
    """h [T, D] the mixer's input, c [T, R] the latents it attends over (its own or another layer's)."""
    T = h.shape[0]
    H, dn, dv, window = m["heads"], m["dim"], m["vdim"], m["mask"]["size"]
    cq = rnd(unit_rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"])
    q = rnd(cq @ W[p + "uq"].T).reshape(T, H, dn)
    c = rnd(c)
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = max(0, i - window + 1)                       # the row itself and the window - 1 rows before it
        for hh in range(H):
            keys = c[lo:i + 1] @ W[p + "uk"][hh * dn:(hh + 1) * dn].T
            vals = c[lo:i + 1] @ W[p + "uv"][hh * dv:(hh + 1) * dv].T
            pr = softmax_rows((keys @ q[i, hh])[None, :] * m["scale"])[0]
            out[i, hh] = pr @ vals
    return rnd(out.reshape(T, H * dv)) @ W[p + "o"].T


# ---- attention with rotated, unit-RMS queries and keys and an output gate -----------------------------------------
def rotate_neighbours(x, pos, base, dims):
    """x [T, heads, d]: pairs (2i, 2i+1) of the first `dims` dimensions turn by pos * base^(-2i/dims)."""
    x = x.copy()
    if dims == 0:
        return x
    i = np.arange(dims // 2, dtype=np.float64)
    freq = (base ** (-2.0 * i / dims)).astype(np.float32)
    ang = (np.asarray(pos, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float64)      # a 32-bit product
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = u * cs - v * sn
    x[..., 1:dims:2] = v * cs + u * sn
    return x


def attention(h, W, p, m, eps, rnd=_same):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, G, d)
    v = rnd(h @ W[p + "v"].T).reshape(T, G, dv)
    q = rnd(unit_rms(rotate_neighbours(q, pos, m["rot"]["base"], m["rot"]["dims"]), eps))
    k = rnd(unit_rms(rotate_neighbours(k, pos, m["rot"]["base"], m["rot"]["dims"]), eps))
    out = np.zeros((T, H, dv))
    for i in range(T):
        for hh in range(H):
            g = hh // (H // G)
            pr = softmax_rows((k[:i + 1, g] @ q[i, hh])[None, :] * m["scale"])[0]
            out[i, hh] = pr @ v[:i + 1, g]
    out = out.reshape(T, H * dv) * sigmoid(h @ W[p + "g"].T)
    return rnd(out) @ W[p + "o"].T


# ---- gated delta rule -------------------------------------------------------------------------------------------------
def short_conv(x, w):
    """x [T, C], w [C, taps]: the last tap weighs the current row, zeros stand before the first."""
    T, C = x.shape
    taps = w.shape[1]
    out = np.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += x[src] * w[:, j]
    return out


def delta(h, W, p, m, eps, rnd=_same):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + UNIT_EPS) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(h @ W[p + "b"].T)
    decay = np.exp(-np.exp(W[p + "A_log"])[None, :] * softplus(h @ W[p + "a"].T + W[p + "dt_bias"][None, :]))
    o = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, hh] = S.T @ q[t, g]
    o = unit_rms(o, eps) * W[p + "norm"][None, None, :]
    o = o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return rnd(o) @ W[p + "o"].T


# ---- mixture of experts -----------------------------------------------------------------------------------------------
def route(z, top):
    """z [E] logits -> (experts picked by descending logit, lowest index first on ties; softmax restricted to the picked)."""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    zz = np.array([z[e] for e in order])
    w = np.exp(zz - zz.max())
    return order, w / w.sum()


def expert(x, W, p, e, limit, rnd=_same):
    g = np.minimum(W[f"{p}e{e}.gate"] @ x, limit)
    u = np.clip(W[f"{p}e{e}.up"] @ x, -limit, limit)
    return W[f"{p}e{e}.down"] @ rnd(g * sigmoid(SWISH_ALPHA * g) * (u + 1.0))


def moe(h, W, p, mlp, rnd=_same):
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    z = h @ W[p + "router"].T + W[p + "router.b"][None, :]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(*route(z[t], top)):
            out[t] += w * expert(h[t], W, p, e, limit, rnd)
    return out


# ---- the model ------------------------------------------------------------------------------------------------------------
def forward(cfg, W, tokens, rnd=_same, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        h = rnd(unit_rms(x, eps) * W[L + "norm1"])
        m, kind = layer["mixer"], layer["type"]
        if kind == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_rows(h, W, L + "mix.", eps)
            y = latent_attention(h, W, L + "mix.", m, latents[i if src is None else src], eps, rnd)
        elif kind == "attention":
            y = attention(h, W, L + "mix.", m, eps, rnd)
        elif kind == "delta":
            y = delta(h, W, L + "mix.", m, eps, rnd)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            y = y + moe(h, W, L + "mlp.", layer["mlp"], rnd)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    return rnd(unit_rms(x, eps) * W["final.norm"]) @ W["embed"].T
