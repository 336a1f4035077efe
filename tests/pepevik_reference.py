"""Plain, slow restatement of the Pepevik decoder in numpy float64: one function per mechanism, written from the design's
equations and sharing no code with zgml_b200/.  Test infrastructure only.

Weights are a dict name -> float64 array with the checkpoint's tensor names; `cfg` is the parsed config.json.  Everything
walks token by token on purpose: a recurrence, a causal mask or a convolution tail cannot then be wrong by a blocking
argument.  `forward` returns the logits and the residual stream after every layer.
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms(x, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps)


def dynamic_tanh(x, W, name):
    """tanh(alpha x) w + b: no statistics of the row."""
    return np.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sigmoid_attention(h, W, pre, m, eps, pos0=0):
    """The left branch: grouped heads, RMS-normed queries and keys, a query temperature that grows with the position, a
    logarithmic distance penalty, and sigmoid weights that are not normalised over the keys.  h [T, width] -> [T, width]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ W[pre + "q"].T).reshape(T, H, d), eps) * W[pre + "q.norm"]
    k = rms((h @ W[pre + "k"].T).reshape(T, G, d), eps) * W[pre + "k.norm"]
    v = (h @ W[pre + "v"].T).reshape(T, G, dv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        qi = q[i] * query_temperature(pos0 + i, m["q_temp"]["coef"], m["q_temp"]["every"])
        for hh in range(H):
            g = hh // (H // G)
            dist = i - np.arange(i + 1)                                    # keys 0 .. i, every one of them visible
            s = (k[:i + 1, g] @ qi[hh]) * m["scale"] - W[pre + "r1"][hh] * np.log(1.0 + W[pre + "r2"][hh] * dist)
            out[i, hh] = sigmoid(s + W[pre + "pb"][hh]) @ v[:i + 1, g]
    return out.reshape(T, H * dv) @ W[pre + "o"].T


def min_gru(h, W, pre):
    """The right branch: gates read the current token only; S_t = (1 - z) S_{t-1} + z c."""
    T = h.shape[0]
    z = sigmoid(h @ W[pre + "z"].T + W[pre + "z.b"])
    u = h @ W[pre + "x"].T + W[pre + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ W[pre + "g"].T)
    S = np.zeros(z.shape[1])
    out = np.zeros_like(z)
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S * gate[t]
    return out @ W[pre + "o"].T


def parallel_mixer(h, W, pre, m, eps):
    left = sigmoid_attention(h, W, pre + "left.", m["left"], eps)
    right = min_gru(h, W, pre + "right.")
    return 0.5 * (rms(left, eps) * W[pre + "left.out"] + rms(right, eps) * W[pre + "right.out"])


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column = current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, C)), x], 0)
    y = np.zeros((T, C)) + b
    for j in range(taps):
        y += xp[j:j + T] * w[:, j]
    return y


def mamba2(h, W, pre, m, eps):
    """State-space recurrence with one scalar decay per head and step: S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zx = h @ W[pre + "in"].T
    z, xbc, dt = zx[:, :inner], zx[:, inner:2 * inner + 2 * G * N], zx[:, 2 * inner + 2 * G * N:]
    assert dt.shape[1] == H
    xbc = silu(causal_conv(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[pre + "dt_bias"])
    S = np.zeros((H, N, P))
    y = np.zeros((T, H, P))
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = math.exp(-math.exp(W[pre + "A_log"][hh]) * dt[t, hh]) * S[hh] + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + W[pre + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[pre + "norm"]
    return y @ W[pre + "o"].T


def dense_ff(h, W, pre):
    return np.maximum(h @ W[pre + "up"].T, 0.0) ** 2 @ W[pre + "down"].T


def route(h, W, pre, r):
    """-> (indices [T, top], weights [T, top]).  Sigmoid scores; the choice is made on score + correction among the experts
    of the best groups (a group counts by its two largest choice scores), the weights are the plain scores of the chosen,
    divided by their sum."""
    s = sigmoid(h @ W[pre + "router"].T)
    choice = s + W[pre + "correction"]
    T, E = s.shape
    cnt, keep = r["groups"]["count"], r["groups"]["keep"]
    per = E // cnt
    idx = np.zeros((T, r["top"]), int)
    wt = np.zeros((T, r["top"]))
    for t in range(T):
        gs = [np.sort(choice[t, g * per:(g + 1) * per])[::-1][:2].sum() for g in range(cnt)]
        kept = np.argsort(-np.asarray(gs), kind="stable")[:keep]
        masked = np.full(E, -np.inf)
        for g in kept:
            masked[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        idx[t] = np.argsort(-masked, kind="stable")[:r["top"]]
        wt[t] = s[t, idx[t]] / (s[t, idx[t]].sum() + 1e-20)
    return idx, wt


def expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def moe(h, W, pre, mlp):
    idx, wt = route(h, W, pre, mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wt[t]):
            out[t] += w * expert(h[t], W, f"{pre}e{e}.")
    return out


def forward(cfg, W, tokens):
    """-> (logits [T, vocab], residual stream after every layer [layers, T, width])."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    T = len(tokens)
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"] + W["pos"][:T]
    stream = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{L.get('weights_of', i)}."
        h = dynamic_tanh(x, W, p + "norm1")
        if L["type"] == "parallel":
            y = parallel_mixer(h, W, p + "mix.", L["mixer"], eps)
        elif L["type"] == "mamba2":
            y = mamba2(h, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + mult * y
        if L.get("mlp") is not None:
            h = dynamic_tanh(x, W, p + "norm2")
            y = dense_ff(h, W, p + "mlp.") if L["mlp"]["kind"] == "dense" else moe(h, W, p + "mlp.", L["mlp"])
            x = x + mult * y
        stream.append(x.copy())
    return dynamic_tanh(x, W, "final.norm") @ W["head"].T, np.stack(stream)
