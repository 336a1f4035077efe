"""Setirax restated in float64 NumPy, token by token, one function per mechanism.  Shares no code with `zgml_b200/`: the GPU
tests compare the framework's sessions against this file.

Notation: x is the stream [T, D]; W are [out, in] matrices applied as `x @ W.T`; `p` maps tensor names to arrays; positions
count from 0.  A layer is post-norm only:  x += rms(mixer(x)) w1;  x += rms(ff(x)) w2  (the sublayers read x itself).
"""
import math

import numpy as np


def rms_norm(x, w, eps):
    x = np.asarray(x, np.float64)
    r = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return r if w is None else r * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: the last tap multiplies the current token, earlier ones reach back; zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    out = np.zeros((T, C))
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out if bias is None else out + bias


def rotary_frequencies(rot):
    """Pair i of `dims` turns by p * f_i; long wavelengths are slowed by `factor`, short ones kept, the band between blended."""
    dims = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if sc:
        out = f.copy()
        for i, fi in enumerate(f):
            wl = 2.0 * math.pi / fi
            if wl < sc["original"] / sc["high"]:
                continue
            if wl > sc["original"] / sc["low"]:
                out[i] = fi / sc["factor"]
            else:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
        f = out
    return f


def rotate_half(v, pos, freqs):
    """v [..., dim]; the first 2 * len(freqs) entries turn, entry i against entry i + len(freqs)."""
    h = len(freqs)
    a = pos * freqs
    c, s = np.cos(a), np.sin(a)
    out = np.array(v, np.float64)
    lo, hi = v[..., :h], v[..., h:2 * h]
    out[..., :h] = lo * c - hi * s
    out[..., h:2 * h] = hi * c + lo * s
    return out


def window_softmax_attention(q, k, v, scale, window, softcap=None, sink=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one sequence from position 0.  Query i weighs keys j with 0 <= i - j < window;
    `sink` [H] adds exp(sink_h) to the denominator only."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            m = s.max() if sink is None else max(s.max(), sink[h])
            e = np.exp(s - m)
            den = e.sum() + (0.0 if sink is None else math.exp(sink[h] - m))
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def latent_attention(h, p, pre, m, eps):
    H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ p[pre + "q"].T).reshape(T, H, dim)
    c = rms_norm(h @ p[pre + "dkv"].T, p[pre + "dkv.norm"], eps)
    k = (c @ p[pre + "uk"].T).reshape(T, H, dim)
    v = (c @ p[pre + "uv"].T).reshape(T, H, vdim)
    o = window_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], sink=p[pre + "sink"])
    return o.reshape(T, H * vdim) @ p[pre + "o"].T


def conv_rotary_attention(h, p, pre, m, eps):
    """The left branch of the pair: projections, a short convolution on q, k and v, rotary on q and k, unit RMS per head,
    capped scores, window, softmax."""
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = causal_conv(h @ p[pre + "q"].T, p[pre + "q.conv"]).reshape(T, H, dim)
    k = causal_conv(h @ p[pre + "k"].T, p[pre + "k.conv"]).reshape(T, G, dim)
    v = causal_conv(h @ p[pre + "v"].T, p[pre + "v.conv"]).reshape(T, G, vdim)
    f = rotary_frequencies(m["rot"])
    for t in range(T):
        q[t] = rotate_half(q[t], t, f)
        k[t] = rotate_half(k[t], t, f)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    o = window_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], softcap=m.get("softcap"))
    return o.reshape(T, H * vdim) @ p[pre + "o"].T


def gated_linear_attention(h, p, pre, m, eps):
    """The right branch of the pair: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, alpha = sigmoid(z)^(1 / tau) per key channel."""
    H, dim, vdim, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ p[pre + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ p[pre + "k"].T).reshape(T, H, dim)
    v = (h @ p[pre + "v"].T).reshape(T, H, vdim)
    z = (h @ p[pre + "a1"].T) @ p[pre + "a2"].T + p[pre + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, dim)
    S = np.zeros((H, dim, vdim))
    o = np.zeros((T, H, vdim))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, p[pre + "norm"], eps).reshape(T, H * vdim)
    g = h @ p[pre + "g"].T
    return (o * g * sigmoid(g)) @ p[pre + "o"].T


def parallel_mixer(h, p, pre, m, eps):
    return m["left_scale"] * conv_rotary_attention(h, p, pre + "left.", m["left"], eps) + \
        m["right_scale"] * gated_linear_attention(h, p, pre + "right.", m["right"], eps)


def rglru(h, p, pre, m):
    """Two branches: a tanh-GELU gate y and a convolved input u; block-diagonal sigmoid gates r and i on u;
    S <- a S + sqrt(1 - a^2) (i u), a = exp(-8 r softplus(lam)); out = W_o (S y)."""
    W, B = m["width"], m["blocks"]
    T = h.shape[0]
    y = gelu_tanh(h @ p[pre + "y"].T + p[pre + "y.b"])
    u = causal_conv(h @ p[pre + "x"].T + p[pre + "x.b"], p[pre + "conv"], p[pre + "conv.b"])
    ub = u.reshape(T, B, W // B)
    r = sigmoid(np.einsum("bok,tbk->tbo", p[pre + "ra"], ub) + p[pre + "ra.b"]).reshape(T, W)
    i = sigmoid(np.einsum("bok,tbk->tbo", p[pre + "ri"], ub) + p[pre + "ri.b"]).reshape(T, W)
    a = np.exp(-8.0 * r * softplus(p[pre + "lam"]))
    S = np.zeros(W)
    out = np.zeros((T, W))
    for t in range(T):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S * y[t]
    return out @ p[pre + "o"].T


def dense_ff(h, p, pre):
    z = np.maximum(h @ p[pre + "up"].T + p[pre + "up.b"], 0.0) ** 2
    return z @ p[pre + "down"].T + p[pre + "down.b"]


def forward(cfg, p, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = np.asarray(p["embed"], np.float64)[np.asarray(tokens)]
    streams = []
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{L.get('weights_of', i)}."
        m = L["mixer"]
        if L["type"] == "latent_attention":
            y = latent_attention(x, p, pre + "mix.", m, eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(x, p, pre + "mix.", m, eps)
        elif L["type"] == "rglru":
            y = rglru(x, p, pre + "mix.", m)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, p[pre + "norm1"], eps)
        if L.get("mlp") is not None:
            x = x + rms_norm(dense_ff(x, p, pre + "mlp."), p[pre + "norm2"], eps)
        streams.append(x.copy())
    z = rms_norm(x, p["final.norm"], eps) @ np.asarray(p["embed"], np.float64).T
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * np.tanh(z / cap)
    return (z, np.stack(streams)) if return_layers else z
