"""Small random Setirax models for the tests: configurations of many shapes and bfloat16-exact random weights (so that the
device, whichever weight format it keeps, and the float64 restatement see the same numbers)."""
import numpy as np


def bf16_exact(x):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def _own(L, mlp, weights_of):
    L["mlp"] = mlp
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def latent_layer(heads=3, dim=8, vdim=12, rank=20, window=9, scale=None, mlp=None, weights_of=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "mask": {"size": window}, "scale": scale if scale is not None else dim ** -0.5}
    return _own({"type": "latent_attention", "mixer": m}, mlp, weights_of)


def pair_layer(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, rot_dims=6, base=50.0, scaling="default", scale=1.0, softcap=5.0, window=7,
               r_heads=2, r_dim=6, r_vdim=10, tau=4.0, left_scale=0.7, right_scale=1.3, mlp=None, weights_of=None):
    """`scale` multiplies the product of two unit-RMS vectors, so scores reach +-scale * dim: the softmax is peaky and the cap bites."""
    rot = {"base": base, "dims": rot_dims}
    if scaling == "default":          # wavelengths of base 50 over 6 dims run from 6.3 to 85: all three regimes occur
        scaling = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 40}
    if scaling:
        rot["scaling"] = scaling
    left = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "rot": rot, "scale": scale, "softcap": softcap, "vdim": vdim}
    right = {"dim": r_dim, "heads": r_heads, "tau": tau, "vdim": r_vdim}
    return _own({"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right": right, "right_scale": right_scale}}, mlp, weights_of)


def lru_layer(width=24, blocks=3, conv=4, mlp=None, weights_of=None):
    return _own({"type": "rglru", "mixer": {"blocks": blocks, "conv": conv, "width": width}}, mlp, weights_of)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers, width=40, vocab=61, eps=1e-5, logit_softcap=6.0):
    return {"architecture": "Setirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": logit_softcap, "layers": layers}


def random_weights(cfg, seed=0, qk_gain=1.0, rank_a=3):
    """name -> float32 array (bfloat16-exact).  `qk_gain` scales the query projection of the latent attention: large values
    make its softmax peaky, so a key that is lost or seen once too often, or a missing sink, moves the output a lot."""
    r = np.random.default_rng(seed)
    D, W = cfg["width"], {}

    def lin(n_out, n_in, gain=1.0):
        return r.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)

    def norm(n):
        return 1.0 + 0.2 * r.standard_normal(n)

    W["embed"] = r.standard_normal((cfg["vocab"], D))
    W["final.norm"] = norm(D)
    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = norm(D)
        if L["type"] == "latent_attention":
            H, d, dv, rk = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            W[p + "mix.q"] = lin(H * d, D, qk_gain)
            W[p + "mix.dkv"] = lin(rk, D)
            W[p + "mix.dkv.norm"] = norm(rk)
            W[p + "mix.uk"] = lin(H * d, rk)
            W[p + "mix.uv"] = lin(H * dv, rk)
            W[p + "mix.sink"] = 1.0 + r.standard_normal(H)
            W[p + "mix.o"] = lin(D, H * dv)
        elif L["type"] == "parallel":
            l, rt = m["left"], m["right"]
            H, G, d, dv, taps = l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["conv"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                W[p + f"mix.left.{n}"] = lin(rows, D)
                W[p + f"mix.left.{n}.conv"] = 0.6 * r.standard_normal((rows, taps)) + (np.arange(taps) == taps - 1)
            W[p + "mix.left.o"] = lin(D, H * dv)
            Hr, dr, vr = rt["heads"], rt["dim"], rt["vdim"]
            W[p + "mix.right.q"] = lin(Hr * dr, D)
            W[p + "mix.right.k"] = lin(Hr * dr, D)
            W[p + "mix.right.v"] = lin(Hr * vr, D)
            W[p + "mix.right.g"] = lin(Hr * vr, D)
            W[p + "mix.right.a1"] = lin(rank_a, D)
            W[p + "mix.right.a2"] = lin(Hr * dr, rank_a, 2.0)
            W[p + "mix.right.a2.b"] = 2.0 + r.standard_normal(Hr * dr)          # decays between a slow leak and a fast one
            W[p + "mix.right.norm"] = norm(vr)
            W[p + "mix.right.o"] = lin(D, Hr * vr)
        else:
            Wd, B, taps = m["width"], m["blocks"], m["conv"]
            bw = Wd // B
            W[p + "mix.y"] = lin(Wd, D)
            W[p + "mix.y.b"] = 0.3 * r.standard_normal(Wd)
            W[p + "mix.x"] = lin(Wd, D)
            W[p + "mix.x.b"] = 0.3 * r.standard_normal(Wd)
            W[p + "mix.conv"] = 0.6 * r.standard_normal((Wd, taps))
            W[p + "mix.conv.b"] = 0.2 * r.standard_normal(Wd)
            W[p + "mix.ra"] = r.standard_normal((B, bw, bw)) / np.sqrt(bw)
            W[p + "mix.ra.b"] = 0.5 * r.standard_normal((B, bw))
            W[p + "mix.ri"] = r.standard_normal((B, bw, bw)) / np.sqrt(bw)
            W[p + "mix.ri.b"] = 0.5 * r.standard_normal((B, bw))
            W[p + "mix.lam"] = -2.0 + 1.5 * r.standard_normal(Wd)               # a from close to 1 down to a fraction
            W[p + "mix.o"] = lin(D, Wd)
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            W[p + "norm2"] = norm(D)
            W[p + "mlp.up"] = lin(ff, D)
            W[p + "mlp.up.b"] = 0.3 * r.standard_normal(ff)
            W[p + "mlp.down"] = lin(D, ff)
            W[p + "mlp.down.b"] = 0.3 * r.standard_normal(D)
    return {k: bf16_exact(np.asarray(v, np.float32)) for k, v in W.items()}


def as_f64(W):
    return {k: v.astype(np.float64) for k, v in W.items()}
