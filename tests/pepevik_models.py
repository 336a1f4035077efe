"""Small random Pepevik models for the tests: configurations of many shapes and bfloat16-exact random weights (so that the
device, whichever weight format it keeps, and the float64 restatement see the same numbers)."""
import numpy as np


def bf16_exact(x):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def ssm_layer(heads=4, vdim=6, state=10, groups=2, conv=3, norm_groups=2, mlp=None, weights_of=None):
    L = {"type": "mamba2", "mlp": mlp, "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def pair_layer(heads=4, kv_heads=2, dim=8, vdim=12, gru=20, scale=None, coef=0.4, every=5, mlp=None, weights_of=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
            "q_temp": {"coef": coef, "every": every}}
    L = {"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": {"width": gru}}}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=12, groups=3, keep=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def config(layers, width=40, vocab=61, eps=1e-5, emb_scale=0.7, mult=0.8, max_positions=400):
    return {"architecture": "Pepevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb_scale}, "residual_mult": mult,
            "max_positions": max_positions, "layers": layers}


def random_weights(cfg, seed=0, qk_gain=1.0):
    """name -> float32 array (bfloat16-exact).  `qk_gain` scales the query side of the attention branch: large values push the
    sigmoid weights toward 0 and 1, so a key that is lost, seen twice or weighed at the wrong distance moves the output a lot."""
    r = np.random.default_rng(seed)
    D, W = cfg["width"], {}

    def lin(n_out, n_in, gain=1.0):
        return r.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)

    def dyt(name):
        W[name] = 1.0 + 0.2 * r.standard_normal(D)
        W[name + ".b"] = 0.1 * r.standard_normal(D)
        W[name + ".alpha"] = np.array(0.5 + 0.5 * r.random())

    W["embed"] = r.standard_normal((cfg["vocab"], D))
    W["pos"] = 0.3 * r.standard_normal((cfg["max_positions"], D))
    W["head"] = lin(cfg["vocab"], D)
    dyt("final.norm")
    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        dyt(p + "norm1")
        if L["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            C = H * P + 2 * G * N
            W[p + "mix.in"] = lin(2 * H * P + 2 * G * N + H, D)
            W[p + "mix.conv"] = 0.6 * r.standard_normal((C, m["conv"]))
            W[p + "mix.conv.b"] = 0.2 * r.standard_normal(C)
            W[p + "mix.dt_bias"] = r.standard_normal(H)
            W[p + "mix.A_log"] = np.log(0.2 + 2.0 * r.random(H))
            W[p + "mix.D"] = r.standard_normal(H)
            W[p + "mix.norm"] = 1.0 + 0.2 * r.standard_normal(H * P)
            W[p + "mix.o"] = lin(D, H * P)
        else:
            l, Wd = m["left"], m["right"]["width"]
            H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            W[p + "mix.left.q"] = lin(H * d, D)
            W[p + "mix.left.k"] = lin(G * d, D)
            W[p + "mix.left.v"] = lin(G * dv, D)
            W[p + "mix.left.q.norm"] = (1.0 + 0.2 * r.standard_normal(d)) * qk_gain
            W[p + "mix.left.k.norm"] = 1.0 + 0.2 * r.standard_normal(d)
            W[p + "mix.left.r1"] = 0.2 + 0.6 * r.random(H)
            W[p + "mix.left.r2"] = 0.1 + 0.9 * r.random(H)
            W[p + "mix.left.pb"] = -1.0 + 0.5 * r.standard_normal(H)
            W[p + "mix.left.o"] = lin(D, H * dv)
            W[p + "mix.left.out"] = 1.0 + 0.2 * r.standard_normal(D)
            for n in ("z", "x", "g"):
                W[p + "mix.right." + n] = lin(Wd, D)
            W[p + "mix.right.z.b"] = 0.5 * r.standard_normal(Wd)
            W[p + "mix.right.x.b"] = 0.5 * r.standard_normal(Wd)
            W[p + "mix.right.o"] = lin(D, Wd)
            W[p + "mix.right.out"] = 1.0 + 0.2 * r.standard_normal(D)
        mlp = L["mlp"]
        if mlp is None:
            continue
        dyt(p + "norm2")
        if mlp["kind"] == "dense":
            W[p + "mlp.up"] = lin(mlp["ff"], D)
            W[p + "mlp.down"] = lin(D, mlp["ff"])
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            W[p + "mlp.router"] = lin(E, D, 2.0)
            W[p + "mlp.correction"] = 0.3 * r.standard_normal(E)
            for e in range(E):
                W[p + f"mlp.e{e}.gate"] = lin(ff, D)
                W[p + f"mlp.e{e}.up"] = lin(ff, D)
                W[p + f"mlp.e{e}.down"] = lin(D, ff)
    return {k: bf16_exact(np.asarray(v, np.float32)) for k, v in W.items()}


def as_f64(W):
    return {k: v.astype(np.float64) for k, v in W.items()}
