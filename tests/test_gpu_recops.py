"""Recurrent-mixer DeviceOps and the new parameters of older ones alone, in one-op programs against NumPy: the values no model
of the framework uses yet (a score table under a softmax, sigmoid weights behind a sliding window, routing without groups,
every activation kind, a head norm without temperature, norm kinds in other pairings, a convolution bias without activation)
and the static checks that refuse a malformed op at compile time."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run(be, ops, sizes, inputs, out_buf, out_shape, externs=()):
    from zgml_b200 import DeviceProgram, ProgramIO
    prog = DeviceProgram(list(ops), list(sizes), [], [], list(externs))
    h = be.compile_program(prog)
    assert h is not None
    got = np.zeros(out_shape, np.float32)
    be.execute_program(h, [ProgramIO(i, np.ascontiguousarray(a, dtype=np.float32).ravel()) for i, a in inputs], [ProgramIO(out_buf, got)])
    be.free_program(h)
    return got


def ctl_words(pos, slot, n=8):
    c = np.zeros(n, np.int32)
    c[0], c[1] = pos, slot
    return c.view(np.float32)


def weights(be, *arrays):
    """f32 arena of the arrays back to back (8-element aligned starts) -> (buffer, offsets)."""
    from zgml_b200 import DeviceBuffer
    parts, offs, n = [], [], 0
    for a in arrays:
        a = np.asarray(a, np.float32).ravel()
        pad = -n % 8
        parts.append(np.zeros(pad, np.float32))
        n += pad
        offs.append(n)
        parts.append(a)
        n += a.size
    flat = np.concatenate(parts + [np.zeros(-n % 8 + 8, np.float32)])
    buf = DeviceBuffer(be, flat.nbytes, zero=False)
    buf.upload(flat)
    return buf, offs


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


@pytest.mark.parametrize("weights_kind,mask,dims", [("softmax", "causal", (4, 2, 8, 12)), ("sigmoid", "window", (2, 1, 64, 32)), ("sigmoid", "block", (3, 3, 7, 5)),
                                                    ("softmax", "window", (6, 2, 5, 3))], ids=["softmax-table", "sigmoid-window", "sigmoid-block-odd", "softmax-window-odd"])
def test_score_table_and_weight_kinds(cuda_backend, weights_kind, mask, dims):
    """A distance table under either kind of weights and every mask, in steps of 10 tokens over 70 positions and then token by
    token (the few-row kernel and its merge of key shares)."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer
    H, G, dk, dv = dims
    n, size = 90, 23
    R, width = n, G * (dk + dv)
    r = np.random.default_rng(sum(dims))
    q = r.standard_normal((n, H, dk)).astype(np.float32) * 1.5
    kv = r.standard_normal((n, width)).astype(np.float32)
    table = (r.standard_normal((H, R)) - 0.02 * np.arange(R)).astype(np.float32)
    cache = DeviceBuffer(cuda_backend, 4 * 2 * R * width)
    tab = DeviceBuffer(cuda_backend, table.nbytes, zero=False)
    tab.upload(table)
    got = []
    steps = [(at, 10) for at in range(0, 70, 10)] + [(at, 1) for at in range(70, n)]
    for at, T in steps:
        ops = [DeviceOp.cache_append(3, 1, 2, 0, 0, T, width, width, width, R),
               DeviceOp.cached_attention(4, 0, 3, 3, 2, 0, 0, G * dk, T, H, G, 1, dk, dv, H * dk, width, width, R, 0.3, mask=mask, mask_size=size if mask != "causal" else 0,
                                         weights=weights_kind, score_table=5, table_len=R)]
        sizes = [T * H * dk, T * width, 8 + T, cache.elems, T * H * dv, tab.elems]
        got.append(run(cuda_backend, ops, sizes, [(0, q[at:at + T]), (1, kv[at:at + T]), (2, ctl_words(at, 1, 8 + T))], 4, (T, H, dv), [ExternBuffer(3, cache), ExternBuffer(5, tab)]))
    got = np.concatenate(got)
    k, v = kv[:, :G * dk].reshape(n, G, dk).astype(np.float64), kv[:, G * dk:].reshape(n, G, dv).astype(np.float64)
    for p in range(n):
        lo = {"causal": 0, "window": max(0, p + 1 - size), "block": p - p % size}[mask]
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:p + 1, g] @ q[p, h].astype(np.float64)) * 0.3 + table[h, p - np.arange(lo, p + 1)]
            w = sigmoid(s) if weights_kind == "sigmoid" else np.exp(s - s.max()) / np.exp(s - s.max()).sum()
            want = w @ v[lo:p + 1, g]
            assert np.abs(got[p, h] - want).max() < 3e-5 * max(1.0, np.abs(want).max()), (p, h)
    cache.free()
    tab.free()


def test_route_kinds(cuda_backend):
    from zgml_b200 import DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(7)
    T, NE, top = 9, 12, 3
    z = r.standard_normal((T, NE)).astype(np.float32) * 2
    corr = (r.standard_normal(NE) * 0.5 - 1.5).astype(np.float32)
    w, (c_off,) = weights(cuda_backend, corr)
    for groups, keep in ((0, 0), (1, 1), (4, 2), (12, 5), (3, 3)):
        got = run(cuda_backend, [DeviceOp.route(0, 1, 2, c_off, T, NE, top, abi.W_F32, mode="corrected_sigmoid", groups=groups, groups_kept=keep)], [T * top * 2, T * NE, w.elems],
                  [(1, z)], 0, (T, top, 2), [ExternBuffer(2, w)])
        s = sigmoid(z.astype(np.float64))
        choice = s + corr
        for t in range(T):
            ch = choice[t].copy()
            if groups > 1:
                per = NE // groups
                score = [np.sort(ch[g * per:(g + 1) * per])[::-1][:2].sum() for g in range(groups)]
                for g in np.argsort(-np.asarray(score), kind="stable")[keep:]:
                    ch[g * per:(g + 1) * per] = -np.inf
            idx = np.argsort(-ch, kind="stable")[:top]
            assert got[t, :, 0].view(np.int32).tolist() == idx.tolist(), (groups, keep, t)
            assert np.abs(got[t, :, 1] - s[t, idx] / s[t, idx].sum()).max() < 1e-6
    w.free()


def test_activation_kinds(cuda_backend):
    from zgml_b200 import DeviceOp
    z = np.concatenate([np.linspace(-6, 6, 97), [0.0, -0.0, 30.0, -30.0]]).astype(np.float32)
    zd = z.astype(np.float64)
    want = {"relu2": np.maximum(zd, 0) ** 2, "silu": zd * sigmoid(zd), "relu": np.maximum(zd, 0),
            "gelu_tanh": 0.5 * zd * (1 + np.tanh(np.sqrt(2 / np.pi) * (zd + 0.044715 * zd ** 3)))}
    for kind, w in want.items():
        got = run(cuda_backend, [DeviceOp.activation(0, 0, z.size, kind)], [z.size], [(0, z)], 0, z.shape)
        assert np.abs(got - w).max() < 1e-5 * max(1.0, np.abs(w).max()), kind


def test_head_norm_and_gated_norm_alone(cuda_backend):
    from zgml_b200 import DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(8)
    T, heads, dim, pad = 5, 3, 10, 4
    x = r.standard_normal((T, pad + heads * dim + 3)).astype(np.float32)
    wq = (1 + 0.3 * r.standard_normal(dim)).astype(np.float32)
    w, (off,) = weights(cuda_backend, wq)
    for coef, every, pos in ((0.0, 0, 11), (0.7, 4, 6)):
        got = run(cuda_backend, [DeviceOp.head_norm(0, 1, off, 2, pad, T, heads, dim, x.shape[1], 1e-5, abi.W_F32, temp_coef=coef, temp_every=every)], [x.size, w.elems, 8],
                  [(0, x), (2, ctl_words(pos, 0))], 0, x.shape, [ExternBuffer(1, w)])
        want = x.astype(np.float64).copy()
        for t in range(T):
            temp = 1.0 + coef * np.log((pos + t + 1) // every + 1) if every else 1.0
            v = want[t, pad:pad + heads * dim].reshape(heads, dim)
            v /= np.sqrt((v ** 2).mean(-1, keepdims=True) + 1e-5)
            v *= wq * temp
        assert np.abs(got - want).max() < 1e-5
    w.free()
    cols, groups = 24, 3
    y, g = r.standard_normal((T, cols)).astype(np.float32), r.standard_normal((T, 5 + cols)).astype(np.float32)
    gw = (1 + 0.3 * r.standard_normal(cols)).astype(np.float32)
    w, (off,) = weights(cuda_backend, gw)
    got = run(cuda_backend, [DeviceOp.gated_norm(0, 1, 2, 3, off, 5, T, cols, groups, 5 + cols, 1e-5, abi.W_F32)], [y.size, y.size, g.size, w.elems], [(1, y), (2, g)], 0, y.shape,
              [ExternBuffer(3, w)])
    v = y.astype(np.float64) * (g[:, 5:] * sigmoid(g[:, 5:].astype(np.float64)))
    v = v.reshape(T, groups, -1)
    want = (v / np.sqrt((v ** 2).mean(-1, keepdims=True) + 1e-5)).reshape(T, cols) * gw
    assert np.abs(got - want).max() < 1e-5
    w.free()


def test_norm_kinds_without_statistics(cuda_backend):
    """Dynamic Tanh alone and with a gain; the plain residual step chained with an RMS norm; a layer norm chained with a Dynamic
    Tanh; rows wider than a CTA."""
    from zgml_b200 import DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(9)
    for T, D in ((3, 40), (2, 1500), (2, 4500), (70, 24)):
        x, res = r.standard_normal((T, D)).astype(np.float32) * 2, r.standard_normal((T, D)).astype(np.float32)
        w1, b1, a1 = (1 + 0.2 * r.standard_normal(D)).astype(np.float32), (0.1 * r.standard_normal(D)).astype(np.float32), np.float32(0.7)
        w2 = (1 + 0.2 * r.standard_normal(D)).astype(np.float32)
        w, (o1, o2) = weights(cuda_backend, np.concatenate([w1, b1, [a1]]), w2)
        xd, rd = x.astype(np.float64), res.astype(np.float64)
        dyt = np.tanh(0.7 * xd) * w1 + b1
        rms = lambda v, wt: v / np.sqrt((v ** 2).mean(-1, keepdims=True) + 1e-5) * wt
        sizes = [x.size, x.size, w.elems, x.size, x.size]
        ext = [ExternBuffer(2, w)]
        got = run(cuda_backend, [DeviceOp.norm(0, 1, 2, o1, T, D, 1e-5, abi.W_F32, kind="dyt")], sizes, [(1, x)], 0, x.shape, ext)
        assert np.abs(got - dyt).max() < 2e-6
        got = run(cuda_backend, [DeviceOp.norm(0, 1, 2, o1, T, D, 1e-5, abi.W_F32, kind="dyt", res=3, gain=0.25)], sizes, [(1, x), (3, res)], 0, x.shape, ext)
        assert np.abs(got - (rd + 0.25 * dyt)).max() < 2e-6
        ops = [DeviceOp.norm(0, 1, None, 0, T, D, 1e-5, abi.W_F32, kind="none", res=3, gain=-1.5, then=4, then_w=2, then_w_off=o2, then_kind="rms")]
        got = run(cuda_backend, ops, sizes, [(1, x), (3, res)], 4, x.shape, ext)
        assert np.abs(got - rms(rd - 1.5 * xd, w2)).max() < 5e-6
        ops = [DeviceOp.norm(0, 1, 2, o2, T, D, 1e-5, abi.W_F32, kind="layer", then=4, then_w=2, then_w_off=o1, then_kind="dyt")]
        got = run(cuda_backend, ops, sizes, [(1, x)], 4, x.shape, ext)
        ln = (xd - xd.mean(-1, keepdims=True)) / np.sqrt(xd.var(-1, keepdims=True) + 1e-5) * w2
        assert np.abs(got - (np.tanh(0.7 * ln) * w1 + b1)).max() < 5e-6
        wb2 = (1 + 0.2 * r.standard_normal(D)).astype(np.float32)
        w3, (p1, p2, p3) = weights(cuda_backend, w2, wb2, np.concatenate([w1, b1, [a1]]))
        sizes = [x.size, x.size, w3.elems, x.size, x.size, x.size]
        ops = [DeviceOp.norm(0, 1, 2, p1, T, D, 1e-5, abi.W_F32, kind="rms", res=3, gain=0.35, src2=5, src2_w_off=p2, then=4, then_w=2, then_w_off=p3, then_kind="dyt")]
        both = rd + 0.35 * (rms(xd, w2) + rms(rd * 2 - 1, wb2))               # two sources, each with its own root mean square and weight
        got = run(cuda_backend, ops, sizes, [(1, x), (3, res), (5, res * 2 - 1)], 4, x.shape, [ExternBuffer(2, w3)])
        assert np.abs(got - (np.tanh(0.7 * both) * w1 + b1)).max() < 5e-6
        ops = [DeviceOp.norm(0, 1, 2, p1, T, D, 1e-5, abi.W_F32, kind="rms", res=3, gain=0.35, src2=5, src2_w_off=p2)]
        got = run(cuda_backend, ops, sizes, [(1, x), (3, res), (5, res * 2 - 1)], 0, x.shape, [ExternBuffer(2, w3)])
        assert np.abs(got - both).max() < 5e-6
        w.free()
        w3.free()


def test_conv_bias_and_embed_positions(cuda_backend):
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(10)
    T, C, taps = 7, 10, 3
    x = r.standard_normal((T, C)).astype(np.float32)
    cw, cb = r.standard_normal((C, taps)).astype(np.float32), r.standard_normal(C).astype(np.float32)
    w, (ow, ob) = weights(cuda_backend, cw, cb)
    tail = DeviceBuffer(cuda_backend, 4 * (taps - 1) * C)
    got = run(cuda_backend, [DeviceOp.causal_conv(0, 1, 2, ow, 3, 4, T, C, taps, abi.W_F32, act="none", bias_off=ob)], [x.size, x.size, w.elems, tail.elems, 8],
              [(1, x), (4, ctl_words(0, 0))], 0, x.shape, [ExternBuffer(2, w), ExternBuffer(3, tail)])
    xp = np.concatenate([np.zeros((taps - 1, C)), x.astype(np.float64)])
    want = cb + sum(xp[j:j + T] * cw[:, j] for j in range(taps))
    assert np.abs(got - want).max() < 1e-5
    w.free()
    tail.free()
    V, D, P = 11, 12, 20
    emb, pos = r.standard_normal((V, D)).astype(np.float32), r.standard_normal((P, D)).astype(np.float32)
    w, (oe, op) = weights(cuda_backend, emb, pos)
    ids = [3, 0, 10, 3]
    ctl = np.zeros(8 + 4, np.int32)
    ctl[0], ctl[8:] = 9, ids
    got = run(cuda_backend, [DeviceOp.embed(0, 1, 2, oe, 4, D, 0.5, abi.W_F32, positions_off=op)], [4 * D, 12, w.elems], [(1, ctl.view(np.float32))], 0, (4, D), [ExternBuffer(2, w)])
    assert np.abs(got - (emb[ids] * 0.5 + pos[9:13])).max() < 1e-6
    w.free()


def test_malformed_ops_are_refused(cuda_backend):
    from zgml_b200 import DeviceOp, DeviceProgram, abi
    f = abi.W_F32
    bad = [
        (DeviceOp.ssm_scan(0, 1, 2, 3, 4, 5, 0, 8, 12, 0, 0, 8, 16, 2, 3, 2, 4, 4, 20, 3, f), [24, 40, 6, 32, 4096, 8]),              # heads not a multiple of groups
        (DeviceOp.ssm_scan(0, 1, 2, 3, 4, 5, 0, 8, 12, 0, 0, 8, 16, 2, 2, 1, 4, 4, 14, 2, f), [16, 28, 4, 32, 4096, 8]),              # C columns leave the row
        (DeviceOp.ssm_scan(0, 1, 2, 3, 4, 5, 0, 8, 12, 0, 0, 8, 16, 2, 2, 1, 4, 4, 16, 2, f), [16, 32, 4, 32, 16, 8]),                # state smaller than the op lays out
        (DeviceOp.min_gru(0, 0, 1, 2, 0, 4, 8, 2, 4, 12), [24, 4, 8]),                                                                # in place
        (DeviceOp.min_gru(0, 1, 2, 3, 0, 4, 10, 2, 4, 12), [8, 24, 4, 8]),                                                            # gate columns leave the row
        (DeviceOp.gated_norm(0, 1, 2, 3, 0, 0, 2, 10, 3, 10, 1e-5, f), [20, 20, 20, 16]),                                             # columns not a multiple of the groups
        (DeviceOp.activation(0, 1, 8, "relu"), [8, 4]),                                                                               # source too short
        (DeviceOp.route(0, 1, 2, 0, 2, 12, 3, f, mode="corrected_sigmoid", groups=5, groups_kept=2), [12, 24, 16]),                   # outputs do not divide into the groups
        (DeviceOp.route(0, 1, 2, 0, 2, 12, 5, f, mode="corrected_sigmoid", groups=6, groups_kept=2), [20, 24, 16]),                   # the kept groups hold fewer outputs than are chosen
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 8, 4, 2, 2, 1, 4, 4, 8, 16, 16, 8, 1.0, score_table=4, table_len=4), [32, 32, 128, 16, 64]),   # table shorter than the reach
        (DeviceOp.cache_append(0, 1, 2, 0, 0, 4, 8, 8, 8, 16, norm_w=3, normed=6, norm_group=4), [128, 32, 16, 8]),                   # normed columns not a multiple of the group
    ]
    for i, (op, sizes) in enumerate(bad):
        assert cuda_backend.compile_program(DeviceProgram([op], sizes, [], [], [])) is None, i


@pytest.mark.parametrize("fmt", ["float32", "bfloat16"])
def test_linear_activation_epilogue(cuda_backend, fmt):
    """Every activation in the epilogue of every form of the matmul: one row, a few rows with an odd K, the exact f32 tile and
    (bfloat16 weights, many rows) the tensor-core product; with and without a bias."""
    from zgml_b200 import DeviceOp, ExternBuffer, abi
    from zgml_b200.host.weights import WeightArena
    wdt = abi.W_F32 if fmt == "float32" else abi.W_BF16
    r = np.random.default_rng(11)

    def bf16(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)).view(np.float32)

    for M, N, K in ((1, 24, 64), (3, 17, 37), (40, 70, 50), (70, 96, 128)):
        W, b = bf16(r.standard_normal((N, K)) / np.sqrt(K)), bf16(0.3 * r.standard_normal(N))
        x = bf16(r.standard_normal((M, K)) * 1.5)                         # bf16-exact inputs: the tensor-core path rounds nothing away
        A = WeightArena(wdt)
        ow, ob = A.add("w", W), A.add("b", b)
        buf = A.upload(cuda_backend)
        z = x.astype(np.float64) @ W.astype(np.float64).T
        for kind in ("relu2", "silu", "gelu_tanh", "relu", None):
            for bias in (False, True):
                zz = z + b if bias else z
                want = {"relu2": np.maximum(zz, 0) ** 2, "silu": zz * sigmoid(zz), "relu": np.maximum(zz, 0), None: zz,
                        "gelu_tanh": 0.5 * zz * (1 + np.tanh(np.sqrt(2 / np.pi) * (zz + 0.044715 * zz ** 3)))}[kind]
                op = DeviceOp.linear(0, 1, 2, ow, M, N, K, wdt, bias=2 if bias else None, bias_off=ob, act=kind)
                got = run(cuda_backend, [op], [M * N, M * K, buf.elems], [(1, x)], 0, (M, N), [ExternBuffer(2, buf)])
                assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max()), (M, N, K, kind, bias)
        buf.free()


def test_cache_append_norms_query_heads(cuda_backend):
    """The append's second job: query heads normed in place in the source rows, with and without the temperature; the key heads
    and the copied columns land in the cache as before."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(12)
    T, H, G, dim, dv, pos, R = 6, 5, 2, 12, 7, 9, 32
    rs, cw = 3 + H * dim + G * (dim + dv) + 2, G * (dim + dv)
    x = r.standard_normal((T, rs)).astype(np.float32)
    wq, wk = (1 + 0.3 * r.standard_normal(dim)).astype(np.float32), (1 + 0.3 * r.standard_normal(dim)).astype(np.float32)
    w, (oq, ok) = weights(cuda_backend, wq, wk)
    for coef, every in ((0.0, 0), (0.8, 4)):
        cache = DeviceBuffer(cuda_backend, 4 * R * cw)
        op = DeviceOp.cache_append(2, 0, 1, 3 + H * dim, 0, T, cw, rs, cw, R, norm_w=3, norm_off=ok, normed=G * dim, eps=1e-5, wdt=abi.W_F32, norm_group=dim,
                                   q_heads=H, q_col=3, q_norm_off=oq, temp_coef=coef, temp_every=every)
        got = run(cuda_backend, [op], [x.size, 8, cache.elems, w.elems], [(0, x), (1, ctl_words(pos, 0))], 0, x.shape, [ExternBuffer(2, cache), ExternBuffer(3, w)])
        rows = cache.download(np.float32, 4 * pos * cw, T * cw).reshape(T, cw)
        want = x.astype(np.float64).copy()
        for t in range(T):
            temp = 1.0 + coef * np.log((pos + t + 1) // every + 1) if every else 1.0
            q = want[t, 3:3 + H * dim].reshape(H, dim)
            q /= np.sqrt((q ** 2).mean(-1, keepdims=True) + 1e-5)
            q *= wq * temp
        assert np.abs(got - want).max() < 1e-5                              # the queries changed, nothing else of the rows did
        k = x[:, 3 + H * dim:3 + H * dim + G * dim].astype(np.float64).reshape(T, G, dim)
        k = k / np.sqrt((k ** 2).mean(-1, keepdims=True) + 1e-5) * wk
        assert np.abs(rows[:, :G * dim] - k.reshape(T, -1)).max() < 1e-5
        assert np.array_equal(rows[:, G * dim:], x[:, 3 + H * dim + G * dim:3 + H * dim + cw])
        cache.free()
    w.free()
