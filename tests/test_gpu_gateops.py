"""The newer parameters of the sequence-model DeviceOps alone, in one-op programs against NumPy, at values no model of the
framework uses: rotary frequencies from a table (both layouts), rotary inside the heads that CACHE_APPEND norms (pairs layout,
computed frequencies, a temperature), capped scores with sinks under grouped heads and two maps with a strided, scaled
destination, the forms of the delta rule in other combinations than any model's, the real-gated recurrent unit with dense gate
columns and no output activation, the smooth cap among the activations, and the static checks that refuse malformed ops."""
import numpy as np
import pytest

from test_gpu_recops import ctl_words, run, sigmoid, weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layout", ["pairs", "halves"])
def test_rotary_from_a_frequency_table(cuda_backend, layout):
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer
    T, heads, hs, dims, pos = 4, 3, 10, 6, 21
    r = np.random.default_rng(1)
    x = r.standard_normal((T, heads * hs)).astype(np.float32)
    f = np.array([0.9, 0.05, 0.31], np.float32)
    tab = DeviceBuffer(cuda_backend, 4 * 16, zero=False)
    tab.upload(np.concatenate([np.zeros(8, np.float32), f, np.zeros(5, np.float32)]))
    got = run(cuda_backend, [DeviceOp.rotary(0, 1, 0, T, heads, hs, heads * hs, dims, 0.0, layout=layout, freqs=2, freqs_off=8)], [x.size, 8, tab.elems],
              [(0, x), (1, ctl_words(pos, 0))], 0, x.shape, [ExternBuffer(2, tab)])
    want = x.astype(np.float64).copy()
    for t in range(T):
        for h in range(heads):
            v = x[t, h * hs:h * hs + dims].astype(np.float64)
            for i in range(dims // 2):
                a, b = (2 * i, 2 * i + 1) if layout == "pairs" else (i, i + dims // 2)
                ang = (pos + t) * float(f[i])
                want[t, h * hs + a] = v[a] * np.cos(ang) - v[b] * np.sin(ang)
                want[t, h * hs + b] = v[b] * np.cos(ang) + v[a] * np.sin(ang)
    assert np.abs(got - want).max() < 2e-5
    tab.free()


@pytest.mark.parametrize("table", [False, True])
def test_cache_append_turns_heads_before_their_norm(cuda_backend, table):
    """Key heads turned, normed and appended; query heads turned and normed in place with a temperature; the other columns copied.
    Pairs layout, 6 of 10 values per head turn; frequencies computed from the base or read from a table."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(2)
    T, H, G, dim, dv, pos, R, hrot, base = 5, 3, 2, 10, 4, 13, 32, 6, 40.0
    rs, cw = 2 + H * dim + G * (dim + dv), G * (dim + dv)
    x = r.standard_normal((T, rs)).astype(np.float32)
    wq, wk = (1 + 0.3 * r.standard_normal(dim)).astype(np.float32), (1 + 0.3 * r.standard_normal(dim)).astype(np.float32)
    w, (oq, ok) = weights(cuda_backend, wq, wk)
    f = np.array([0.7, 0.11, 0.013], np.float32) if table else (base ** (-2.0 * np.arange(3) / hrot)).astype(np.float32)
    tab = DeviceBuffer(cuda_backend, 4 * 8, zero=False)
    tab.upload(np.concatenate([np.zeros(4, np.float32), f, np.zeros(1, np.float32)]))
    cache = DeviceBuffer(cuda_backend, 4 * R * cw)
    op = DeviceOp.cache_append(2, 0, 1, 2 + H * dim, 0, T, cw, rs, cw, R, norm_w=3, norm_off=ok, normed=G * dim, eps=1e-5, wdt=abi.W_F32, norm_group=dim,
                               q_heads=H, q_col=2, q_norm_off=oq, temp_coef=0.5, temp_every=4, head_rot=hrot, rot_base=base, rot_layout="pairs",
                               freqs=4 if table else None, freqs_off=4)
    got = run(cuda_backend, [op], [x.size, 8, cache.elems, w.elems, tab.elems], [(0, x), (1, ctl_words(pos, 0))], 0, x.shape,
              [ExternBuffer(2, cache), ExternBuffer(3, w), ExternBuffer(4, tab)])
    rows = cache.download(np.float32, 4 * pos * cw, T * cw).reshape(T, cw)

    def turned_unit(v, p):
        v = v.astype(np.float64).copy()
        for i in range(hrot // 2):
            a, b, ang = 2 * i, 2 * i + 1, p * float(f[i])
            v[a], v[b] = v[a] * np.cos(ang) - v[b] * np.sin(ang), v[b] * np.cos(ang) + v[a] * np.sin(ang)
        return v / np.sqrt((v ** 2).mean() + 1e-5)

    want = x.astype(np.float64).copy()
    for t in range(T):
        temp = 1.0 + 0.5 * np.log((pos + t + 1) // 4 + 1)
        for h in range(H):
            want[t, 2 + h * dim:2 + (h + 1) * dim] = turned_unit(x[t, 2 + h * dim:2 + (h + 1) * dim], pos + t) * wq * temp
        for g in range(G):
            k = turned_unit(x[t, 2 + H * dim + g * dim:2 + H * dim + (g + 1) * dim], pos + t) * wk
            assert np.abs(rows[t, g * dim:(g + 1) * dim] - k).max() < 2e-5
    assert np.abs(got - want).max() < 2e-5                                  # the queries changed, nothing else of the rows did
    assert np.array_equal(rows[:, G * dim:], x[:, 2 + H * dim + G * dim:])
    for b in (cache, w, tab):
        b.free()


@pytest.mark.parametrize("dims", [(4, 2, 2, 8, 12, 9), (6, 2, 1, 64, 32, 70), (3, 3, 1, 7, 5, 4)], ids=["two-maps", "aligned-long-window", "odd"])
def test_capped_scores_sinks_and_a_strided_destination(cuda_backend, dims):
    """Window mask over a wrapping ring, scores capped, one sink per (head, map), the result scaled and written into the middle of
    wider rows; steps of 10 tokens (the tiled or per-query kernels), then single tokens (key shares and their merge)."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    H, G, maps, dk, dv, window = dims
    T, n, cap, out_scale, scale = 10, 64, 2.0, 0.6, 0.5
    R, kw, vw = window - 1 + T, G * maps * dk, G * dv
    width, drs, dcol = kw + vw, H * maps * dv + 12, 8
    r = np.random.default_rng(sum(dims))
    q = (r.standard_normal((n, H * maps, dk)) * 1.5).astype(np.float32)
    kv = r.standard_normal((n, width)).astype(np.float32)
    sink = r.standard_normal(H * maps).astype(np.float32)
    sw, (so,) = weights(cuda_backend, sink)
    ring = DeviceBuffer(cuda_backend, 4 * 2 * R * width)
    want = np.zeros((n, H * maps, dv))
    for i in range(n):
        lo = max(0, i - window + 1)
        for hm in range(H * maps):
            h, m = hm // maps, hm % maps
            g = h // (H // G)
            k = kv[lo:i + 1, (g * maps + m) * dk:(g * maps + m + 1) * dk].astype(np.float64)
            v = kv[lo:i + 1, kw + g * dv:kw + (g + 1) * dv].astype(np.float64)
            s = cap * np.tanh(k @ q[i, hm].astype(np.float64) * scale / cap)
            e = np.exp(s)
            want[i, hm] = out_scale * (e / (e.sum() + np.exp(float(sink[hm])))) @ v
    got = np.zeros((n, H * maps, dv))

    def step(Tn, at):
        ops = [DeviceOp.cache_append(3, 1, 2, 0, 0, Tn, width, width, width, R),
               DeviceOp.cached_attention(4, 0, 3, 3, 2, 0, 0, kw, Tn, H, G, maps, dk, dv, H * maps * dk, width, width, R, scale, mask="window", mask_size=window,
                                         softcap=cap, sink=5, sink_off=so, sink_wdt=abi.W_F32, out_scale=out_scale, dst_rs=drs, dst_col=dcol)]
        out = run(cuda_backend, ops, [Tn * H * maps * dk, Tn * width, 8, ring.elems, Tn * drs, sw.elems],
                  [(0, q[at:at + Tn]), (1, kv[at:at + Tn]), (2, ctl_words(at, 1)), (4, np.full((Tn, drs), 7.0, np.float32))], 4, (Tn, drs),
                  [ExternBuffer(3, ring), ExternBuffer(5, sw)])
        assert np.all(out[:, :dcol] == 7.0) and np.all(out[:, dcol + H * maps * dv:] == 7.0)      # the columns beside the heads are not touched
        got[at:at + Tn] = out[:, dcol:dcol + H * maps * dv].reshape(Tn, H * maps, dv)

    for at in range(0, 50, T):
        step(T, at)
    for at in range(50, n):
        step(1, at)
    assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max())
    ring.free()
    sw.free()


def _rule_reference(form, S, q, k, v, beta_l, a, gate, A_log, dt_bias, norm_w, tau, q_scale, eps, unit_eps, out_scale):
    """The delta rule in its forms from the state S, token by token in float64: plain (no unit vectors, no correction), decay
    kind, gate kind."""
    T, H, dim = q.shape
    vdim = v.shape[2]
    S = S.copy()
    out = np.zeros((T, H, vdim))
    for t in range(T):
        for h in range(H):
            z = a[t, h] + dt_bias[h]
            g = np.exp(-np.logaddexp(0, -z) / tau) if form["sigmoid_decay"] else np.exp(-np.exp(A_log[h]) * np.logaddexp(0, z))
            qt, kt = q[t, h] * q_scale, k[t, h]
            if not form["plain"]:
                qt, kt = q[t, h] * q_scale / np.sqrt((q[t, h] ** 2).sum() + unit_eps), k[t, h] / np.sqrt((k[t, h] ** 2).sum() + unit_eps)
            S[h] = g[:, None] * S[h]
            u = v[t, h] if form["plain"] else sigmoid(beta_l[t, h]) * (v[t, h] - S[h].T @ kt)
            S[h] = S[h] + np.outer(kt, u)
            o = S[h].T @ qt
            gt = gate[t, h]
            out[t, h] = o / np.sqrt((o ** 2).mean() + eps) * norm_w * (gt * sigmoid(gt) if form["silu_gate"] else sigmoid(gt)) * out_scale
    return out, S


@pytest.mark.parametrize("T", [1, 5, 40])
@pytest.mark.parametrize("form", [dict(plain=True, sigmoid_decay=False, silu_gate=False), dict(plain=False, sigmoid_decay=True, silu_gate=True),
                                  dict(plain=True, sigmoid_decay=True, silu_gate=False)], ids=["plain-exp-decay", "corrected-sigmoid-decay-silu", "plain-sigmoid-decay"])
def test_forms_of_the_delta_rule(cuda_backend, form, T):
    """Single tokens, short steps (the in-kernel preparation) and long ones (the prepared walk); the state carries over two steps."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(7)
    H, dim, vdim, tau, eps, unit_eps, q_scale, out_scale = 3, 20, 12, 3.0, 1e-5, 1e-6, 0.4, 1.5
    qrs, drs, dcol = 2 * H * dim + 2 * H * vdim + H, H * vdim + 5, 3
    A_log, dt_bias, norm_w = r.standard_normal(H) * 0.5, r.standard_normal((H, dim)) + 1.5, 1 + 0.2 * r.standard_normal(vdim)
    w, (oA, odt, onw) = weights(cuda_backend, A_log, dt_bias, norm_w)
    state = DeviceBuffer(cuda_backend, 4 * 2 * H * dim * vdim)
    S_want = np.zeros((H, dim, vdim))
    for rep in range(2):
        proj = r.standard_normal((T, qrs)).astype(np.float32)
        a = r.standard_normal((T, H * dim)).astype(np.float32)
        q, k = proj[:, :H * dim].reshape(T, H, dim), proj[:, H * dim:2 * H * dim].reshape(T, H, dim)
        v, gate = proj[:, 2 * H * dim:2 * H * dim + H * vdim].reshape(T, H, vdim), proj[:, 2 * H * dim + H * vdim:2 * H * dim + 2 * H * vdim].reshape(T, H, vdim)
        beta = proj[:, 2 * H * dim + 2 * H * vdim:]
        op = DeviceOp.delta_rule(0, 1, None if form["plain"] else 1, 2, 1, 3, 4, 5, 0, H * dim, 2 * H * dim, 2 * H * dim + 2 * H * vdim, oA, odt, onw, T, H, H, dim, vdim, qrs, qrs,
                                 H * dim, qrs, abi.W_F32, eps, unit_eps, q_scale, gate_off=2 * H * dim + H * vdim, plain=form["plain"],
                                 decay_tau=tau if form["sigmoid_decay"] else None, silu_gate=form["silu_gate"], out_scale=out_scale, dst_rs=drs, dst_col=dcol)
        got = run(cuda_backend, [op], [T * drs, proj.size, a.size, w.elems, state.elems, 8], [(1, proj), (2, a), (5, ctl_words(rep * T, 1))], 0, (T, drs),
                  [ExternBuffer(3, w), ExternBuffer(4, state)])
        f64 = lambda x: x.astype(np.float64)
        want, S_want = _rule_reference(form, S_want, f64(q), f64(k), f64(v), f64(beta), f64(a).reshape(T, H, dim), f64(gate), A_log, dt_bias, norm_w, tau, q_scale, eps, unit_eps, out_scale)
        assert np.abs(got[:, dcol:dcol + H * vdim].reshape(T, H, vdim) - want).max() < 2e-4 * max(1.0, np.abs(want).max()), rep
        S_got = state.download(np.float32, 4 * H * dim * vdim, H * dim * vdim).reshape(H, dim, vdim)      # slot 1
        assert np.abs(S_got - S_want).max() < 2e-5 * max(1.0, np.abs(S_want).max()), rep
    w.free()
    state.free()


def test_rg_lru_alone(cuda_backend):
    """Dense gate columns (one block as wide as the unit), no activation on the output branch, another rate than the usual one;
    a step of 70 tokens (segments side by side), then single tokens from the state it left, in slot 1."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(9)
    W, rate = 19, 3.0
    rb, ib, lam = r.standard_normal(W) * 0.5, r.standard_normal(W) * 0.5, r.standard_normal(W) - 1.0
    w, (orb, oib, olam) = weights(cuda_backend, rb, ib, lam)
    state = DeviceBuffer(cuda_backend, 4 * 2 * W)
    n = 76
    u, gates, y = r.standard_normal((n, W + 3)).astype(np.float32), r.standard_normal((n, 2 * W + 1)).astype(np.float32), r.standard_normal((n, W)).astype(np.float32)
    S, want = np.zeros(W), np.zeros((n, W))
    for t in range(n):
        a = np.exp(-rate * sigmoid(gates[t, 1:1 + W].astype(np.float64) + rb) * np.logaddexp(0, lam))
        S = a * S + np.sqrt(1 - a * a) * sigmoid(gates[t, 1 + W:].astype(np.float64) + ib) * u[t, 3:]
        want[t] = S * y[t]
    got = np.zeros((n, W))
    for at, T in [(0, 70)] + [(t, 1) for t in range(70, n)]:
        op = DeviceOp.rg_lru(0, 1, 2, 3, 4, 5, 6, 3, 1, 1 + W, 0, orb, oib, olam, T, W, W + 3, 2 * W + 1, W, W, W, abi.W_F32, rate=rate, y_act=None)
        got[at:at + T] = run(cuda_backend, [op], [T * W, T * (W + 3), T * (2 * W + 1), T * W, w.elems, state.elems, 8],
                             [(1, u[at:at + T]), (2, gates[at:at + T]), (3, y[at:at + T]), (6, ctl_words(at, 1))], 0, (T, W), [ExternBuffer(4, w), ExternBuffer(5, state)])
    assert np.abs(got - want).max() < 1e-5 * max(1.0, np.abs(want).max())
    assert np.all(state.download(np.float32, 0, W) == 0.0)                   # slot 0 was never touched
    w.free()
    state.free()


def test_smooth_cap_among_the_activations(cuda_backend):
    from zgml_b200 import DeviceOp, ExternBuffer, abi
    from zgml_b200.host.weights import WeightArena
    z = np.linspace(-40, 40, 101).astype(np.float32)
    got = run(cuda_backend, [DeviceOp.activation(0, 0, z.size, "softcap", 7.5)], [z.size], [(0, z)], 0, z.shape)
    assert np.abs(got - 7.5 * np.tanh(z.astype(np.float64) / 7.5)).max() < 1e-5
    r = np.random.default_rng(3)
    for M, N, K in ((1, 24, 64), (3, 17, 37), (40, 70, 50), (70, 96, 128)):      # one row, a few rows, the exact tile, the tensor-core product
        for wdt in (abi.W_F32, abi.W_BF16):
            u = np.ascontiguousarray(r.standard_normal((N, K)), dtype=np.float32).view(np.uint32) & np.uint32(0xFFFF0000)
            Wm = u.view(np.float32)
            x = (np.ascontiguousarray(r.standard_normal((M, K)) * 1.5, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
            A = WeightArena(wdt)
            ow = A.add("w", Wm)
            buf = A.upload(cuda_backend)
            want = 2.0 * np.tanh(x.astype(np.float64) @ Wm.astype(np.float64).T / 2.0)
            got = run(cuda_backend, [DeviceOp.linear(0, 1, 2, ow, M, N, K, wdt, act="softcap", act_param=2.0)], [M * N, M * K, buf.elems], [(1, x)], 0, (M, N), [ExternBuffer(2, buf)])
            assert np.abs(got - want).max() < 2e-5, (M, N, K, wdt)
            buf.free()


def test_malformed_ops_are_refused(cuda_backend):
    from zgml_b200 import DeviceOp, DeviceProgram, abi
    bad = [
        (DeviceOp.activation(0, 0, 8, "softcap", 0.0), [8]),                                                                         # a cap of zero
        (DeviceOp.linear(0, 1, 2, 0, 2, 4, 4, abi.W_F32, act="softcap"), [8, 8, 16]),                                                # the epilogue's cap without its parameter
        (DeviceOp.rotary(0, 1, 0, 2, 2, 6, 12, 6, 0.0, freqs=2, freqs_off=6), [24, 8, 8]),                                           # the table ends before dims / 2 frequencies
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 8, 4, 2, 2, 1, 8, 8, 16, 32, 32, 8, 1.0, dst_rs=20, dst_col=8), [80, 64, 256, 16]),      # heads leave the destination row
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 8, 4, 2, 2, 1, 8, 8, 16, 32, 32, 8, 1.0, sink=4, sink_off=7, sink_wdt=abi.W_F32), [64, 64, 256, 16, 8]),   # sinks past their buffer
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 8, 4, 2, 2, 1, 8, 8, 16, 32, 32, 8, 1.0, weights="sigmoid", sink=4, sink_wdt=abi.W_F32), [64, 64, 256, 16, 8]),   # a sink without a softmax
        (DeviceOp.cache_append(0, 1, 2, 0, 0, 4, 16, 16, 16, 8, norm_w=3, normed=16, wdt=abi.W_F32, norm_group=8, head_rot=10, rot_base=10.0), [128, 64, 16, 8]),   # more rotary dims than the head holds
        (DeviceOp.cache_append(0, 1, 2, 0, 0, 4, 16, 16, 16, 8, norm_w=3, normed=16, wdt=abi.W_F32, norm_group=0, head_rot=4, rot_base=10.0), [128, 64, 16, 16]),   # head rotary without heads
        (DeviceOp.delta_rule(0, 1, None, 2, 1, 3, 4, 5, 0, 8, 16, 0, 0, 0, 0, 2, 2, 2, 4, 4, 32, 0, 8, 32, abi.W_F32, 1e-5, 0.0, 1.0, gate_off=24, plain=True, decay_tau=0.0), [16, 64, 16, 32, 32, 8]),  # tempered decay without a temperature
        (DeviceOp.delta_rule(0, 1, None, 2, 1, 3, 4, 5, 0, 8, 16, 0, 0, 0, 0, 2, 2, 2, 4, 4, 32, 0, 8, 32, abi.W_F32, 1e-5, 0.0, 1.0, gate_off=24, plain=True, dst_rs=6), [16, 64, 16, 32, 32, 8]),      # heads wider than the destination row
        (DeviceOp.rg_lru(0, 1, 2, 3, 4, 5, 6, 0, 0, 4, 0, 0, 8, 16, 2, 8, 8, 16, 3, 6, 8, abi.W_F32), [16, 16, 32, 16, 32, 8, 8]),  # channels do not divide into gate blocks
        (DeviceOp.rg_lru(0, 1, 2, 3, 4, 5, 6, 0, 0, 4, 0, 0, 8, 16, 2, 8, 8, 16, 4, 8, 8, abi.W_F32, rate=0.0), [16, 16, 32, 16, 32, 8, 8]),   # no rate
    ]
    for i, (op, sizes) in enumerate(bad):
        assert cuda_backend.compile_program(DeviceProgram([op], sizes, [], [], [])) is None, i
