"""Host side of Setirax without a GPU: configuration errors, ring and state sizing, the shape of the lowering on a fake device,
the rotary frequency schedule, and properties of the float64 restatement that the GPU tests lean on (causality, windows, sinks,
the recurrences' first steps)."""
import json
import math

import numpy as np
import pytest

import setirax_reference as ref
from setirax_models import as_f64, config, dense, latent_layer, lru_layer, pair_layer, random_weights


class FakeBuffer:
    def __init__(self, be, nbytes, zero=True):
        self.nbytes = (int(nbytes) + 15) & ~15
        self.elems = self.nbytes // 4

    def upload(self, host, byte_offset=0):
        pass

    def fill_zero(self, byte_offset, nbytes):
        pass

    def free(self):
        pass


@pytest.fixture
def fake_device(monkeypatch):
    import zgml_b200.host.setirax as M
    import zgml_b200.host.state as S
    import zgml_b200.host.weights as Wt
    monkeypatch.setattr(Wt, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(S, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(M, "DeviceBuffer", FakeBuffer)


STACK = config([latent_layer(mlp=dense()), pair_layer(mlp=dense()), lru_layer(), latent_layer(weights_of=0, mlp=dense()), pair_layer(weights_of=1, mlp=dense()),
                lru_layer(width=10, blocks=2, conv=1, mlp=dense(ff=8))])


def test_config_errors():
    from zgml_b200.host.setirax import SetiraxConfig
    cfg = SetiraxConfig.from_dict(STACK)
    assert [L["weights"] for L in cfg.layers] == [0, 1, 2, 0, 1, 5] and cfg.logit_softcap == 6.0
    for mutate in (lambda c: c.__setitem__("architecture", "Other"),
                   lambda c: c["layers"][0].__setitem__("type", "attention"),
                   lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3),      # heads not a multiple
                   lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 5),
                   lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 10),  # more than the head holds
                   lambda c: c["layers"][1]["mixer"]["right"].__setitem__("tau", 0.0),
                   lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0),
                   lambda c: c["layers"][2]["mixer"].__setitem__("blocks", 5),                # width does not divide
                   lambda c: c["layers"][3].__setitem__("weights_of", 3),                     # itself
                   lambda c: c["layers"][3].__setitem__("weights_of", 1),                     # another kind of layer
                   lambda c: c["layers"][3].__setitem__("weights_of", 9),                     # no such layer
                   lambda c: c["layers"][3]["mixer"].__setitem__("kv_rank", 24),              # other tensor sizes than the layer whose weights it uses
                   lambda c: (c["layers"][0].__setitem__("weights_of", 3), c["layers"][3].__setitem__("weights_of", 0)),     # a circle
                   lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe")):
        bad = json.loads(json.dumps(STACK))
        mutate(bad)
        with pytest.raises(ValueError):
            SetiraxConfig.from_dict(bad)


def test_shared_weights_through_chains_with_constants_of_their_own():
    """A reference may lead through another layer that shares weights, may point forward, and the layer keeps its own window, scale
    and cap; only what sizes the tensors must agree."""
    from zgml_b200.host.setirax import SetiraxConfig
    c = json.loads(json.dumps(STACK))
    c["layers"][4]["weights_of"] = 1
    c["layers"].append(pair_layer(weights_of=4, window=3, softcap=0.0, tau=2.0, mlp=dense()))      # 6 -> 4 -> 1
    del c["layers"][3]["weights_of"]
    c["layers"][0]["weights_of"] = 3                                                                 # a reference forward: layer 0 runs with layer 3's tensors
    cfg = SetiraxConfig.from_dict(c)
    assert [L["weights"] for L in cfg.layers] == [3, 1, 2, 3, 1, 5, 1]
    assert cfg.layers[6]["mixer"]["left"]["mask"]["size"] == 3 and cfg.layers[1]["mixer"]["left"]["mask"]["size"] == 7


def test_state_and_lowering_shape(fake_device):
    from zgml_b200 import abi
    from zgml_b200.host.setirax import SetiraxConfig, SetiraxModel
    from zgml_b200.host.state import SequenceStatePool
    W = random_weights(STACK)
    m = SetiraxModel(None, SetiraxConfig.from_dict(STACK), lambda n: W[n], "bfloat16", has=lambda n: n in W)
    assert sorted(m.buffers) == [-1, 0, 1, 2, 5]                      # layers 3 and 4 have no tensors of their own
    assert not m.bounded_context
    specs = {s.name: s for s in m.state_specs(16, 100)}
    assert list(specs) == ["l0.latent", "l1.kv", "l1.tail", "l1.gla", "l2.tail", "l2.lru", "l3.latent", "l4.kv", "l4.tail", "l4.gla", "l5.lru"]   # but rings and states of their own
    assert specs["l0.latent"].elems == (9 - 1 + 16) * 20 and specs["l1.kv"].elems == (7 - 1 + 16) * 2 * (8 + 12)      # what the window reaches back plus one step
    assert specs["l1.tail"].elems == 2 * (4 * 8 + 2 * (8 + 12)) and specs["l1.gla"].elems == 2 * 6 * 10 and specs["l2.tail"].elems == 3 * 24 and specs["l5.lru"].elems == 10
    assert not specs["l0.latent"].zero_on_acquire and not specs["l1.kv"].zero_on_acquire
    assert all(specs[n].zero_on_acquire for n in ("l1.tail", "l1.gla", "l2.tail", "l2.lru"))
    pool = SequenceStatePool(None, list(specs.values()), 2)
    for T, head, rows in ((1, "last", 1), (16, "all", 16), (4, "none", 0)):
        lp = m.lower(T, head, pool)
        ops = lp.program.ops
        tags = [op.tag for op in ops]
        assert tags[0] == abi.OP_EMBED and lp.logits_rows == rows and (lp.buf_logits is None) == (head == "none")
        assert tags.count(abi.OP_CACHED_ATTENTION) == 4 and tags.count(abi.OP_CACHE_APPEND) == 4 and tags.count(abi.OP_HEAD_LINEAR) == 2 * 2 + 2
        assert tags.count(abi.OP_DELTA_RULE) == 2 and tags.count(abi.OP_ROTARY) == 0 and tags.count(abi.OP_RG_LRU) == 2 and tags.count(abi.OP_CAUSAL_CONV) == 2 + 2
        assert tags.count(abi.OP_ACTIVATION) == 0 and sum(op.tag == abi.OP_LINEAR and op.u.seq.n[6] == abi.ACTIVATIONS["relu2"] + 1 for op in ops) == 5
        app = [op for op in ops if op.tag == abi.OP_CACHE_APPEND]
        assert [op.u.seq.n[10] for op in app] == [0, 6, 0, 6] and abi.NO_BUF not in (app[1].u.seq.buf[4], app[3].u.seq.buf[4])      # rotary rides in the append, from the layer's table
        att = [op for op in ops if op.tag == abi.OP_CACHED_ATTENTION]
        assert [op.u.seq.buf[6] != abi.NO_BUF for op in att] == [True, False, True, False]       # sinks on the latent layers only
        assert [op.u.seq.f[1] for op in att] == [0.0, 5.0, 0.0, 5.0] and all(op.u.seq.off[3] == abi.MASK_WINDOW for op in att)
        assert att[0].u.seq.buf[2] != att[2].u.seq.buf[2] and att[0].u.seq.buf[6] == att[2].u.seq.buf[6]     # a ring per layer, one set of weights
        rule = [op for op in ops if op.tag == abi.OP_DELTA_RULE]
        assert all(op.u.seq.n[10] == abi.DELTA_PLAIN | abi.DELTA_SIGMOID_DECAY | abi.DELTA_SILU_GATE | abi.DELTA_OUT_SCALE and op.u.seq.buf[2] == abi.NO_BUF for op in rule)
        # both branches of a pair write into one row, which one product with the stacked output weights turns into their scaled sum
        assert att[1].u.seq.buf[0] == rule[0].u.seq.buf[0] and att[1].u.seq.n[10] == rule[0].u.seq.n[11] == 4 * 12 + 2 * 10 and rule[0].u.seq.n[12] == 4 * 12
        assert abs(att[1].u.seq.f[2] - 0.7) < 1e-6 and abs(rule[0].u.seq.f[4] - 1.3) < 1e-6
        # the norm sits on every sublayer's result and carries the residual; nothing is normed before a sublayer
        norms = [op for op in ops if op.tag == abi.OP_NORM]
        assert len(norms) == 6 + 5 and all(op.u.seq.buf[3] != abi.NO_BUF for op in norms)
        assert [op.u.seq.buf[4] != abi.NO_BUF for op in norms] == [False] * 10 + [head != "none"]     # the final norm rides in the last residual step
        if head != "none":      # the head is the embedding table, capped in the product's epilogue
            assert ops[-1].tag == abi.OP_LINEAR and ops[-1].u.seq.n[6] == abi.ACTIVATIONS["softcap"] + 1 and ops[-1].u.seq.f[0] == 6.0 and ops[-1].u.seq.off[0] == m.arenas[-1].off["embed"]
        ext = [e.buf_idx for e in lp.program.externs]
        assert len(set(ext)) == len(ext) == 5 + 11 + 2                             # weight arenas + state buffers + a frequency table per turning layer, each once


def test_layers_without_a_window_keep_every_position(fake_device):
    from zgml_b200.host.setirax import SetiraxConfig, SetiraxModel
    layer = latent_layer()
    del layer["mixer"]["mask"]
    cfg = config([layer])
    W = random_weights(cfg)
    m = SetiraxModel(None, SetiraxConfig.from_dict(cfg), lambda n: W[n], "float32", has=lambda n: n in W)
    assert m.bounded_context and m.capacity(16, 100) == 100 and m.capacity(16, None) == 4096
    assert m.state_specs(16, 100)[0].elems == 100 * 20


def test_rotary_frequency_schedule():
    from zgml_b200.host.setirax import rotary_frequencies
    plain = rotary_frequencies({"base": 100.0, "dims": 8})
    assert plain.dtype == np.float32 and np.allclose(plain, [1.0, 100.0 ** -0.25, 0.1, 100.0 ** -0.75])
    sc = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 40}
    got = rotary_frequencies({"base": 50.0, "dims": 6, "scaling": sc})
    want = []
    for i in range(3):
        f = 50.0 ** (-2.0 * i / 6)
        wl = 2 * math.pi / f
        if wl < 40 / 3.0:
            want.append(f)
        elif wl > 40 / 1.0:
            want.append(f / 4.0)
        else:
            s = (40 / wl - 1.0) / 2.0
            want.append((1 - s) * f / 4.0 + s * f)
    assert np.allclose(got, want, rtol=1e-6)
    assert got[0] == plain[0] and want[1] not in (50.0 ** (-1 / 3), 50.0 ** (-1 / 3) / 4.0) and np.isclose(got[2], 50.0 ** (-2 / 3) / 4.0)    # kept, blended, slowed
    assert np.allclose(got, ref.rotary_frequencies({"base": 50.0, "dims": 6, "scaling": sc}), rtol=1e-6)


def test_restatement_is_causal_windowed_and_carries_its_states():
    toks = np.random.default_rng(0).integers(0, STACK["vocab"], 30).tolist()
    W = as_f64(random_weights(STACK, seed=3, qk_gain=4.0))
    full = ref.forward(STACK, W, toks)
    assert np.allclose(ref.forward(STACK, W, toks[:17]), full[:17], atol=1e-11)
    other = list(toks)
    other[0] = (other[0] + 1) % STACK["vocab"]
    assert np.abs(ref.forward(STACK, W, other)[-1] - full[-1]).max() > 1e-9            # through the recurrent states the first token still reaches the last position
    only = config([latent_layer(window=4)])
    Wl = as_f64(random_weights(only, seed=1))
    a, b = ref.forward(only, Wl, toks), ref.forward(only, Wl, other)
    assert np.abs(a[3] - b[3]).max() > 1e-9 and np.abs(a[4:] - b[4:]).max() == 0.0      # position 3 is the last one whose window holds token 0


def test_restatement_attention_and_sink():
    r = np.random.default_rng(2)
    q, k, v = r.standard_normal((5, 2, 3)), r.standard_normal((5, 1, 3)), r.standard_normal((5, 1, 4))
    out = ref.window_softmax_attention(q, k, v, 0.5, 2, softcap=1.5, sink=np.array([0.3, -50.0]))
    s = 1.5 * np.tanh(np.array([k[2, 0] @ q[3, 0], k[3, 0] @ q[3, 0]]) * 0.5 / 1.5)
    w = np.exp(s) / (np.exp(s).sum() + math.exp(0.3))                                    # the sink is neither scaled nor capped and has no value
    assert np.allclose(out[3, 0], w @ v[2:4, 0])
    s1 = 1.5 * np.tanh(np.array([k[2, 0] @ q[3, 1], k[3, 0] @ q[3, 1]]) * 0.5 / 1.5)
    assert np.allclose(out[3, 1], (np.exp(s1) / np.exp(s1).sum()) @ v[2:4, 0])           # a sink far below the scores weighs nothing
    assert np.allclose(out[0, 0], v[0, 0] * math.exp(s0 := 1.5 * math.tanh(k[0, 0] @ q[0, 0] * 0.5 / 1.5)) / (math.exp(s0) + math.exp(0.3)))


def test_restatement_recurrences():
    r = np.random.default_rng(5)
    m = {"width": 4, "blocks": 2}
    W = {"p.y": r.standard_normal((4, 3)), "p.y.b": r.standard_normal(4), "p.x": r.standard_normal((4, 3)), "p.x.b": r.standard_normal(4),
         "p.conv": np.array([[0.0, 1.0]] * 4), "p.conv.b": np.zeros(4), "p.ra": r.standard_normal((2, 2, 2)), "p.ra.b": r.standard_normal((2, 2)),
         "p.ri": r.standard_normal((2, 2, 2)), "p.ri.b": r.standard_normal((2, 2)), "p.lam": r.standard_normal(4), "p.o": np.eye(4)}
    h = r.standard_normal((3, 3))
    out = ref.rglru(h, W, "p.", m)
    u = h @ W["p.x"].T + W["p.x.b"]
    y = ref.gelu_tanh(h @ W["p.y"].T + W["p.y.b"])
    gate = lambda w, b, t: ref.sigmoid(np.concatenate([w[0] @ u[t, :2], w[1] @ u[t, 2:]]) + b.ravel())
    a0 = np.exp(-8.0 * gate(W["p.ra"], W["p.ra.b"], 0) * ref.softplus(W["p.lam"]))
    s0 = np.sqrt(1 - a0 ** 2) * gate(W["p.ri"], W["p.ri.b"], 0) * u[0]                  # the first token starts from zero like every other
    assert np.allclose(out[0], s0 * y[0])
    a1 = np.exp(-8.0 * gate(W["p.ra"], W["p.ra.b"], 1) * ref.softplus(W["p.lam"]))
    assert np.allclose(out[1], (a1 * s0 + np.sqrt(1 - a1 ** 2) * gate(W["p.ri"], W["p.ri.b"], 1) * u[1]) * y[1])
    g = {"heads": 1, "dim": 2, "vdim": 2, "tau": 2.0}
    Wg = {"p.q": r.standard_normal((2, 3)), "p.k": r.standard_normal((2, 3)), "p.v": r.standard_normal((2, 3)), "p.g": r.standard_normal((2, 3)),
          "p.a1": r.standard_normal((1, 3)), "p.a2": r.standard_normal((2, 1)), "p.a2.b": r.standard_normal(2), "p.norm": np.ones(2), "p.o": np.eye(2)}
    out = ref.gated_linear_attention(h, Wg, "p.", g, 0.0)
    q, k, v = h @ Wg["p.q"].T / math.sqrt(2), h @ Wg["p.k"].T, h @ Wg["p.v"].T
    alpha = ref.sigmoid((h @ Wg["p.a1"].T) @ Wg["p.a2"].T + Wg["p.a2.b"]) ** 0.5
    S1 = alpha[1][:, None] * np.outer(k[0], v[0]) + np.outer(k[1], v[1])                # the decay scales the rows of the key channels
    o1 = S1.T @ q[1]
    gt = h[1] @ Wg["p.g"].T
    assert np.allclose(out[1], o1 / np.sqrt(np.mean(o1 ** 2)) * gt * ref.sigmoid(gt))
    x = r.standard_normal((5, 2))
    c = ref.causal_conv(x, np.array([[1.0, 2.0, 3.0], [0.0, 0.0, 1.0]]), np.array([0.5, 0.0]))
    assert np.allclose(c[0], [3 * x[0, 0] + 0.5, x[0, 1]]) and np.allclose(c[2, 0], x[0, 0] + 2 * x[1, 0] + 3 * x[2, 0] + 0.5)
