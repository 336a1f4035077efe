"""Host side of Pepevik without a GPU: configuration errors, state sizing, the shape of the lowering on a fake device, the
distance table, and properties of the float64 restatement that the GPU tests lean on (causality, the recurrences carried
across a cut, routing inside the best groups)."""
import json

import numpy as np
import pytest

import pepevik_reference as ref
from pepevik_models import as_f64, config, dense, moe, pair_layer, random_weights, ssm_layer


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
    import zgml_b200.host.pepevik as P
    import zgml_b200.host.state as S
    import zgml_b200.host.weights as Wt
    monkeypatch.setattr(Wt, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(S, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(P, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(P, "seq_state_elems", lambda op: 1024)          # the library's own state layout: any size will do here
    monkeypatch.setattr(P, "seq_scratch_elems", lambda op: 64)


STACK = config([ssm_layer(mlp=dense()), pair_layer(mlp=moe()), pair_layer(weights_of=1, mlp=moe()), ssm_layer(weights_of=0, mlp=dense()), pair_layer(heads=2, kv_heads=1, gru=6)])


def test_config_errors():
    from zgml_b200.host.pepevik import PepevikConfig
    cfg = PepevikConfig.from_dict(STACK)
    assert [L["weights"] for L in cfg.layers] == [0, 1, 1, 0, 4]
    for mutate in (lambda c: c.__setitem__("architecture", "Other"),
                   lambda c: c["layers"][0].__setitem__("type", "attention"),
                   lambda c: c["layers"][0]["mixer"].__setitem__("groups", 3),             # heads not a multiple
                   lambda c: c["layers"][0]["mixer"].__setitem__("norm_groups", 5),
                   lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3),
                   lambda c: c["layers"][1]["mixer"]["left"]["q_temp"].__setitem__("every", 0),
                   lambda c: c["layers"][2].__setitem__("weights_of", 2),                  # itself
                   lambda c: c["layers"][2].__setitem__("weights_of", 0),                  # another kind of layer
                   lambda c: c["layers"][4].__setitem__("weights_of", 2),                  # a layer without tensors of its own
                   lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9),
                   lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4),
                   lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 0),
                   lambda c: c["layers"][0]["mlp"].__setitem__("kind", "conv")):
        bad = json.loads(json.dumps(STACK))
        mutate(bad)
        with pytest.raises(ValueError):
            PepevikConfig.from_dict(bad)


def test_state_and_lowering_shape(fake_device):
    from zgml_b200 import abi
    from zgml_b200.host.pepevik import PepevikConfig, PepevikModel
    from zgml_b200.host.state import SequenceStatePool
    W = random_weights(STACK)
    m = PepevikModel(None, PepevikConfig.from_dict(STACK), lambda n: W[n], "bfloat16")
    assert sorted(k for k in m.buffers) == [-1, 0, 1, 4]                    # layers 2 and 3 have no tensors of their own
    specs = {s.name: s for s in m.state_specs(16, 100)}
    assert list(specs) == ["l0.ssm", "l0.tail", "l1.kv", "l1.gru", "l2.kv", "l2.gru", "l3.ssm", "l3.tail", "l4.kv", "l4.gru"]   # but states of their own
    assert specs["l1.kv"].elems == 100 * 2 * (8 + 12) and specs["l1.gru"].elems == 20 and specs["l0.tail"].elems == 2 * (4 * 6 + 2 * 2 * 10)
    assert specs["l0.ssm"].zero_on_acquire and specs["l0.tail"].zero_on_acquire and specs["l1.gru"].zero_on_acquire and not specs["l1.kv"].zero_on_acquire
    assert m.capacity(16, 100) == 100 and m.capacity(16, 10 ** 6) == STACK["max_positions"] and m.capacity(16, None) == STACK["max_positions"]
    pool = SequenceStatePool(None, list(specs.values()), 2)
    for T, head, rows in ((1, "last", 1), (16, "all", 16), (4, "none", 0)):
        lp = m.lower(T, head, pool)
        ops = lp.program.ops
        tags = [op.tag for op in ops]
        assert tags[0] == abi.OP_EMBED and ops[0].u.seq.n[3] == 1 and lp.logits_rows == rows and (lp.buf_logits is None) == (head == "none")
        assert tags.count(abi.OP_SSM_SCAN) == 2 and tags.count(abi.OP_CAUSAL_CONV) == 2 and tags.count(abi.OP_GATED_NORM) == 2
        assert tags.count(abi.OP_CACHED_ATTENTION) == 3 and tags.count(abi.OP_CACHE_APPEND) == 3 and tags.count(abi.OP_HEAD_NORM) == 0 and tags.count(abi.OP_MIN_GRU) == 3
        assert tags.count(abi.OP_ACTIVATION) == 0 and sum(op.tag == abi.OP_LINEAR and op.u.seq.n[6] == 1 for op in ops) == 2     # relu^2 rides in the up projection
        assert tags.count(abi.OP_MOE_FFN) == 2 and tags.count(abi.OP_ROUTE) == 2
        att = [op for op in ops if op.tag == abi.OP_CACHED_ATTENTION]
        assert all(op.u.seq.off[5] == abi.WEIGHTS_SIGMOID and op.u.seq.buf[5] != abi.NO_BUF and op.u.seq.off[6] == 100 for op in att)
        assert att[0].u.seq.buf[5] == att[1].u.seq.buf[5] != att[2].u.seq.buf[5]      # one distance table per set of weights
        assert att[0].u.seq.buf[2] != att[1].u.seq.buf[2]                               # but a cache per layer
        # every residual step rides in the Dynamic Tanh that opens the next sublayer, the pair's sum of two normed results too
        norms = [op for op in ops if op.tag == abi.OP_NORM]
        chained = [op for op in norms if op.u.seq.buf[4] != abi.NO_BUF]
        assert all(op.u.seq.n[4] == abi.NORM_DYNAMIC_TANH for op in chained)
        assert len(norms) == 1 + (9 if head != "none" else 8) and len(chained) == len(norms) - 1
        assert sum(op.u.seq.n[7] for op in norms) == (3 if head != "none" else 2)
        ext = [e.buf_idx for e in lp.program.externs]
        assert len(set(ext)) == len(ext) == 4 + 10 + 2                                 # weight arenas + state buffers + distance tables, each once


def test_distance_table():
    from zgml_b200.host.pepevik import distance_score_table
    r1, r2, pb = np.array([0.5, 0.25]), np.array([1.0, 0.125]), np.array([-1.0, 2.0])
    t = distance_score_table(r1, r2, pb, 50)
    assert t.shape == (2, 50) and t.dtype == np.float32
    assert np.allclose(t[:, 0], pb) and np.allclose(t[1, 8], 2.0 - 0.25 * np.log(2.0), atol=1e-6)
    d = np.arange(50)
    assert np.abs(t - (pb[:, None] - r1[:, None] * np.log(1.0 + r2[:, None] * d))).max() < 1e-6


def test_restatement_is_causal_and_carries_its_states():
    toks = np.random.default_rng(0).integers(0, STACK["vocab"], 30).tolist()
    W = as_f64(random_weights(STACK, seed=3, qk_gain=4.0))
    full, _ = ref.forward(STACK, W, toks)
    assert np.allclose(ref.forward(STACK, W, toks[:17])[0], full[:17], atol=1e-11)
    other = list(toks)
    other[0] = (other[0] + 1) % STACK["vocab"]
    assert np.abs(ref.forward(STACK, W, other)[0][-1] - full[-1]).max() > 1e-9          # the first token still reaches the last position
    assert ref.query_temperature(3, 0.5, 5) == 1.0 and np.isclose(ref.query_temperature(4, 0.5, 5), 1.0 + 0.5 * np.log(2.0))


def test_restatement_routing():
    W = {"p.router": np.eye(6), "p.correction": np.array([0.0, 0.0, 0.5, 0.0, 0.0, 0.0])}
    r = {"top": 2, "groups": {"count": 3, "keep": 1}}
    z = np.array([[3.0, 2.9, -1.0, 0.0, 2.0, 2.5]])                          # groups {0, 1} {2, 3} {4, 5}
    idx, w = ref.route(z, W, "p.", r)
    s = ref.sigmoid(z[0])
    assert idx.tolist() == [[0, 1]] and np.allclose(w, s[[0, 1]] / s[[0, 1]].sum())      # weights leave the correction out
    r["groups"]["keep"] = 2
    idx, _ = ref.route(z, W, "p.", r)
    assert idx.tolist() == [[0, 1]]
    W["p.correction"] = np.array([0.0, -1.0, 0.0, 0.0, 0.1, 0.0])
    idx, _ = ref.route(z, W, "p.", r)
    assert idx.tolist() == [[4, 0]]                                          # the correction decides the choice
    W["p.correction"] = np.full(6, -5.0)
    r["groups"]["keep"] = 1
    idx, _ = ref.route(z, W, "p.", r)
    assert idx.tolist() == [[0, 1]]                                          # negative choice scores: the dropped groups still lose


def test_restatement_recurrences():
    r = np.random.default_rng(5)
    W = {"p.z": r.standard_normal((3, 4)), "p.z.b": r.standard_normal(3), "p.x": r.standard_normal((3, 4)), "p.x.b": r.standard_normal(3),
         "p.g": r.standard_normal((3, 4)), "p.o": np.eye(3)}
    h = r.standard_normal((6, 4))
    out = ref.min_gru(h, W, "p.")
    z = ref.sigmoid(h @ W["p.z"].T + W["p.z.b"])
    u = h @ W["p.x"].T + W["p.x.b"]
    c = np.where(u >= 0, u + 0.5, ref.sigmoid(u))
    g = h @ W["p.g"].T
    assert np.allclose(out[0], z[0] * c[0] * ref.silu(g[0]))                 # the state starts at zero
    assert np.allclose(out[1], ((1 - z[1]) * z[0] * c[0] + z[1] * c[1]) * ref.silu(g[1]))
    x = r.standard_normal((5, 2))
    y = ref.causal_conv(x, np.array([[1.0, 2.0, 3.0], [0.0, 0.0, 1.0]]), np.array([0.5, 0.0]))
    assert np.allclose(y[0], [3 * x[0, 0] + 0.5, x[0, 1]]) and np.allclose(y[2, 0], x[0, 0] + 2 * x[1, 0] + 3 * x[2, 0] + 0.5)
