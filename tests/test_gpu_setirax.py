"""Setirax on the CUDA backend against the float64 restatement (tests/setirax_reference.py): every mechanism alone, the stream
after every layer, whole prompts, token-by-token decoding through the rings and the recurrent states, prompts cut into portions
down to two tokens, interleaved requests in several slots, slot reuse, the edges of every window in prompts and decoded (with
controls that are off by one), the sink, a key far back found by construction, the first tokens of a sequence, long decoding
over rings that wrap, many shapes, and greedy generation through the registry's entry point and the trace replayer."""
import copy
import json
import os
import subprocess

import numpy as np
import pytest

import setirax_reference as ref
from setirax_models import as_f64, config, dense, latent_layer, lru_layer, pair_layer, random_weights

pytestmark = pytest.mark.gpu

TOL = 2e-4   # of the logits' scale; f32 accumulation against float64


def tol(dtype):
    """A bfloat16 session rounds the activations that enter a tensor-core matmul (steps of more than 8 tokens) to bf16."""
    return TOL if dtype == "float32" else 3e-2


def open_model(be, cfg, W, dtype="float32", n_slots=1, max_chunk=16, keep_layers=False, max_context=None):
    from zgml_b200.host.session import SequenceSession
    from zgml_b200.host.setirax import SetiraxConfig, SetiraxModel
    model = SetiraxModel(be, SetiraxConfig.from_dict(cfg), lambda n: W[n], dtype, has=lambda n: n in W)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, keep_layers=keep_layers, max_context=max_context)


def close(s):
    s.close()
    s.model.close()


def rel(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want)) / (np.max(np.abs(want)) + 1e-30))


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def forward(cfg, W, toks):
    return ref.forward(cfg, as_f64(W), toks, return_layers=True)


MIXED = config([latent_layer(mlp=dense()), pair_layer(mlp=dense(ff=24)), lru_layer(), latent_layer(weights_of=0, mlp=dense()),
                pair_layer(heads=3, kv_heads=3, dim=6, vdim=4, conv=2, rot_dims=2, window=5, r_heads=1, r_dim=5, r_vdim=7, tau=1.0, mlp=dense(ff=9)),
                pair_layer(weights_of=1, mlp=dense(ff=24)), lru_layer(weights_of=2), lru_layer(width=10, blocks=10, conv=2, mlp=dense(ff=12))])


# ── each mechanism alone (a one-layer model without a feed-forward isolates its mixer) ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("layer", [
    latent_layer(),
    latent_layer(heads=1, dim=16, vdim=4, rank=6, window=40),                     # one head; a window longer than the prompt's first steps
    latent_layer(heads=5, dim=3, vdim=7, rank=70, window=1),                      # a query sees itself and the sink only
    latent_layer(heads=2, dim=12, vdim=12, rank=12, window=33, scale=0.5),        # every size equal; a window across a 32-key block
    latent_layer(heads=4, dim=68, vdim=36, rank=132, window=20),
    pair_layer(),
    pair_layer(heads=6, kv_heads=2, dim=10, vdim=5, conv=1, rot_dims=10, window=12, scaling=None),     # three heads per key head, one tap, every dim turns, plain schedule
    pair_layer(heads=2, kv_heads=1, dim=16, vdim=16, conv=5, rot_dims=4, softcap=0.0, window=3, r_heads=3, r_dim=4, r_vdim=4, tau=16.0),
    pair_layer(heads=1, kv_heads=1, dim=36, vdim=68, conv=2, rot_dims=36, base=10000.0, window=50, r_heads=1, r_dim=40, r_vdim=36, tau=0.5,
               scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}),
    pair_layer(heads=4, kv_heads=4, dim=8, vdim=8, softcap=1.0, scale=0.25, window=64, r_heads=4, r_dim=16, r_vdim=20, left_scale=1.0, right_scale=1.0),
    lru_layer(),
    lru_layer(width=32, blocks=1, conv=1),                                        # one block: a full gate matrix; one tap: no carried inputs
    lru_layer(width=21, blocks=21, conv=2),                                       # blocks of one channel: scalar gates
    lru_layer(width=130, blocks=2, conv=6),
], ids=["latent", "latent-1head", "latent-window1", "latent-equal", "latent-wide", "pair", "pair-grouped-1tap", "pair-nocap", "pair-wide", "pair-mha", "lru", "lru-1block",
        "lru-scalar-gates", "lru-wide"])
def test_mixer_alone(cuda_backend, layer, dtype):
    cfg = config([layer], width=40, vocab=61)
    W = random_weights(cfg, seed=5, qk_gain=4.0)
    toks = tokens(cfg, 75)
    want, stream = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64, keep_layers=True)
    got = s.feed("a", toks, range(75))
    if dtype == "float32":
        assert rel(s.layer_streams(64, "all")[0], stream[0][:64]) < TOL
    assert rel(got, want) < tol(dtype)
    close(s)


@pytest.mark.parametrize("silent", ["left", "right"])
def test_branches_of_the_pair_alone(cuda_backend, silent):
    """With the scale of one branch at zero the layer is the other branch alone: the windowed attention, or the gated linear
    attention; prompt and token by token."""
    layer = pair_layer(left_scale=0.0 if silent == "left" else 0.8, right_scale=0.0 if silent == "right" else 1.7)
    cfg = config([layer], width=32, vocab=40)
    W = random_weights(cfg, seed=21)
    toks = tokens(cfg, 30)
    want, stream = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True, n_slots=2)
    assert rel(s.feed("a", toks, range(30))[:16], want[:16]) < TOL
    assert rel(s.layer_streams(16, "all")[0], stream[0][:16]) < TOL
    decoded = np.concatenate([s.feed("d", [t], [0]) for t in toks])
    assert rel(decoded, want) < TOL
    close(s)


@pytest.mark.parametrize("mlp", [dense(), dense(ff=7), dense(ff=300), None], ids=["dense", "dense-7", "dense-300", "none"])
def test_feed_forward(cuda_backend, mlp):
    """The stream after the layer is compared too, so a fault in the activation or a bias cannot hide behind the final norm."""
    cfg = config([lru_layer(width=8, blocks=2, conv=2, mlp=mlp)], width=36, vocab=50, logit_softcap=0.0)
    W = random_weights(cfg, seed=9)
    toks = tokens(cfg, 19)
    want, stream = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True)
    got = s.feed("a", toks[:16], range(16))
    assert rel(s.layer_streams(16, "all")[0], stream[0][:16]) < TOL
    assert rel(got, want[:16]) < TOL
    close(s)


def test_logit_cap(cuda_backend):
    """A cap well inside the logits' range bends most of them; without the key there is no cap."""
    for cap in (1.5, 0.0):
        cfg = config([lru_layer(mlp=dense())], logit_softcap=cap)
        if not cap:
            del cfg["logit_softcap"]
        W = random_weights(cfg, seed=3)
        toks = tokens(cfg, 12)
        want = ref.forward(cfg, as_f64(W), toks)
        assert (np.abs(want).max() <= 1.5) == bool(cap)
        s = open_model(cuda_backend, cfg, W, "float32")
        assert rel(np.concatenate([s.feed("a", toks[:9], range(9))] + [s.feed("a", [t], [0]) for t in toks[9:]]), want) < TOL
        close(s)


def test_layer_streams_of_a_mixed_stack(cuda_backend):
    """Layers that run with another layer's weights keep rings and states of their own."""
    W = random_weights(MIXED, seed=2)
    toks = tokens(MIXED, 16)
    want, stream = forward(MIXED, W, toks)
    s = open_model(cuda_backend, MIXED, W, "float32", keep_layers=True)
    got = s.feed("a", toks, range(16))
    layers = s.layer_streams(16, "all")
    assert len(layers) == len(MIXED["layers"])
    for i in range(len(MIXED["layers"])):
        assert rel(layers[i], stream[i]) < TOL, f"layer {i}"
    assert rel(got, want) < TOL
    close(s)


def test_shared_weights_with_constants_of_their_own(cuda_backend):
    """Layers that run with another layer's tensors keep their own window, cap, scales, temperature and rotary schedule; a
    reference may lead through a layer that itself shares weights, and may point forward."""
    layers = [pair_layer(weights_of=2, window=12, base=500.0, scaling=None, mlp=dense()),
              pair_layer(weights_of=0, window=3, softcap=0.0, tau=2.0, scale=0.5, left_scale=1.0, mlp=dense()),
              pair_layer(mlp=dense()), latent_layer(mlp=dense()), latent_layer(weights_of=3, window=4, scale=0.9, mlp=dense())]
    cfg = config(layers)
    direct = copy.deepcopy(cfg)
    direct["layers"][1]["weights_of"] = 2                   # what the chain 1 -> 0 -> 2 comes to
    W = random_weights(cfg, seed=31, qk_gain=2.0)
    toks = tokens(cfg, 40)
    want, stream = forward(direct, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True)
    got = np.concatenate([s.feed("a", toks[:32], range(32))] + [s.feed("a", [t], [0]) for t in toks[32:]])
    layers_got = s.layer_streams(32, "all")
    for i in range(len(layers)):
        assert rel(layers_got[i], stream[i][:32]) < TOL, f"layer {i}"
    assert rel(got, want) < TOL
    close(s)


# ── prefill against decoding, portions, first tokens ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_prefill_equals_token_by_token(cuda_backend, dtype):
    W = random_weights(MIXED, seed=3, qk_gain=3.0)
    toks = tokens(MIXED, 40)
    want, _ = forward(MIXED, W, toks)
    s = open_model(cuda_backend, MIXED, W, dtype, n_slots=2)
    whole = s.feed("whole", toks, range(40))
    single = np.concatenate([s.feed("single", [t], [0]) for t in toks])
    assert rel(whole, want) < tol(dtype) and rel(single, want) < TOL     # single tokens take the exact row kernels in both formats
    close(s)


@pytest.mark.parametrize("cuts", [[2] * 20, [1, 2, 3, 5, 7, 9, 13], [37, 2, 1], [16, 16, 8], [3, 37]], ids=["twos", "growing", "long-then-short", "menu", "short-then-long"])
def test_portions(cuda_backend, cuts):
    """However a prompt is cut — inside a window, inside a convolution's reach, two tokens at a time — the logits stay the same."""
    W = random_weights(MIXED, seed=4, qk_gain=3.0)
    toks = tokens(MIXED, 40)
    want, _ = forward(MIXED, W, toks)
    s = open_model(cuda_backend, MIXED, W, "float32", max_chunk=32)
    got, at = [], 0
    for n in cuts:
        got.append(s.feed("a", toks[at:at + n], range(n)))
        at += n
    assert at == 40 and rel(np.concatenate(got), want) < TOL
    close(s)


def test_first_tokens(cuda_backend):
    """Position 0 alone (zeros before the convolutions' start, empty states, one visible key beside the sink), then positions 1
    and 2 one by one; then the three as one step in a slot that was used before."""
    W = random_weights(MIXED, seed=6)
    toks = tokens(MIXED, 3)
    want, _ = forward(MIXED, W, toks)
    s = open_model(cuda_backend, MIXED, W, "float32")
    got = np.concatenate([s.feed("a", [t], [0]) for t in toks])
    assert rel(got, want) < TOL
    s.release("a")
    assert rel(s.feed("b", toks, [0, 1, 2]), want) < TOL
    close(s)


# ── requests side by side, slots ──
def test_interleaved_requests_and_slot_reuse(cuda_backend):
    W = random_weights(MIXED, seed=7, qk_gain=2.0)
    reqs = {"a": tokens(MIXED, 29, 1), "b": tokens(MIXED, 11, 2), "c": tokens(MIXED, 40, 3)}
    want = {k: forward(MIXED, W, v)[0] for k, v in reqs.items()}
    s = open_model(cuda_backend, MIXED, W, "float32", n_slots=2)
    got = {k: [] for k in reqs}
    # a and b advance in turns, in unequal portions, inside ONE step call each time
    plan = [(("a", 9), ("b", 2)), (("b", 5), ("a", 1)), (("a", 19), ("b", 4))]
    at = {k: 0 for k in reqs}
    for step in plan:
        entries = [{"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))} for k, n in step]
        last = step is plan[-1]
        for (k, n), rows in zip(step, s.step(entries, end=["a", "b"] if last else [])):
            got[k].append(rows)
            at[k] += n
    for k in "ab":
        assert rel(np.concatenate(got[k]), want[k]) < TOL, k
    # c takes a slot that held another sequence: nothing of it may leak (recurrent states and convolution inputs are cleared,
    # the rings are masked by position)
    assert not s.pool.live()
    assert rel(s.feed("c", reqs["c"], range(40)), want["c"]) < TOL
    close(s)


# ── what a query must and must not see ──
@pytest.mark.parametrize("layer,key", [(latent_layer(heads=2, dim=8, vdim=8, rank=12, window=11), None), (pair_layer(heads=2, kv_heads=1, window=11, right_scale=0.0, scale=1.5), "left")],
                         ids=["latent", "left"])
def test_window_edges_in_prompt_and_decoding(cuda_backend, layer, key):
    """Sharp attention weights and a window of 11: the device agrees with the restatement at every position, as a prompt and
    decoded, and differs from restatements whose window is one key longer or shorter (so that a test passing with a window
    that is off by one is impossible)."""
    cfg = config([layer], width=32, vocab=40)
    W = random_weights(cfg, seed=8, qk_gain=8.0)
    toks = tokens(cfg, 48)
    want, _ = forward(cfg, W, toks)
    for delta in (-1, 1):
        other = copy.deepcopy(cfg)
        m = other["layers"][0]["mixer"]
        (m[key] if key else m)["mask"]["size"] += delta
        control, _ = forward(other, W, toks)
        first = 11 + min(delta, 0)                           # the first position whose window differs
        assert np.abs(control[:first] - want[:first]).max() < 1e-9
        assert np.abs(control[first:] - want[first:]).max() > 1e-2 * np.abs(want).max()
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=32)
    prompt = s.feed("p", toks, range(48))
    decoded = np.concatenate([s.feed("d", toks[:9], range(9))] + [s.feed("d", [t], [0]) for t in toks[9:]])
    assert rel(prompt, want) < TOL and rel(decoded, want) < TOL
    close(s)


def test_sink(cuda_backend):
    """Sinks that weigh about as much as the keys: a restatement without them is far away, the device is not.  One head's sink is
    very negative (it weighs nothing), another's dominates."""
    cfg = config([latent_layer(heads=3, dim=8, vdim=8, rank=10, window=6)], width=32, vocab=40)
    W = random_weights(cfg, seed=11, qk_gain=2.0)
    W["l0.mix.sink"][:] = np.array([-30.0, 1.0, 6.0], np.float32)
    toks = tokens(cfg, 20)
    want, _ = forward(cfg, W, toks)
    Wn = dict(W)
    Wn["l0.mix.sink"] = np.full(3, -1e4, np.float32)
    assert np.abs(forward(cfg, Wn, toks)[0] - want).max() > 5e-2 * np.abs(want).max()
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2)
    assert rel(s.feed("p", toks, range(20)), want) < TOL
    assert rel(np.concatenate([s.feed("d", [t], [0]) for t in toks]), want) < TOL
    close(s)


def test_far_key_among_hundreds(cuda_backend):
    """The last query of a latent-attention layer is made to weigh one early position among 300 and hardly any other.  Without
    positions a score depends on the two tokens alone, so the pair of token ids (and the head) whose score stands out most
    against every other key token is found from the weights; that head's queries are then scaled up, the key token is placed once,
    far back, the query token last.  Changing the far token must move the restatement's last logits, and the device must agree with
    the restatement, in a prompt and with the last tokens decoded; the window is 20 keys longer than the distance."""
    n, far = 300, 4
    cfg = config([latent_layer(heads=2, dim=8, vdim=8, rank=12, window=n - far + 20)], width=32, vocab=40)
    W = random_weights(cfg, seed=12)
    m = cfg["layers"][0]["mixer"]
    H, dim = m["heads"], m["dim"]
    Wd = as_f64(W)
    x = Wd["embed"]                                          # [vocab, width]: the mixer's input of every token id (the first layer reads the embedding itself)
    q = (x @ Wd["l0.mix.q"].T).reshape(-1, H, dim)
    c = ref.rms_norm(x @ Wd["l0.mix.dkv"].T, Wd["l0.mix.dkv.norm"], cfg["norm"]["eps"])
    k = (c @ Wd["l0.mix.uk"].T).reshape(-1, H, dim)
    S = np.einsum("ahd,bhd->hab", q, k) * m["scale"]
    margin = np.full(S.shape, -np.inf)
    for b in range(S.shape[2]):
        margin[:, :, b] = S[:, :, b] - np.delete(S, b, axis=2).max(axis=2)
    hd, a_tok, b_tok = np.unravel_index(np.argmax(margin), margin.shape)
    gain = np.float32(2.0 ** np.ceil(np.log2(12.0 / margin[hd, a_tok, b_tok])))      # the far key leads every other by 12 or more: a power of two keeps the weights bfloat16
    W["l0.mix.q"][hd * dim:(hd + 1) * dim] *= gain
    W["l0.mix.sink"][:] = 0.0
    pool = [t for t in range(cfg["vocab"]) if t != b_tok]
    toks = [pool[i] for i in np.random.default_rng(1).integers(0, len(pool), n)]
    toks[far], toks[-1] = int(b_tok), int(a_tok)
    want, _ = forward(cfg, W, toks)
    moved = list(toks)
    moved[far] = pool[0]
    assert np.abs(forward(cfg, W, moved)[0][-1] - want[-1]).max() > 1e-2 * np.abs(want).max(), "the construction lost its far key"
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=64)
    assert rel(s.feed("p", toks, range(n)), want) < TOL
    s.feed("d", toks[:n - 5], [])
    decoded = np.concatenate([s.feed("d", [t], [0]) for t in toks[n - 5:]])
    assert rel(decoded, want[n - 5:]) < TOL
    close(s)


@pytest.mark.parametrize("layer", [latent_layer(heads=4, dim=16, vdim=16, rank=132, window=260), pair_layer(heads=8, kv_heads=1, dim=4, vdim=4, rot_dims=4, window=200, scale=0.5),
                                   pair_layer(heads=2, kv_heads=2, dim=88, vdim=72, rot_dims=64, window=129, scale=0.1)], ids=["latent-wide", "8-per-group", "88"])
def test_long_windows_and_split_decoding(cuda_backend, layer):
    """Windows beyond one key tile of the prompt kernel (64) and one share of the decoding kernel (32), key and value sizes beyond
    one slice, and windows long enough that single-token steps deal their keys to several CTAs whose shares are merged (with the
    sink, where there is one)."""
    cfg = config([layer], width=48, vocab=50)
    W = random_weights(cfg, seed=18, qk_gain=3.0)
    n = 300
    toks = tokens(cfg, n)
    want, _ = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=128)
    assert rel(s.feed("p", toks, range(n)), want) < TOL
    s.feed("d", toks[:n - 12], [])
    decoded = np.concatenate([s.feed("d", toks[i:i + 1], [0]) for i in range(n - 12, n - 4)] + [s.feed("d", toks[n - 4:], range(4))])
    assert rel(decoded, want[n - 12:]) < TOL
    close(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_steps_expand_the_latent(cuda_backend, dtype):
    """Steps of 128 tokens run a latent layer in the expanded form: keys and values per head from one product over the ring's rows of
    the sequence's slot, then multi-head attention over them.  Sharp softmaxes, sinks, a ring of 99 + 128 rows that wraps, the second
    slot (after a request that left other latents there), steps that start anywhere; the shorter steps and single tokens that follow
    run absorbed over the same ring.  The float32 session is made to expand too, so the comparison is exact."""
    cfg = config([latent_layer(heads=3, dim=16, vdim=24, rank=64, window=100, mlp=dense()), lru_layer(), latent_layer(heads=3, dim=16, vdim=24, rank=64, window=100, weights_of=0, mlp=dense())],
                 width=64, vocab=50)
    W = random_weights(cfg, seed=29, qk_gain=4.0)
    n = 470
    toks = tokens(cfg, n)
    want, _ = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, dtype, n_slots=2, max_chunk=128)
    s.model.expand_float32 = True
    s.feed("first", toks[:3], [])                            # takes slot 0 and keeps it
    s.feed("other", toks[50:300], [])                        # leaves its latents in slot 1
    s.release("other")
    got = np.concatenate([s.feed("a", toks[:5], range(5)), s.feed("a", toks[5:460], range(455))] + [s.feed("a", [t], [0]) for t in toks[460:]])   # 4 + 1, then 128 x 3 + 64 + 4 + 2 + 1
    assert s.pool.slot("a") == 1
    tags = [op.tag for op in s.program(128, "all")[0].program.ops]
    from zgml_b200 import abi
    assert tags.count(abi.OP_HEAD_LINEAR) == 1 and abi.OP_HEAD_LINEAR in [op.tag for op in s.program(64, "all")[0].program.ops]      # only the recurrent block's gates are left at 128
    if dtype == "float32":
        assert rel(got, want) < TOL
    else:
        err = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
        assert np.median(err) < 3e-2 and np.mean(err < 6e-2) > 0.9
    close(s)


def test_long_steps_walk_segments_side_by_side(cuda_backend):
    """Steps of 256 tokens: the recurrent unit cuts them into 64 segments walked side by side and the gated linear attention
    takes its prepared walk; the states they leave must carry on into smaller steps and single tokens, in a slot that is not the
    first, after a request that used the same slot before."""
    cfg = config([lru_layer(width=70, blocks=5, conv=4, mlp=dense()), pair_layer(r_heads=3, r_dim=20, r_vdim=36, window=30, mlp=dense()), lru_layer(width=70, blocks=5, conv=4, weights_of=0, mlp=dense())],
                 width=48, vocab=50)
    W = random_weights(cfg, seed=23)
    n = 600
    toks = tokens(cfg, n)
    want, _ = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=256)
    s.feed("first", toks[:5], [])                           # takes slot 0 and keeps it
    s.feed("other", toks[100:400], [])                      # leaves its states in slot 1
    s.release("other")
    got = np.concatenate([s.feed("a", toks[:570], range(570))] + [s.feed("a", [t], [0]) for t in toks[570:]])   # 256 + 256 + 32 + 16 + 8 + 2, then single tokens
    assert s.pool.slot("a") == 1
    assert rel(got, want) < TOL
    close(s)


def test_long_decoding_over_rings_that_wrap(cuda_backend):
    """150 decoded tokens through every kind of state: rings of window - 1 + 4 rows that wrap a dozen times, the matrix and
    channel states, the convolutions' inputs."""
    cfg = config([latent_layer(window=9, mlp=dense()), pair_layer(window=7, mlp=dense()), lru_layer(), latent_layer(window=9, weights_of=0, mlp=dense()),
                  pair_layer(window=7, weights_of=1, mlp=dense())])
    W = random_weights(cfg, seed=13, qk_gain=3.0)
    toks = tokens(cfg, 160)
    want, _ = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=4)
    assert s.pool.buffers["l0.latent"].elems == (9 - 1 + 4) * 20
    got = np.concatenate([s.feed("a", toks[:10], range(10))] + [s.feed("a", [t], [0]) for t in toks[10:]])
    assert rel(got, want) < TOL
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_wider_model(cuda_backend, dtype):
    """Sizes at which the bfloat16 session takes the tensor-core matmuls (widths multiples of 64, steps of 64 tokens)."""
    cfg = config([latent_layer(heads=4, dim=32, vdim=32, rank=64, window=48, mlp=dense(ff=256)),
                  pair_layer(heads=4, kv_heads=2, dim=32, vdim=32, rot_dims=16, window=40, scale=0.2, r_heads=2, r_dim=32, r_vdim=64, mlp=dense(ff=192)),
                  lru_layer(width=192, blocks=4, conv=4, mlp=dense(ff=128))], width=128, vocab=200)
    W = random_weights(cfg, seed=15, rank_a=8)
    toks = tokens(cfg, 100)
    want, _ = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64)
    got = s.feed("a", toks, range(100))
    if dtype == "float32":
        assert rel(got, want) < TOL
    else:      # inputs rounded to bfloat16 in every product of three layers: the bulk of the positions bounds the error
        err = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
        assert np.median(err) < 3e-2 and np.mean(err < 6e-2) > 0.9
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_odd_sizes(cuda_backend, dtype):
    """Nothing is a multiple of 4: the unaligned forms of every kernel (scalar loads, one warp per query, exact matmuls)."""
    cfg = config([latent_layer(heads=3, dim=5, vdim=7, rank=9, window=5, mlp=dense(ff=13)),
                  pair_layer(heads=3, kv_heads=1, dim=6, vdim=7, conv=3, rot_dims=2, window=6, r_heads=3, r_dim=5, r_vdim=3, mlp=dense(ff=11)),
                  lru_layer(width=15, blocks=5, conv=3), latent_layer(heads=3, dim=5, vdim=7, rank=9, window=5, weights_of=0, mlp=dense(ff=13))], width=37, vocab=53)
    W = random_weights(cfg, seed=19, qk_gain=2.0)
    toks = tokens(cfg, 41)
    want, _ = forward(cfg, W, toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=32)
    got = np.concatenate([s.feed("a", toks[:35], range(35))] + [s.feed("a", [t], [0]) for t in toks[35:]])
    assert rel(got, want) < tol(dtype)
    close(s)


def test_layers_without_a_window_bound_the_sequence(cuda_backend):
    """A configuration without a mask attends over every earlier position: the cache holds what the caller asks for and a step
    past it is refused."""
    layer = latent_layer(window=9)
    del layer["mixer"]["mask"]
    cfg = config([layer, lru_layer()])
    W = random_weights(cfg, seed=1)
    toks = tokens(cfg, 24)
    full = copy.deepcopy(cfg)
    full["layers"][0]["mixer"]["mask"] = {"size": 1000}
    want, _ = forward(full, W, toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=8, max_context=24)
    assert s.context_limit == 24
    assert rel(s.feed("a", toks, range(24)), want) < TOL
    with pytest.raises(ValueError):
        s.feed("a", [0], [0])
    close(s)


# ── the entry points ──
def _write_model(tmp_path, cfg, W):
    from zgml_b200.host.safetensors import write_safetensors
    d = os.path.join(tmp_path, "model")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), W)
    return d


def test_greedy_generation_through_the_registry(cuda_backend, tmp_path):
    from zgml_b200.host.registry import open_session
    W = random_weights(MIXED, seed=16)
    d = _write_model(tmp_path, MIXED, W)
    prompt = tokens(MIXED, 9)
    want, seq = [], list(prompt)
    for _ in range(12):
        want.append(int(np.argmax(ref.forward(MIXED, as_f64(W), seq)[-1])))
        seq.append(want[-1])
    s = open_session(cuda_backend, d, "float32", n_slots=1, max_chunk=8, max_tokens=32)
    assert s.generate(prompt, 12) == want
    assert not s.pool.live()
    close(s)


def test_trace_replay_from_the_command_line(tmp_path):
    W = random_weights(MIXED, seed=17)
    d = _write_model(tmp_path, MIXED, W)
    toks = tokens(MIXED, 30)
    want, _ = forward(MIXED, W, toks)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[17:19], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[19:], "want": [10]}], "end": ["r"]}]
    out = os.path.join(tmp_path, "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    got0 = np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(1, -1)
    assert rel(got0, want[[0, 16]]) < TOL and rel(got2, want[[29]]) < TOL
