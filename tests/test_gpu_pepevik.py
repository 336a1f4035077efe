"""Pepevik on the CUDA backend against the float64 restatement (tests/pepevik_reference.py): every mechanism alone, the
stream after every layer, whole prompts, token-by-token decoding through the cache and the recurrent states, prompts cut
into portions down to two tokens, interleaved requests in several slots, slot reuse, a key far back found by construction,
the positions where the query temperature steps, the first tokens of a sequence, long decoding, many shapes, and greedy
generation through the registry's entry point and the command line's trace replayer."""
import json
import os
import subprocess

import numpy as np
import pytest

import pepevik_reference as ref
from pepevik_models import as_f64, config, dense, moe, pair_layer, random_weights, ssm_layer

pytestmark = pytest.mark.gpu

TOL = 2e-4   # of the logits' scale; f32 accumulation against float64


def tol(dtype):
    """A bfloat16 session rounds the activations that enter a tensor-core matmul (steps of more than 8 tokens) to bf16."""
    return TOL if dtype == "float32" else 3e-2


def open_model(be, cfg, W, dtype="float32", n_slots=1, max_chunk=16, keep_layers=False, max_context=256):
    from zgml_b200.host.pepevik import PepevikConfig, PepevikModel
    from zgml_b200.host.session import SequenceSession
    model = PepevikModel(be, PepevikConfig.from_dict(cfg), lambda n: W[n], dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, keep_layers=keep_layers, max_context=max_context)


def close(s):
    s.close()
    s.model.close()


def rel(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want)) / (np.max(np.abs(want)) + 1e-30))


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


MIXED = config([ssm_layer(mlp=dense()), pair_layer(mlp=moe()), pair_layer(weights_of=1, mlp=moe()), ssm_layer(heads=3, vdim=5, state=7, groups=1, conv=4, norm_groups=3, mlp=moe(experts=4, top=1, groups=2, keep=1)),
                pair_layer(heads=3, kv_heads=3, dim=6, vdim=4, gru=9, every=3), ssm_layer(weights_of=0, mlp=dense()), pair_layer(weights_of=1, mlp=moe())])


# ── each mechanism alone (a one-layer model without a feed-forward isolates its mixer) ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("layer", [
    ssm_layer(),
    ssm_layer(heads=6, vdim=8, state=16, groups=3, conv=4, norm_groups=1),
    ssm_layer(heads=2, vdim=33, state=5, groups=2, conv=1, norm_groups=6),       # one tap: no carried inputs; more norm parts than heads
    ssm_layer(heads=1, vdim=4, state=200, groups=1, conv=6, norm_groups=2),      # a state of many rows: every lane of a column holds some
    ssm_layer(heads=4, vdim=64, state=64, groups=1, conv=2, norm_groups=4),
    ssm_layer(heads=2, vdim=6, state=300, groups=2, conv=2, norm_groups=1),
    ssm_layer(heads=2, vdim=20, state=2, groups=1, conv=3, norm_groups=1),       # fewer state rows than a thread holds
    pair_layer(),
    pair_layer(heads=6, kv_heads=2, dim=5, vdim=9, gru=7, every=1),              # three heads per key head; the temperature steps at every position
    pair_layer(heads=1, kv_heads=1, dim=40, vdim=3, gru=64, coef=0.0),
    pair_layer(heads=2, kv_heads=2, dim=16, vdim=16, gru=40, every=1000),        # no step of the temperature inside the prompt
    pair_layer(heads=4, kv_heads=1, dim=68, vdim=132, gru=130, every=7),
], ids=["ssm", "ssm-3groups", "ssm-1tap", "ssm-state200", "ssm-64x64", "ssm-state300", "ssm-state2", "pair", "pair-grouped", "pair-1head", "pair-flat-temp", "pair-wide"])
def test_mixer_alone(cuda_backend, layer, dtype):
    cfg = config([layer], width=40, vocab=61)
    W = random_weights(cfg, seed=5, qk_gain=4.0)
    toks = tokens(cfg, 45)
    want, stream = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64, keep_layers=True)
    got = s.feed("a", toks, range(45))
    if dtype == "float32":
        assert rel(s.layer_streams(32, "all")[0], stream[0][:32]) < TOL
    assert rel(got, want) < tol(dtype)
    close(s)


@pytest.mark.parametrize("silent", ["left", "right"])
def test_branches_of_the_pair_alone(cuda_backend, silent):
    """With the output weight of one branch at zero the layer is the other branch alone: sigmoid attention, or the recurrent unit."""
    cfg = config([pair_layer(heads=4, kv_heads=2, dim=8, vdim=12, gru=20, every=4)], width=32, vocab=40)
    W = random_weights(cfg, seed=21, qk_gain=5.0)
    W[f"l0.mix.{silent}.out"][:] = 0.0
    toks = tokens(cfg, 30)
    want, stream = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True, n_slots=2)
    assert rel(s.feed("a", toks, range(30))[:16], want[:16]) < TOL
    assert rel(s.layer_streams(16, "all")[0], stream[0][:16]) < TOL
    decoded = np.concatenate([s.feed("d", [t], [0]) for t in toks])
    assert rel(decoded, want) < TOL
    close(s)


@pytest.mark.parametrize("mlp", [dense(), dense(ff=7), dense(ff=300), moe(), moe(experts=3, top=1, ff=7, groups=1, keep=1), moe(experts=4, top=4, ff=40, groups=2, keep=2),
                                 moe(experts=32, top=5, ff=16, groups=8, keep=3), moe(experts=6, top=2, ff=12, groups=6, keep=4), None],
                         ids=["dense", "dense-7", "dense-300", "moe", "top1-no-groups", "all-experts", "32-experts-8-groups", "groups-of-one", "none"])
def test_feed_forward(cuda_backend, mlp):
    """The stream after the layer is compared too, so a fault in the activation, the routing or the expert weights cannot hide
    behind the final Dynamic Tanh."""
    cfg = config([ssm_layer(heads=2, vdim=4, state=4, groups=1, conv=2, norm_groups=1, mlp=mlp)], width=36, vocab=50)
    W = random_weights(cfg, seed=9)
    toks = tokens(cfg, 19)
    want, stream = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True)
    got = s.feed("a", toks[:16], range(16))
    assert rel(s.layer_streams(16, "all")[0], stream[0][:16]) < TOL
    assert rel(got, want[:16]) < TOL
    close(s)


def test_routing_with_negative_choice_scores(cuda_backend):
    """Corrections far below zero make every choice score negative.  An expert of a dropped group must count as minus infinity:
    counted as 0 it would beat every kept expert.  The best group is made to hold one strong and otherwise weak experts, so the
    second and third choice must come from the second-best group."""
    mlp = moe(experts=9, top=3, ff=8, groups=3, keep=2)
    cfg = config([ssm_layer(heads=2, vdim=4, state=4, groups=1, conv=2, norm_groups=1, mlp=mlp)], width=36, vocab=50)
    W = random_weights(cfg, seed=10)
    W["l0.mlp.correction"][:] = np.array([-2.0, -4.5, -4.75, -3.0, -3.25, -3.5, -2.5, -2.75, -6.0], np.float32)
    toks = tokens(cfg, 24)
    Wd = as_f64(W)
    want, stream = ref.forward(cfg, Wd, toks)
    x = Wd["embed"][toks] * cfg["embedding"]["scale"] + Wd["pos"][:len(toks)]
    x = x + cfg["residual_mult"] * ref.mamba2(ref.dynamic_tanh(x, Wd, "l0.norm1"), Wd, "l0.mix.", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    h = ref.dynamic_tanh(x, Wd, "l0.norm2")
    choice = ref.sigmoid(h @ Wd["l0.mlp.router"].T) + Wd["l0.mlp.correction"]
    assert (choice < 0).all()                              # a dropped expert counted as 0 would be chosen first at every token
    idx, _ = ref.route(h, Wd, "l0.mlp.", mlp["router"])
    assert len({tuple(sorted(set(e // 3 for e in r))) for r in idx.tolist()}) > 1     # the kept pair of groups changes from token to token
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True)
    got = s.feed("a", toks[:16], range(16))
    assert rel(s.layer_streams(16, "all")[0], stream[0][:16]) < TOL
    assert rel(got, want[:16]) < TOL
    single = np.concatenate([s.feed("a", [t], [0]) for t in toks[16:]])
    assert rel(single, want[16:]) < TOL
    close(s)


def test_layer_streams_of_a_mixed_stack(cuda_backend):
    """Layers that run with another layer's weights keep states of their own."""
    W = random_weights(MIXED, seed=2)
    toks = tokens(MIXED, 16)
    want, stream = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, "float32", keep_layers=True)
    got = s.feed("a", toks, range(16))
    layers = s.layer_streams(16, "all")
    assert len(layers) == len(MIXED["layers"])
    for i in range(len(MIXED["layers"])):
        assert rel(layers[i], stream[i]) < TOL, f"layer {i}"
    assert rel(got, want) < TOL
    close(s)


# ── prefill against decoding, portions, first tokens ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_prefill_equals_token_by_token(cuda_backend, dtype):
    W = random_weights(MIXED, seed=3, qk_gain=3.0)
    toks = tokens(MIXED, 40)
    want, _ = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, dtype, n_slots=2)
    whole = s.feed("whole", toks, range(40))
    single = np.concatenate([s.feed("single", [t], [0]) for t in toks])
    assert rel(whole, want) < tol(dtype) and rel(single, want) < TOL     # single tokens take the exact row kernels in both formats
    close(s)


@pytest.mark.parametrize("cuts", [[2] * 20, [1, 2, 3, 5, 7, 9, 13], [37, 2, 1], [16, 16, 8], [3, 37]], ids=["twos", "growing", "long-then-short", "menu", "short-then-long"])
def test_portions(cuda_backend, cuts):
    """However a prompt is cut — inside a convolution's reach, two tokens at a time — the logits stay the same."""
    W = random_weights(MIXED, seed=4, qk_gain=3.0)
    toks = tokens(MIXED, 40)
    want, _ = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, "float32", max_chunk=32)
    got, at = [], 0
    for n in cuts:
        got.append(s.feed("a", toks[at:at + n], range(n)))
        at += n
    assert at == 40 and rel(np.concatenate(got), want) < TOL
    close(s)


def test_first_tokens(cuda_backend):
    """Position 0 alone (zeros before the convolution's start, an empty state, one visible key), then positions 1 and 2 one by one."""
    W = random_weights(MIXED, seed=6)
    toks = tokens(MIXED, 3)
    want, _ = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, "float32")
    got = np.concatenate([s.feed("a", [t], [0]) for t in toks])
    assert rel(got, want) < TOL
    s.release("a")
    assert rel(s.feed("b", toks, [0, 1, 2]), want) < TOL
    close(s)


# ── requests side by side, slots ──
def test_interleaved_requests_and_slot_reuse(cuda_backend):
    W = random_weights(MIXED, seed=7, qk_gain=2.0)
    Wd = as_f64(W)
    reqs = {"a": tokens(MIXED, 29, 1), "b": tokens(MIXED, 11, 2), "c": tokens(MIXED, 40, 3)}
    want = {k: ref.forward(MIXED, Wd, v)[0] for k, v in reqs.items()}
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
    # the cache is masked by position)
    assert not s.pool.live()
    assert rel(s.feed("c", reqs["c"], range(40)), want["c"]) < TOL
    with pytest.raises(ValueError):
        s.feed("c", [0] * 300, [])                        # past the positions the session's cache holds
    close(s)


def test_positions_stop_at_the_table(cuda_backend):
    """The cache is never sized past the learned position table, whatever the caller asks for."""
    cfg = config([pair_layer()], max_positions=24)
    W = random_weights(cfg, seed=1)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=8, max_context=1000)
    assert s.context_limit == 24
    toks = tokens(cfg, 24)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    assert rel(s.feed("a", toks, range(24)), want) < TOL
    with pytest.raises(ValueError):
        s.feed("a", [0], [0])
    close(s)


# ── what a query must and must not see ──
def test_temperature_steps_in_prompt_and_decoding(cuda_backend):
    """One attention branch with sharp weights and a temperature that steps every 6 positions: position p is in step
    floor((p + 1) / 6).  The device agrees with the restatement at every position, as a prompt and decoded, and differs from a
    restatement whose steps begin one position later."""
    cfg = config([pair_layer(heads=2, kv_heads=1, dim=8, vdim=8, coef=1.5, every=6)], width=32, vocab=40)
    W = random_weights(cfg, seed=8, qk_gain=6.0)
    W["l0.mix.right.out"][:] = 0.0
    Wd = as_f64(W)
    toks = tokens(cfg, 32)
    want, _ = ref.forward(cfg, Wd, toks)
    real = ref.query_temperature
    try:
        ref.query_temperature = lambda p, coef, every: real(p - 1, coef, every)
        control, _ = ref.forward(cfg, Wd, toks)
    finally:
        ref.query_temperature = real
    assert np.abs(control[5] - want[5]).max() > 1e-2 * np.abs(want).max() and np.abs(control[4] - want[4]).max() < 1e-12
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=32)
    prompt = s.feed("p", toks, range(32))
    decoded = np.concatenate([s.feed("d", toks[:3], range(3))] + [s.feed("d", [t], [0]) for t in toks[3:]])
    assert rel(prompt, want) < TOL and rel(decoded, want) < TOL
    assert rel(prompt, control) > 20 * TOL
    close(s)


def test_far_key_among_hundreds(cuda_backend):
    """The last query is made to weigh one early position among 300 and hardly any other.  With the position table at zero a
    score depends on the two tokens, the query's position and the distance alone, so the pair of token ids whose score stands
    out most against every other key token is found from the weights; the key token is placed once, far back, the query token
    last, and the per-head score bias is set so that the far key's weight is large and every other weight small.  Changing the
    far token must move the restatement's last logits, and the device must agree with the restatement, in a prompt and with the
    last tokens decoded."""
    cfg = config([pair_layer(heads=2, kv_heads=2, dim=8, vdim=8, coef=0.3, every=64)], width=32, vocab=40)
    W = random_weights(cfg, seed=12, qk_gain=6.0)
    W["pos"][:] = 0.0
    W["l0.mix.right.out"][:] = 0.0
    W["l0.mix.left.r1"][:] = 0.25
    m = cfg["layers"][0]["mixer"]["left"]
    H, dim = m["heads"], m["dim"]
    n, far = 300, 4
    Wd = as_f64(W)
    eps = cfg["norm"]["eps"]
    h = ref.dynamic_tanh(Wd["embed"] * cfg["embedding"]["scale"], Wd, "l0.norm1")                # [vocab, width]: the mixer's input of every token id
    q = ref.rms((h @ Wd["l0.mix.left.q"].T).reshape(-1, H, dim), eps) * Wd["l0.mix.left.q.norm"] * ref.query_temperature(n - 1, 0.3, 64)
    k = ref.rms((h @ Wd["l0.mix.left.k"].T).reshape(-1, H, dim), eps) * Wd["l0.mix.left.k.norm"]
    S = np.einsum("ahd,bhd->hab", q, k) * m["scale"]
    margin = np.full(S.shape, -np.inf)
    for b in range(S.shape[2]):
        margin[:, :, b] = S[:, :, b] - np.delete(S, b, axis=2).max(axis=2)
    hd, a_tok, b_tok = np.unravel_index(np.argmax(margin), margin.shape)
    penalty = Wd["l0.mix.left.r1"][hd] * np.log(1.0 + Wd["l0.mix.left.r2"][hd] * (n - 1 - far))
    W["l0.mix.left.pb"][:] = -30.0                                                                 # the other head says nothing
    W["l0.mix.left.pb"][hd] = np.float32(np.floor(-(S[hd, a_tok, b_tok] - penalty) + 2.0))        # the far key weighs about sigmoid(2)
    Wd = as_f64(W)
    pool = [t for t in range(cfg["vocab"]) if t != b_tok]
    toks = [pool[i] for i in np.random.default_rng(1).integers(0, len(pool), n)]
    toks[far], toks[-1] = int(b_tok), int(a_tok)
    want, _ = ref.forward(cfg, Wd, toks)
    moved = list(toks)
    moved[far] = pool[0]
    assert np.abs(ref.forward(cfg, Wd, moved)[0][-1] - want[-1]).max() > 1e-2 * np.abs(want).max(), "the construction lost its far key"
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=64, max_context=320)
    assert rel(s.feed("p", toks, range(n)), want) < TOL
    s.feed("d", toks[:n - 5], [])
    decoded = np.concatenate([s.feed("d", [t], [0]) for t in toks[n - 5:]])
    assert rel(decoded, want[n - 5:]) < TOL
    close(s)


@pytest.mark.parametrize("layer", [pair_layer(heads=4, kv_heads=2, dim=68, vdim=132, gru=24, every=50), pair_layer(heads=8, kv_heads=1, dim=4, vdim=4, gru=8, every=128),
                                   pair_layer(heads=2, kv_heads=2, dim=88, vdim=72, gru=300, every=200)], ids=["wide", "8-per-group", "88"])
def test_long_cache_and_split_decoding(cuda_backend, layer):
    """Keys beyond one tile of the prompt kernel (64) and one share of the decoding kernel (32), key and value sizes beyond one
    slice, and a cache long enough that single-token steps deal their keys to several CTAs whose unnormalised shares add up."""
    cfg = config([layer], width=48, vocab=50)
    W = random_weights(cfg, seed=18, qk_gain=3.0)
    W["l0.mix.left.pb"] -= 2.0                              # sums over 300 keys stay moderate
    n = 300
    toks = tokens(cfg, n)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=128, max_context=512)
    assert rel(s.feed("p", toks, range(n)), want) < TOL
    s.feed("d", toks[:n - 12], [])
    decoded = np.concatenate([s.feed("d", toks[i:i + 1], [0]) for i in range(n - 12, n - 4)] + [s.feed("d", toks[n - 4:], range(4))])
    assert rel(decoded, want[n - 12:]) < TOL
    close(s)


def test_long_steps_walk_segments_side_by_side(cuda_backend):
    """Steps of 256 tokens: the state-space scan cuts them into segments walked side by side (each first from an empty state, then
    from the state the fold gives it) and the recurrent unit into 64; the states they leave must carry on into smaller steps and
    single tokens, in a slot that is not the first, after a request that used the same slot before."""
    cfg = config([ssm_layer(heads=4, vdim=8, state=24, groups=2, conv=4, norm_groups=2, mlp=dense()), ssm_layer(heads=2, vdim=12, state=200, groups=1, conv=2, norm_groups=3),
                  pair_layer(heads=2, kv_heads=1, dim=8, vdim=8, gru=70, every=100, mlp=moe()), ssm_layer(heads=4, vdim=8, state=24, groups=2, conv=4, norm_groups=2, weights_of=0, mlp=dense())],
                 width=48, vocab=50, max_positions=700)
    W = random_weights(cfg, seed=23, qk_gain=2.0)
    n = 600
    toks = tokens(cfg, n)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=256, max_context=640)
    s.feed("first", toks[:5], [])                           # takes slot 0 and keeps it
    s.feed("other", toks[100:400], [])                      # leaves its states in slot 1
    s.release("other")
    got = np.concatenate([s.feed("a", toks[:570], range(570))] + [s.feed("a", [t], [0]) for t in toks[570:]])   # 256 + 256 + 32 + 16 + 8 + 2, then single tokens
    assert s.pool.slot("a") == 1
    assert rel(got, want) < TOL
    close(s)


def test_long_decoding(cuda_backend):
    """150 decoded tokens through every kind of state: the recurrent states, the convolution inputs and a growing cache."""
    cfg = config([ssm_layer(mlp=moe()), pair_layer(mlp=dense(), every=16), ssm_layer(weights_of=0, mlp=moe()), pair_layer(weights_of=1, mlp=dense(), every=16)])
    W = random_weights(cfg, seed=13, qk_gain=3.0)
    toks = tokens(cfg, 160)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=4)
    got = np.concatenate([s.feed("a", toks[:10], range(10))] + [s.feed("a", [t], [0]) for t in toks[10:]])
    assert rel(got, want) < TOL
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_wider_model(cuda_backend, dtype):
    """Sizes at which the bfloat16 session takes the tensor-core matmuls and the grouped expert path (width and expert width
    multiples of 64, steps of 64 tokens)."""
    cfg = config([ssm_layer(heads=8, vdim=32, state=32, groups=2, conv=4, norm_groups=4, mlp=moe(experts=4, top=2, ff=64, groups=2, keep=2)),
                  pair_layer(heads=4, kv_heads=2, dim=32, vdim=32, gru=192, every=32, mlp=dense(ff=256)),
                  ssm_layer(heads=4, vdim=64, state=128, groups=1, conv=4, norm_groups=1, mlp=moe(experts=6, top=1, ff=128, groups=3, keep=2))], width=128, vocab=200)
    W = random_weights(cfg, seed=15)
    toks = tokens(cfg, 100)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64)
    got = s.feed("a", toks, range(100))
    if dtype == "float32":
        assert rel(got, want) < TOL
    else:      # a rounded input may flip a close expert choice at single positions: the bulk must agree
        err = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
        assert np.median(err) < 3e-2 and np.mean(err < 6e-2) > 0.9
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_odd_sizes(cuda_backend, dtype):
    """Nothing is a multiple of 4: the unaligned forms of every kernel (scalar loads, one warp per query, exact matmuls)."""
    cfg = config([ssm_layer(heads=3, vdim=5, state=7, groups=3, conv=3, norm_groups=5, mlp=moe(experts=3, top=2, ff=11, groups=1, keep=1)),
                  pair_layer(heads=3, kv_heads=1, dim=5, vdim=7, gru=13, every=3, mlp=dense(ff=13)),
                  pair_layer(heads=2, kv_heads=2, dim=7, vdim=3, gru=5, every=2), ssm_layer(heads=3, vdim=5, state=7, groups=3, conv=3, norm_groups=5, weights_of=0,
                                                                                            mlp=moe(experts=3, top=2, ff=11, groups=1, keep=1))], width=37, vocab=53)
    W = random_weights(cfg, seed=19, qk_gain=2.0)
    toks = tokens(cfg, 41)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=32)
    got = np.concatenate([s.feed("a", toks[:35], range(35))] + [s.feed("a", [t], [0]) for t in toks[35:]])
    assert rel(got, want) < tol(dtype)
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
        want.append(int(np.argmax(ref.forward(MIXED, as_f64(W), seq)[0][-1])))
        seq.append(want[-1])
    s = open_session(cuda_backend, d, "float32", n_slots=1, max_chunk=8, max_tokens=32)
    assert s.generate(prompt, 12) == want
    assert not s.pool.live()
    close(s)


def test_trace_replay_from_the_command_line(tmp_path):
    W = random_weights(MIXED, seed=17)
    d = _write_model(tmp_path, MIXED, W)
    toks = tokens(MIXED, 30)
    want, _ = ref.forward(MIXED, as_f64(W), toks)
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
