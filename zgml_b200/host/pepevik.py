"""Pepevik: a pre-norm decoder stack with learned positions and a Dynamic Tanh in place of every norm.  A layer's mixer is
either a Mamba-2 state-space recurrence, or two mixers side by side on the same input — sigmoid attention over every earlier
position (grouped heads, RMS-normed queries and keys, a query temperature that grows with the position, a logarithmic
distance penalty, weights that are not normalised over the keys) and a minimal gated recurrent unit — whose RMS-normed outputs
are averaged.  Feed-forwards are dense (squared ReLU) or a routed mixture of gated experts with sigmoid scores and a choice
restricted to the best groups of experts.  A layer may run with another layer's weights and a state of its own.

This file is the model's configuration reader, its weight packer and its LOWERING to a DeviceProgram; the arithmetic is in the
sequence-model DeviceOps of the CUDA library (csrc/seqops.cu, csrc/mixops.cu, csrc/recops.cu) and all state in the session's
`SequenceStatePool`.  Every size and per-model constant comes from config.json or a tensor's shape.

Per layer (x: f32 stream, m: the residual multiplier):   x += m mixer(DyT(x; norm1));   x += m ff(DyT(x; norm2))
    DyT(x; n) = tanh(alpha x) w + b.  The residual step that closes a sublayer and the Dynamic Tanh that opens the next are
    ONE launch (NORM with the kinds "none" + "dyt").

mamba2      [z | x | B | C | dt] = W_in h in ONE matmul; CAUSAL_CONV (bias, SiLU) over x | B | C; SSM_SCAN; GATED_NORM
            (y silu(z), RMS norm in equal parts, weight); W_o.
parallel    [q | k | v | z | u | g] = W h + b in ONE matmul for both branches.  Left: CACHE_APPEND norms the key heads on
            their way into the cache and the query heads (with the temperature) in place, CACHED_ATTENTION with sigmoid weights;
            the distance penalty and the per-head score bias are ONE table per layer, pb_h - r1_h ln(1 + r2_h d), evaluated in
            f32 at load for every distance the cache can hold.  Right: MIN_GRU.  Each branch has its own W_o; the two RMS
            norms of the results and their sum are one residual step with two sources.
feed-forward dense: W_up with relu^2 in its epilogue, W_down.  moe: router matmul, ROUTE "corrected_sigmoid" with groups, MOE_FFN.
"""
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import abi
from ..backend import CudaBackend, DeviceBuffer, DeviceOp, DeviceProgram, ExternBuffer, ProgramIO, seq_scratch_elems, seq_state_elems
from .safetensors import SafetensorsFile
from .session import LoweredProgram
from .state import SequenceStatePool, StateSpec
from .weights import WeightArena

ARCHITECTURE = "Pepevik"
DEFAULT_CONTEXT = 4096     # positions a sequence may reach when the caller names no bound (never more than the position table holds)
MIXERS = ("mamba2", "parallel")


@dataclass(frozen=True)
class PepevikConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    max_positions: int
    layers: tuple            # of dicts: {"type", "mixer", "mlp", "weights": index of the layer whose tensors it uses}

    @classmethod
    def from_dict(cls, c: dict) -> "PepevikConfig":
        if c.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture = {c.get('architecture')!r}")
        layers = []
        for i, L in enumerate(c["layers"]):
            kind, m, mlp = L["type"], L["mixer"], L.get("mlp")
            if kind not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            owner = L.get("weights_of", i)
            if "weights_of" in L:
                if not (0 <= owner < i) or "weights_of" in c["layers"][owner]:
                    raise ValueError(f"layer {i}: weights_of must name an earlier layer with tensors of its own")
                o = c["layers"][owner]
                if (o["type"], o["mixer"], o.get("mlp")) != (kind, m, mlp):
                    raise ValueError(f"layer {i}: differs from layer {owner}, whose weights it uses")
            if kind == "mamba2":
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"] or m["conv"] < 1:
                    raise ValueError(f"layer {i}: heads must be a multiple of groups, heads * vdim of norm_groups, conv >= 1")
            else:
                if m["left"]["heads"] % m["left"]["kv_heads"]:
                    raise ValueError(f"layer {i}: heads not a multiple of kv_heads")
                if m["left"]["q_temp"]["every"] < 1:
                    raise ValueError(f"layer {i}: q_temp.every must be positive")
            if mlp is not None:
                if mlp.get("kind") not in ("dense", "moe"):
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
                if mlp["kind"] == "moe":
                    r = mlp["router"]
                    g = r.get("groups") or {"count": 1, "keep": 1}
                    if not (1 <= r["top"] <= r["experts"]) or r["experts"] % g["count"] or not (1 <= g["keep"] <= g["count"]) or \
                            g["keep"] * (r["experts"] // g["count"]) < r["top"]:
                        raise ValueError(f"layer {i}: top must lie in 1 .. experts, experts divide into groups, and the kept groups hold top experts")
            layers.append({"type": kind, "mixer": m, "mlp": mlp, "weights": owner})
        return cls(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), float(c["embedding"]["scale"]), float(c["residual_mult"]),
                   int(c["max_positions"]), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "PepevikConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


def distance_score_table(r1, r2, pb, n: int) -> np.ndarray:
    """[H, n] f32: what is added to the scaled score of head h at distance d, pb_h - r1_h ln(1 + r2_h d), in f32 like every
    other part of the score."""
    f = np.float32
    d = np.arange(n, dtype=f)[None, :]
    r1, r2, pb = (np.asarray(a, dtype=f)[:, None] for a in (r1, r2, pb))
    return (pb - r1 * np.log1p(r2 * d).astype(f)).astype(f)


class PepevikModel:
    """Weights resident in HBM (one arena per layer that has tensors + one for the tables, the final norm and the head) and
    the lowering."""

    bounded_context = True     # the attention branch caches every position and positions are looked up in a table

    def __init__(self, be: CudaBackend, cfg: PepevikConfig, tensors, dtype: str = "bfloat16"):
        """tensors: name -> f32 array accessor (`tensors(name)`), e.g. SafetensorsFile.f32."""
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.be, self.cfg, self.dtype = be, cfg, dtype
        self.wdt = abi.W_BF16 if dtype == "bfloat16" else abi.W_F32
        self.vocab, self.width = cfg.vocab, cfg.width
        self.layer_meta: Dict[int, dict] = {}
        self.arenas: Dict[int, WeightArena] = {}
        self.buffers: Dict[int, DeviceBuffer] = {}
        self._tables: Dict[tuple, DeviceBuffer] = {}
        self._head_consts: Dict[int, tuple] = {}
        D = cfg.width

        def dyt(A, name, p):       # weight | bias | alpha, in this order: what NORM kind "dyt" reads from one offset
            w, b, alpha = tensors(p), tensors(p + ".b"), tensors(p + ".alpha")
            assert w.shape == (D,) and b.shape == (D,) and alpha.size == 1, f"{p}: shapes {w.shape} {b.shape} {alpha.shape}"
            A.add(name, np.concatenate([w, b, alpha.reshape(1)]))

        for i, L in enumerate(cfg.layers):
            if L["weights"] != i:
                continue
            p, m = f"l{i}.", L["mixer"]
            A = WeightArena(self.wdt)
            meta = {}
            dyt(A, "norm1", p + "norm1")
            if L["type"] == "mamba2":
                H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
                inner, C = H * P, H * P + 2 * G * N
                w_in, conv = tensors(p + "mix.in"), tensors(p + "mix.conv")
                assert w_in.shape == (inner + C + H, D) and conv.shape == (C, taps), f"{p}mix.in {w_in.shape}, conv {conv.shape}"
                A.add("in", w_in)
                A.add("conv", conv)
                A.add("conv.b", tensors(p + "mix.conv.b"))
                for n in ("dt_bias", "A_log", "D"):
                    t = tensors(p + "mix." + n)
                    assert t.shape == (H,)
                    A.add(n, t)
                nw, o = tensors(p + "mix.norm"), tensors(p + "mix.o")
                assert nw.shape == (inner,) and o.shape == (D, inner)
                A.add("gnorm", nw)
                A.add("o", o)
                meta.update(n_in=inner + C + H, inner=inner, C=C)
            else:
                l, W = m["left"], m["right"]["width"]
                H, G, dim, vdim = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
                pl, pr = p + "mix.left.", p + "mix.right."
                parts = [tensors(pl + "q"), tensors(pl + "k"), tensors(pl + "v"), tensors(pr + "z"), tensors(pr + "x"), tensors(pr + "g")]
                shapes = [(H * dim, D), (G * dim, D), (G * vdim, D), (W, D), (W, D), (W, D)]
                assert [t.shape for t in parts] == shapes, f"{p}mix: projection shapes {[t.shape for t in parts]}"
                A.add("in", np.concatenate(parts, 0))
                zb, xb = tensors(pr + "z.b"), tensors(pr + "x.b")
                assert zb.shape == (W,) and xb.shape == (W,)
                nq = H * dim + G * (dim + vdim)
                A.add("in.b", np.concatenate([np.zeros(nq, np.float32), zb, xb, np.zeros(W, np.float32)]))
                for n in ("q.norm", "k.norm"):
                    t = tensors(pl + n)
                    assert t.shape == (dim,)
                    A.add(n, t)
                lo, ro = tensors(pl + "o"), tensors(pr + "o")
                assert lo.shape == (D, H * vdim) and ro.shape == (D, W)
                A.add("left.o", lo)
                A.add("right.o", ro)
                for n, t in (("left.out", tensors(pl + "out")), ("right.out", tensors(pr + "out"))):
                    assert t.shape == (D,)
                    A.add(n, t)
                r1, r2, pb = tensors(pl + "r1"), tensors(pl + "r2"), tensors(pl + "pb")
                assert r1.shape == (H,) and r2.shape == (H,) and pb.shape == (H,)
                self._head_consts[i] = (r1, r2, pb)
                meta.update(n_in=nq + 3 * W, W=W, k_col=H * dim, z_col=nq)
            mlp = L["mlp"]
            if mlp is not None:
                dyt(A, "norm2", p + "norm2")
                if mlp["kind"] == "dense":
                    up, down = tensors(p + "mlp.up"), tensors(p + "mlp.down")
                    ff = up.shape[0]
                    assert up.shape == (ff, D) and down.shape == (D, ff) and ff == mlp.get("ff", ff)
                    A.add("up", up)
                    A.add("down", down)
                    meta.update(ff=ff)
                else:
                    r = mlp["router"]
                    E, top, ff = r["experts"], r["top"], mlp["expert"]["ff"]
                    g = r.get("groups") or {"count": 1, "keep": 1}
                    router, corr = tensors(p + "mlp.router"), tensors(p + "mlp.correction")
                    assert router.shape == (E, D) and corr.shape == (E,)
                    A.add("router", router)
                    A.add("correction", corr)
                    for part, shape in (("gate", (ff, D)), ("up", (ff, D)), ("down", (D, ff))):
                        stack = [tensors(p + f"mlp.e{e}.{part}") for e in range(E)]
                        assert all(s.shape == shape for s in stack)
                        A.add(part, np.stack(stack))
                    meta.update(E=E, top=top, ff=ff, groups=g["count"], keep=g["keep"])
            self.layer_meta[i], self.arenas[i] = meta, A
            self.buffers[i] = A.upload(be)
        A = WeightArena(self.wdt)
        emb, pos, head = tensors("embed"), tensors("pos"), tensors("head")
        assert emb.shape == (cfg.vocab, D) and head.shape == (cfg.vocab, D) and pos.ndim == 2 and pos.shape[1] == D and pos.shape[0] >= 1, f"pos: shape {pos.shape}"
        self.positions = min(cfg.max_positions, pos.shape[0])      # a sequence can go as far as both the configuration and the table allow
        A.add("embed", emb)
        A.add("pos", pos)
        dyt(A, "final.norm", "final.norm")
        A.add("head", head)
        self.arenas[-1] = A
        self.buffers[-1] = A.upload(be)

    @classmethod
    def load(cls, be: CudaBackend, model_dir: str, dtype: str = "bfloat16") -> "PepevikModel":
        cfg = PepevikConfig.from_json(os.path.join(model_dir, "config.json"))
        sf = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
        try:
            return cls(be, cfg, sf.f32, dtype)
        finally:
            sf.close()

    def weight_bytes(self) -> int:
        return sum(b.nbytes for b in self.buffers.values())

    # ── state ──
    def capacity(self, max_chunk: int, max_context: Optional[int]) -> int:
        """Positions a sequence of the session may reach: what the caller asks for, never more than the position table holds."""
        return min(max(int(max_context) if max_context else DEFAULT_CONTEXT, max_chunk), self.positions)

    def _ssm_state_elems(self, m: dict) -> int:
        probe = DeviceOp.ssm_scan(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, m["heads"], m["groups"], m["state"], m["vdim"], 1, 1, self.wdt)
        n = seq_state_elems(probe)
        if not n:
            raise ValueError(f"state size {m['state']} is more than the state-space scan holds per head")
        return n

    def state_specs(self, max_chunk: int, max_context: Optional[int] = None) -> List[StateSpec]:
        capacity = self.capacity(max_chunk, max_context)
        specs = []
        for i, L in enumerate(self.cfg.layers):
            m = L["mixer"]
            if L["type"] == "mamba2":
                specs.append(StateSpec(f"l{i}.ssm", self._ssm_state_elems(m), True))
                if m["conv"] > 1:
                    specs.append(StateSpec(f"l{i}.tail", (m["conv"] - 1) * (m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]), True))
            else:
                l = m["left"]
                specs.append(StateSpec(f"l{i}.kv", capacity * l["kv_heads"] * (l["dim"] + l["vdim"]), False))    # masked by position: no clearing
                specs.append(StateSpec(f"l{i}.gru", m["right"]["width"], True))
        return specs

    def _score_table(self, owner: int, n: int) -> DeviceBuffer:
        """The distance penalty and the per-head score bias of the attention branch, one f32 table [H, n] per set of weights."""
        if (owner, n) not in self._tables:
            t = distance_score_table(*self._head_consts[owner], n)
            buf = DeviceBuffer(self.be, t.nbytes, zero=False)
            buf.upload(np.ascontiguousarray(t))
            self._tables[(owner, n)] = buf
        return self._tables[(owner, n)]

    # ── lowering ──
    def lower(self, T: int, head: str, pool: SequenceStatePool, keep_layers: bool = False) -> LoweredProgram:
        cfg, wdt, D, eps, mult = self.cfg, self.wdt, self.cfg.width, self.cfg.norm_eps, self.cfg.residual_mult
        sizes: List[int] = []
        externs: List[ExternBuffer] = []
        ops = []

        def new(n):
            sizes.append(max(int(n), 1))
            return len(sizes) - 1

        ext_of: Dict[int, int] = {}

        def ext(buf: DeviceBuffer):      # one program buffer per device buffer (layers that share weights name the same one)
            if id(buf) not in ext_of:
                sizes.append(buf.elems)
                externs.append(ExternBuffer(len(sizes) - 1, buf))
                ext_of[id(buf)] = len(sizes) - 1
            return ext_of[id(buf)]

        ctl = new(abi.CTL_IDS + T)
        gl, GA = ext(self.buffers[-1]), self.arenas[-1]
        TD = T * D
        xs = [new(TD), new(TD)]
        h, y = new(TD), new(TD)
        proj = new(T * max(m["n_in"] for m in self.layer_meta.values()))
        shared: Dict[str, int] = {}

        def scratch(name, n):      # activations reused by every layer that needs them
            if name not in shared or sizes[shared[name]] < n:
                shared[name] = new(n)
            return shared[name]

        def next_x(cur):
            if keep_layers:
                return new(TD)
            return xs[1] if cur == xs[0] else xs[0]

        x = xs[0]
        ops.append(DeviceOp.embed(x, ctl, gl, GA.off["embed"], T, D, cfg.embedding_scale, wdt, positions_off=GA.off["pos"]))
        # The residual step that closes a sublayer waits for the Dynamic Tanh that opens the next one: one launch for both.
        pending: List[tuple] = []          # (src, kind, weight buffer, weight offset, gain, second source, its weight offset): x += gain * kind(src ...)

        def open_norm(dst, wb, w_off):
            nonlocal x
            if pending:
                src, kind, pw, p_off, gain, src2, p2_off = pending.pop()
                nx = next_x(x)
                ops.append(DeviceOp.norm(nx, src, pw, p_off, T, D, eps, wdt, kind=kind, res=x, gain=gain, then=dst, then_w=wb, then_w_off=w_off, then_kind="dyt",
                                         src2=src2, src2_w_off=p2_off))
                x = nx
            else:
                ops.append(DeviceOp.norm(dst, x, wb, w_off, T, D, eps, wdt, kind="dyt"))

        def flush():
            nonlocal x
            if pending:
                src, kind, pw, p_off, gain, src2, p2_off = pending.pop()
                nx = next_x(x)
                ops.append(DeviceOp.norm(nx, src, pw, p_off, T, D, eps, wdt, kind=kind, res=x, gain=gain, src2=src2, src2_w_off=p2_off))
                x = nx

        layer_bufs = []
        slots = pool.n_slots
        for i, L in enumerate(cfg.layers):
            owner = L["weights"]
            m, meta, A, wb = L["mixer"], self.layer_meta[owner], self.arenas[owner], ext(self.buffers[owner])
            ni = meta["n_in"]
            open_norm(h, wb, A.off["norm1"])
            if keep_layers and i:
                layer_bufs.append(x)                    # the stream after layer i - 1 exists once its last residual step has run
            if L["type"] == "mamba2":
                H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
                inner, C = meta["inner"], meta["C"]
                ops.append(DeviceOp.linear(proj, h, wb, A.off["in"], T, ni, D, wdt))
                conv = scratch("conv", T * C)
                tail = ext(pool.buffers[f"l{i}.tail"]) if taps > 1 else ctl    # one tap: no carried inputs, the operand is unused
                ops.append(DeviceOp.causal_conv(conv, proj, wb, A.off["conv"], tail, ctl, T, C, taps, wdt, "silu", src_off=inner, src_rs=ni,
                                                bias_off=A.off["conv.b"]))
                mix = scratch("mix", T * inner)
                ops.append(DeviceOp.ssm_scan(mix, conv, proj, wb, ext(pool.buffers[f"l{i}.ssm"]), ctl, 0, inner, inner + G * N, inner + C,
                                             A.off["A_log"], A.off["dt_bias"], A.off["D"], T, H, G, N, P, C, ni, wdt))
                ops.append(DeviceOp.gated_norm(mix, mix, proj, wb, A.off["gnorm"], 0, T, inner, m["norm_groups"], ni, eps, wdt))
                ops.append(DeviceOp.linear(y, mix, wb, A.off["o"], T, D, inner, wdt))
                pending.append((y, "none", None, 0, mult, None, 0))
            else:
                l, W = m["left"], meta["W"]
                H, G, dim, vdim = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
                ops.append(DeviceOp.linear(proj, h, wb, A.off["in"], T, ni, D, wdt, bias=wb, bias_off=A.off["in.b"]))
                cache = pool.buffers[f"l{i}.kv"]
                cw = G * (dim + vdim)
                R = cache.elems // (slots * cw)
                # one launch norms the key heads on their way into the cache and the query heads (with the temperature) in place
                ops.append(DeviceOp.cache_append(ext(cache), proj, ctl, meta["k_col"], 0, T, cw, ni, cw, R, norm_w=wb, norm_off=A.off["k.norm"], normed=G * dim,
                                                 eps=eps, wdt=wdt, norm_group=dim, q_heads=H, q_col=0, q_norm_off=A.off["q.norm"], temp_coef=l["q_temp"]["coef"],
                                                 temp_every=l["q_temp"]["every"]))
                att = scratch("att", T * H * vdim)
                ops.append(DeviceOp.cached_attention(att, proj, ext(cache), ext(cache), ctl, 0, 0, G * dim, T, H, G, 1, dim, vdim, ni, cw, cw, R, l["scale"],
                                                     weights="sigmoid", score_table=ext(self._score_table(owner, R)), table_len=R))
                gru = scratch("gru", T * W)
                ops.append(DeviceOp.min_gru(gru, proj, ext(pool.buffers[f"l{i}.gru"]), ctl, meta["z_col"], meta["z_col"] + W, meta["z_col"] + 2 * W, T, W, ni))
                yr = scratch("right", TD)
                ops.append(DeviceOp.linear(y, att, wb, A.off["left.o"], T, D, H * vdim, wdt))
                ops.append(DeviceOp.linear(yr, gru, wb, A.off["right.o"], T, D, W, wdt))
                # half the sum of the two RMS-normed results, times the multiplier: ONE residual step with two sources
                pending.append((y, "rms", wb, A.off["left.out"], 0.5 * mult, yr, A.off["right.out"]))
            mlp = L["mlp"]
            if mlp is not None:
                open_norm(h, wb, A.off["norm2"])
                if mlp["kind"] == "dense":
                    ff = meta["ff"]
                    u = scratch("ff", T * ff)
                    ops.append(DeviceOp.linear(u, h, wb, A.off["up"], T, ff, D, wdt, act="relu2"))      # the squared ReLU rides in the epilogue
                    ops.append(DeviceOp.linear(y, u, wb, A.off["down"], T, D, ff, wdt))
                else:
                    E, ff, top = meta["E"], meta["ff"], meta["top"]
                    rl, rt = scratch("router", T * E), scratch("route", T * top * 2)
                    ops.append(DeviceOp.linear(rl, h, wb, A.off["router"], T, E, D, wdt))
                    ops.append(DeviceOp.route(rt, rl, wb, A.off["correction"], T, E, top, wdt, mode="corrected_sigmoid", groups=meta["groups"],
                                              groups_kept=meta["keep"]))
                    moe_op = DeviceOp.moe_ffn(y, h, rt, wb, 0, A.off["gate"], A.off["up"], A.off["down"], T, D, ff, E, top, wdt, float("inf"), 1.0,
                                              up_offset=0.0)
                    moe_op.u.seq.buf[4] = scratch("expert", seq_scratch_elems(moe_op))   # the library knows what its kernels stage
                    ops.append(moe_op)
                pending.append((y, "none", None, 0, mult, None, 0))
        logits, rows = None, 0
        if head != "none":
            open_norm(h, gl, GA.off["final.norm"])
            rows = T if head == "all" else 1
            logits = new(rows * cfg.vocab)
            ops.append(DeviceOp.linear(logits, h, gl, GA.off["head"], rows, cfg.vocab, D, wdt, src_off=0 if head == "all" else (T - 1) * D))
        elif keep_layers:
            flush()
        pending.clear()                                 # a step without a head carries state only: its last residual step feeds nothing
        if keep_layers:
            layer_bufs.append(x)
        prog = DeviceProgram(ops, sizes, [], [], externs)
        return LoweredProgram(prog, ctl, logits, rows, layer_bufs if keep_layers else None)

    def close(self):
        for b in list(self.buffers.values()) + list(self._tables.values()):
            b.free()
        self.buffers, self._tables = {}, {}


def synthetic_config(width: int, n_layers: int, heads: int, kv_heads: int, dim: int, experts: int, top: int, ff: int, vocab: int, max_positions: int = 4096,
                     ssm_heads: Optional[int] = None, ssm_vdim: int = 64, state: int = 128, ssm_groups: int = 1, gru_width: Optional[int] = None,
                     expert_groups: int = 4, groups_kept: int = 2) -> dict:
    """config.json contents of a random-init model: layers alternate between the state-space mixer and the pair of sigmoid
    attention and gated recurrent unit; feed-forwards alternate between routed experts and a dense layer as wide as the experts
    a token uses."""
    ssm_heads = ssm_heads or 2 * width // ssm_vdim
    layers = []
    for i in range(n_layers):
        mlp = ({"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": expert_groups, "keep": groups_kept}}}
               if i % 2 == 0 else {"kind": "dense", "ff": top * ff})
        if i % 2 == 0:
            mixer = {"conv": 4, "groups": ssm_groups, "heads": ssm_heads, "norm_groups": ssm_groups, "state": state, "vdim": ssm_vdim}
            layers.append({"type": "mamba2", "mixer": mixer, "mlp": mlp})
        else:
            left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "q_temp": {"coef": 0.1, "every": 1024}}
            layers.append({"type": "parallel", "mixer": {"left": left, "right": {"width": gru_width or width}}, "mlp": mlp})
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "residual_mult": 1.0,
            "max_positions": max_positions, "layers": layers}


def synthetic_tensors(cfg: dict, seed: int = 0):
    """Accessor name -> random f32 tensor of the shape the configuration implies (benchmarks and smoke runs; values are scaled
    like a trained model's so that activations stay O(1))."""
    D = cfg["width"]

    def shape_of(name):
        if name in ("embed", "head"):
            return (cfg["vocab"], D)
        if name == "pos":
            return (cfg["max_positions"], D)
        if name.endswith(".alpha"):
            return ()
        if name.startswith("final.norm"):
            return (D,)
        layer, rest = name.split(".", 1)
        L = cfg["layers"][int(layer[1:])]
        m = L["mixer"]
        if rest.startswith("norm"):
            return (D,)
        if rest.startswith("mlp."):
            part = rest.split(".", 1)[1]
            if L["mlp"]["kind"] == "dense":
                return {"up": (L["mlp"]["ff"], D), "down": (D, L["mlp"]["ff"])}[part]
            E, ff = L["mlp"]["router"]["experts"], L["mlp"]["expert"]["ff"]
            return {"router": (E, D), "correction": (E,), "gate": (ff, D), "up": (ff, D), "down": (D, ff)}[part.split(".")[-1]]
        t = rest[len("mix."):]
        if L["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            C = H * P + 2 * G * N
            return {"in": (2 * H * P + 2 * G * N + H, D), "conv": (C, m["conv"]), "conv.b": (C,), "dt_bias": (H,), "A_log": (H,), "D": (H,), "norm": (H * P,),
                    "o": (D, H * P)}[t]
        l, W = m["left"], m["right"]["width"]
        H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
        return {"left.q": (H * d, D), "left.k": (G * d, D), "left.v": (G * dv, D), "left.q.norm": (d,), "left.k.norm": (d,), "left.r1": (H,), "left.r2": (H,),
                "left.pb": (H,), "left.o": (D, H * dv), "left.out": (D,), "right.z": (W, D), "right.z.b": (W,), "right.x": (W, D), "right.x.b": (W,),
                "right.g": (W, D), "right.o": (D, W), "right.out": (D,)}[t]

    def get(name):
        import zlib
        shp = shape_of(name)
        r = np.random.default_rng([seed, zlib.crc32(name.encode())])
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            return np.array(0.5, np.float32)
        if last in ("norm", "out") or name.endswith((".norm1", ".norm2")) or last in ("q.norm", "k.norm"):
            return np.ones(shp, np.float32)
        if last == "b" or last in ("correction", "dt_bias", "D", "r1", "r2"):
            return (r.random(shp, dtype=np.float32) * 0.2).astype(np.float32)
        if last == "A_log":
            return np.log(1.0 + 3.0 * r.random(shp, dtype=np.float32)).astype(np.float32)
        if last == "pb":
            return (-4.0 - r.random(shp, dtype=np.float32)).astype(np.float32)    # few keys weigh much: sums over a long context stay O(1)
        if name == "pos":
            return ((r.random(shp, dtype=np.float32) - 0.5) * 0.2).astype(np.float32)
        a = r.random(shp, dtype=np.float32)
        a -= 0.5
        a *= np.float32(np.sqrt(12.0 / shp[-1]))
        return a

    return get
