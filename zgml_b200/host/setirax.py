"""Setirax: a post-norm decoder stack, x += rms(mixer(x)) w1, x += rms(ff(x)) w2 (the sublayers read the stream itself; only
their results are normed).  A layer's mixer is one of
  * latent attention inside a sliding window: keys and values are expanded per head from one RMS-normed latent, which is all the
    cache holds; no positions; a learned sink per head joins the softmax's denominator,
  * two mixers side by side on the same input, their results added with configured scales: grouped-head attention whose
    queries, keys and values pass a short causal convolution, then rotary positions on a scaled frequency schedule, then a
    weightless RMS norm per head, with smoothly capped scores inside a sliding window; and gated linear attention, a matrix
    state per head that decays per key channel (S <- diag(alpha) S + k v^T, o = S^T q), read out through an RMS norm per head and a
    SiLU gate,
  * a recurrent block with a real-gated linear recurrent unit: a tanh-GELU branch times a convolved branch that passes an
    elementwise recurrence whose two gates are block-diagonal products.
Feed-forwards are dense (squared ReLU, biases) or absent; the head is the embedding table, with smoothly capped logits.  A layer may
run with another layer's weights and a cache or state of its own.

This file is the model's configuration reader, its weight packer and its LOWERING to a DeviceProgram; the arithmetic is in the
sequence-model DeviceOps of the CUDA library (csrc/seqops.cu, csrc/mixops.cu, csrc/recops.cu) and all state in the session's
`SequenceStatePool`.  Every size and per-model constant comes from config.json or a tensor's shape.

latent      [q | dkv] = W x in ONE matmul; CACHE_APPEND norms the latent on its way into the ring.  Short steps run ABSORBED:
            q' = W_uk^T q per head (HEAD_LINEAR), CACHED_ATTENTION of q' over the latent itself (one key head that is also the
            value, window mask, sinks), then W_uv per head (HEAD_LINEAR) and W_o.  Scores (W_uk^T q) . c = q . (W_uk c) are the
            same numbers in another order of summation.  Long steps of bfloat16 sessions run EXPANDED: one tensor-core product
            turns every row of the sequence's ring into keys | values per head (program scratch, recomputed by each such step),
            and ordinary multi-head attention runs over them.  Only the latent is ever cached.
pair        [q | k | v | q' | k' | v' | g | a1] = W x in ONE matmul for both branches.  Left: CAUSAL_CONV over q | k | v, CACHE_APPEND
            (every key head turned by its rotary position — frequencies from a table evaluated at load — then brought to unit RMS on
            its way into the ring, values copied, query heads turned and normed in place), CACHED_ATTENTION (cap, window) writing left_scale * heads into the left
            columns of a shared row.  Right: the decay logits' second stage (LINEAR), DELTA_RULE in its plain form (no unit
            vectors, no correction; tempered-sigmoid decay; SiLU gate) writing right_scale * heads into the right columns.  ONE
            matmul over the shared row with [W_o left | W_o right] is the scaled sum of the two branches.
rglru       [y | x] = W h + b in ONE matmul; CAUSAL_CONV (bias) over x; the two gates' block-diagonal products as ONE HEAD_LINEAR
            over the stacked blocks; RG_LRU (tanh-GELU of y on the way out); W_o.
"""
import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .. import abi
from ..backend import CudaBackend, DeviceBuffer, DeviceOp, DeviceProgram, ExternBuffer
from .safetensors import SafetensorsFile
from .session import LoweredProgram
from .state import SequenceStatePool, StateSpec
from .weights import WeightArena

ARCHITECTURE = "Setirax"
DEFAULT_CONTEXT = 4096     # positions a sequence may reach when a layer attends without a window and the caller names no bound
MIXERS = ("latent_attention", "parallel", "rglru")
LRU_RATE = 8.0             # log a = -8 r softplus(lam): fixed by the design
EXPAND_MIN_TOKENS = 128    # steps from this size on expand a latent layer's keys and values per head (bfloat16 sessions)


def rotary_frequencies(rot: dict) -> np.ndarray:
    """[dims / 2] f32: pair i turns by p * f_i, f_i = base^(-2i / dims).  With `scaling` (factor, low, high, original): a pair whose
    wavelength 2 pi / f is shorter than original / high keeps f, one longer than original / low turns `factor` times slower, and
    in between the two are blended linearly in original / wavelength."""
    dims = int(rot["dims"])
    f = float(rot["base"]) ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        wl = 2.0 * math.pi / f
        blend = (original / wl - low) / (high - low) if high != low else np.ones_like(f)
        mixed = (1.0 - blend) * f / factor + blend * f
        f = np.where(wl < original / high, f, np.where(wl > original / low, f / factor, mixed))
    return f.astype(np.float32)


def _tensor_sizes(kind: str, m: dict, mlp: Optional[dict]) -> tuple:
    """What of a layer's entry sizes its tensors: two layers that share weights must agree on it (constants such as a window, a
    scale or a cap may differ; each layer runs with its own)."""
    if kind == "latent_attention":
        t = (m["heads"], m["dim"], m["vdim"], m["kv_rank"])
    elif kind == "parallel":
        l, r = m["left"], m["right"]
        t = (l["heads"], l["kv_heads"], l["dim"], l["vdim"], int(l.get("conv") or 0), r["heads"], r["dim"], r["vdim"])
    else:
        t = (m["width"], m["blocks"], int(m.get("conv") or 1))
    return t + ((mlp.get("ff"),) if mlp else ())


def _window(m: dict) -> Optional[int]:
    mask = m.get("mask")
    return int(mask["size"]) if mask else None


@dataclass(frozen=True)
class SetiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float       # 0: none
    layers: tuple              # of dicts: {"type", "mixer", "mlp", "weights": index of the layer whose tensors it uses}

    @classmethod
    def from_dict(cls, c: dict) -> "SetiraxConfig":
        if c.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} config: architecture = {c.get('architecture')!r}")
        layers = []
        for i, L in enumerate(c["layers"]):
            kind, m, mlp = L["type"], L["mixer"], L.get("mlp")
            if kind not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            owner, seen = i, {i}
            while "weights_of" in c["layers"][owner]:       # the layer whose tensors it runs with, through any chain of references
                owner = c["layers"][owner]["weights_of"]
                if not isinstance(owner, int) or not (0 <= owner < len(c["layers"])) or owner in seen:
                    raise ValueError(f"layer {i}: weights_of must lead to a layer with tensors of its own")
                seen.add(owner)
            if owner != i:
                o = c["layers"][owner]
                if o["type"] != kind or (o.get("mlp") is None) != (mlp is None) or _tensor_sizes(kind, o["mixer"], o.get("mlp")) != _tensor_sizes(kind, m, mlp):
                    raise ValueError(f"layer {i}: its sizes differ from layer {owner}'s, whose weights it uses")
            if kind == "latent_attention":
                if min(m["heads"], m["dim"], m["vdim"], m["kv_rank"]) < 1:
                    raise ValueError(f"layer {i}: sizes must be positive")
            elif kind == "parallel":
                l, r = m["left"], m["right"]
                if l["heads"] % l["kv_heads"]:
                    raise ValueError(f"layer {i}: heads not a multiple of kv_heads")
                rot = l.get("rot")
                if rot and (rot["dims"] % 2 or rot["dims"] > l["dim"] or rot["dims"] < 2):
                    raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
                if not (r["tau"] > 0):
                    raise ValueError(f"layer {i}: tau must be positive")
            else:
                if m["width"] % m["blocks"] or m.get("conv", 1) < 1:
                    raise ValueError(f"layer {i}: width must divide into blocks, conv >= 1")
            for part in ([m] if kind == "latent_attention" else [m["left"]] if kind == "parallel" else []):
                w = _window(part)
                if w is not None and w < 1:
                    raise ValueError(f"layer {i}: mask.size must be positive")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append({"type": kind, "mixer": m, "mlp": mlp, "weights": owner})
        return cls(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), float(c.get("logit_softcap") or 0.0), tuple(layers))

    @classmethod
    def from_json(cls, path: str) -> "SetiraxConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))


class SetiraxModel:
    """Weights resident in HBM (one arena per layer that has tensors + one for the embedding and the final norm) and the lowering."""

    def __init__(self, be: CudaBackend, cfg: SetiraxConfig, tensors, dtype: str = "bfloat16", has=None):
        """tensors: name -> f32 array accessor (`tensors(name)`), e.g. SafetensorsFile.f32; `has(name)`: whether a tensor exists."""
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.be, self.cfg, self.dtype = be, cfg, dtype
        self.wdt = abi.W_BF16 if dtype == "bfloat16" else abi.W_F32
        self.vocab, self.width = cfg.vocab, cfg.width
        self.layer_meta: Dict[int, dict] = {}
        self.arenas: Dict[int, WeightArena] = {}
        self.buffers: Dict[int, DeviceBuffer] = {}
        self._freqs: Dict[int, DeviceBuffer] = {}
        self.expand_float32 = False      # float32 sessions keep latent layers absorbed; set before the first long step to run them expanded as well
        # a layer that attends without a window caches every position: the session then bounds the sequence
        self.bounded_context = any(_window(L["mixer"] if L["type"] == "latent_attention" else L["mixer"]["left"]) is None
                                   for L in cfg.layers if L["type"] != "rglru")
        has = has or (lambda name: True)
        D = cfg.width

        def get(name, shape):
            t = tensors(name)
            assert tuple(t.shape) == tuple(shape), f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}"
            return t

        for i, L in enumerate(cfg.layers):
            if L["weights"] != i:
                continue
            p, m = f"l{i}.", L["mixer"]
            A = WeightArena(self.wdt)
            meta = {}
            A.add("norm1", get(p + "norm1", (D,)))
            if L["type"] == "latent_attention":
                H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
                A.add("in", np.concatenate([get(p + "mix.q", (H * dim, D)), get(p + "mix.dkv", (rank, D))], 0))
                A.add("dkv.norm", get(p + "mix.dkv.norm", (rank,)))
                uk, uv = get(p + "mix.uk", (H * dim, rank)), get(p + "mix.uv", (H * vdim, rank))
                A.add("ukT", uk.reshape(H, dim, rank).transpose(0, 2, 1))     # [H, rank, dim]: q' = W_uk^T q per head
                A.add("uv", uv)                                               # [H, vdim, rank] as stored
                A.add("ukv", np.concatenate([uk, uv], 0))                     # long steps expand keys | values of the ring's rows in one product
                meta["sink"] = has(p + "mix.sink")
                if meta["sink"]:
                    A.add("sink", get(p + "mix.sink", (H,)))
                A.add("o", get(p + "mix.o", (D, H * vdim)))
                meta.update(n_in=H * dim + rank)
            elif L["type"] == "parallel":
                l, r = m["left"], m["right"]
                H, G, dim, vdim = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
                Hr, dr, vr = r["heads"], r["dim"], r["vdim"]
                pl, pr = p + "mix.left.", p + "mix.right."
                a1 = tensors(pr + "a1")
                ra = a1.shape[0]
                C = H * dim + G * (dim + vdim)
                A.add("in", np.concatenate([get(pl + "q", (H * dim, D)), get(pl + "k", (G * dim, D)), get(pl + "v", (G * vdim, D)),
                                            get(pr + "q", (Hr * dr, D)), get(pr + "k", (Hr * dr, D)), get(pr + "v", (Hr * vr, D)),
                                            get(pr + "g", (Hr * vr, D)), get(pr + "a1", (ra, D))], 0))
                taps = int(l.get("conv") or 0)
                if taps:
                    A.add("conv", np.concatenate([get(pl + "q.conv", (H * dim, taps)), get(pl + "k.conv", (G * dim, taps)), get(pl + "v.conv", (G * vdim, taps))], 0))
                A.add("unit", np.ones(dim, np.float32))                       # the weightless per-head norm, as a weight of ones
                A.add("a2", get(pr + "a2", (Hr * dr, ra)))
                A.add("a2.b", get(pr + "a2.b", (Hr * dr,)))
                A.add("gla.norm", get(pr + "norm", (vr,)))
                A.add("o", np.concatenate([get(pl + "o", (D, H * vdim)), get(pr + "o", (D, Hr * vr))], 1))    # one product = the sum of both branches
                rq = C
                meta.update(n_in=C + 2 * Hr * dr + 2 * Hr * vr + ra, C=C, taps=taps, rank_a=ra, rq=rq, rk=rq + Hr * dr, rv=rq + 2 * Hr * dr,
                            rg=rq + 2 * Hr * dr + Hr * vr, ra1=rq + 2 * Hr * dr + 2 * Hr * vr, mix=H * vdim + Hr * vr)
            else:
                W, B = m["width"], m["blocks"]
                bw, taps = W // B, int(m.get("conv") or 1)
                A.add("in", np.concatenate([get(p + "mix.y", (W, D)), get(p + "mix.x", (W, D))], 0))
                A.add("in.b", np.concatenate([get(p + "mix.y.b", (W,)), get(p + "mix.x.b", (W,))]))
                if taps > 1 or has(p + "mix.conv"):
                    A.add("conv", get(p + "mix.conv", (W, taps)))
                    A.add("conv.b", get(p + "mix.conv.b", (W,)))
                    meta["conv"] = True
                A.add("gates", np.concatenate([get(p + "mix.ra", (B, bw, bw)), get(p + "mix.ri", (B, bw, bw))], 1))     # [B, 2 bw, bw]: both gates of a block in one product
                A.add("ra.b", get(p + "mix.ra.b", (B, bw)))
                A.add("ri.b", get(p + "mix.ri.b", (B, bw)))
                A.add("lam", get(p + "mix.lam", (W,)))
                A.add("o", get(p + "mix.o", (D, W)))
                meta.update(n_in=2 * W, taps=taps, bw=bw)
            if L["mlp"] is not None:
                up = tensors(p + "mlp.up")
                ff = up.shape[0]
                assert ff == L["mlp"].get("ff", ff), f"{p}mlp.up: {ff} rows, the configuration says {L['mlp'].get('ff')}"
                A.add("norm2", get(p + "norm2", (D,)))
                A.add("up", get(p + "mlp.up", (ff, D)))
                A.add("up.b", get(p + "mlp.up.b", (ff,)))
                A.add("down", get(p + "mlp.down", (D, ff)))
                A.add("down.b", get(p + "mlp.down.b", (D,)))
                meta.update(ff=ff)
            self.layer_meta[i], self.arenas[i] = meta, A
            self.buffers[i] = A.upload(be)
        for i, L in enumerate(cfg.layers):      # a frequency table per layer that turns its heads: the schedule is the layer's own constant
            rot = L["mixer"]["left"].get("rot") if L["type"] == "parallel" else None
            if rot:
                f = rotary_frequencies(rot)
                self._freqs[i] = DeviceBuffer(be, max(f.nbytes, 16), zero=False)
                self._freqs[i].upload(np.ascontiguousarray(np.concatenate([f, np.zeros(max(0, 4 - f.size), np.float32)])))
        A = WeightArena(self.wdt)
        A.add("embed", get("embed", (cfg.vocab, D)))
        A.add("final.norm", get("final.norm", (D,)))
        self.arenas[-1] = A
        self.buffers[-1] = A.upload(be)

    @classmethod
    def load(cls, be: CudaBackend, model_dir: str, dtype: str = "bfloat16") -> "SetiraxModel":
        cfg = SetiraxConfig.from_json(os.path.join(model_dir, "config.json"))
        sf = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
        try:
            return cls(be, cfg, sf.f32, dtype, has=sf.__contains__)
        finally:
            sf.close()

    def weight_bytes(self) -> int:
        return sum(b.nbytes for b in self.buffers.values())

    # ── state ──
    def capacity(self, max_chunk: int, max_context: Optional[int]) -> int:
        """Positions a sequence may reach where a layer keeps every position (no window)."""
        return max(int(max_context) if max_context else DEFAULT_CONTEXT, max_chunk)

    def _rows(self, window: Optional[int], max_chunk: int, max_context: Optional[int]) -> int:
        """Rows of a key ring: what the window reaches back plus one step; every position where there is no window."""
        cap = self.capacity(max_chunk, max_context)
        return cap if window is None else window - 1 + max_chunk

    def state_specs(self, max_chunk: int, max_context: Optional[int] = None) -> List[StateSpec]:
        specs = []
        for i, L in enumerate(self.cfg.layers):
            m = L["mixer"]
            if L["type"] == "latent_attention":
                specs.append(StateSpec(f"l{i}.latent", self._rows(_window(m), max_chunk, max_context) * m["kv_rank"], False))    # masked by position: no clearing
            elif L["type"] == "parallel":
                l, r = m["left"], m["right"]
                specs.append(StateSpec(f"l{i}.kv", self._rows(_window(l), max_chunk, max_context) * l["kv_heads"] * (l["dim"] + l["vdim"]), False))
                taps = int(l.get("conv") or 0)
                if taps > 1:
                    specs.append(StateSpec(f"l{i}.tail", (taps - 1) * (l["heads"] * l["dim"] + l["kv_heads"] * (l["dim"] + l["vdim"])), True))
                specs.append(StateSpec(f"l{i}.gla", r["heads"] * r["dim"] * r["vdim"], True))
            else:
                taps = int(m.get("conv") or 1)
                if taps > 1:
                    specs.append(StateSpec(f"l{i}.tail", (taps - 1) * m["width"], True))
                specs.append(StateSpec(f"l{i}.lru", m["width"], True))
        return specs

    def _expands(self, T: int, R: int, m: dict) -> bool:
        """Whether a step of T tokens runs a latent layer in the expanded form.  Expanding costs 2 R rank H (dim + vdim) FLOPs on the
        tensor cores per step; the absorbed form costs (2 rank - dim - vdim) more multiply-adds per (query, key, head) in f32.  Worth it
        for long steps of bfloat16 sessions whose latent fits the tensor-core product (rank a multiple of 8, at least 64); float32
        sessions, whose products are exact f32 tiles either way, and short steps stay absorbed."""
        rank, per_head = m["kv_rank"], m["dim"] + m["vdim"]
        return (self.wdt == abi.W_BF16 or self.expand_float32) and T >= EXPAND_MIN_TOKENS and rank % 8 == 0 and rank >= 64 and 2 * rank > per_head

    # ── lowering ──
    def lower(self, T: int, head: str, pool: SequenceStatePool, keep_layers: bool = False) -> LoweredProgram:
        cfg, wdt, D, eps = self.cfg, self.wdt, self.cfg.width, self.cfg.norm_eps
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
        y = new(TD)
        proj = new(T * max(m["n_in"] for m in self.layer_meta.values()))
        shared: Dict[str, int] = {}

        def scratch(name, n):      # activations reused by every layer that needs them
            if name not in shared or sizes[shared[name]] < n:
                shared[name] = new(n)
            return shared[name]

        x = xs[0]
        ops.append(DeviceOp.embed(x, ctl, gl, GA.off["embed"], T, D, 1.0, wdt))

        sublayers = sum(1 + (L["mlp"] is not None) for L in cfg.layers)
        h = scratch("head.in", TD) if head != "none" else None

        def close(wb, w_off):      # x <- x + rms(y) w: the norm sits on the sublayer's result only
            nonlocal x, sublayers
            nx = new(TD) if keep_layers else (xs[1] if x == xs[0] else xs[0])
            sublayers -= 1
            if sublayers == 0 and h is not None:      # the stack's last residual step and the model's final norm are one launch
                ops.append(DeviceOp.norm(nx, y, wb, w_off, T, D, eps, wdt, kind="rms", res=x, then=h, then_w=gl, then_w_off=GA.off["final.norm"], then_kind="rms"))
            else:
                ops.append(DeviceOp.norm(nx, y, wb, w_off, T, D, eps, wdt, kind="rms", res=x))
            x = nx

        layer_bufs = []
        slots = pool.n_slots
        for i, L in enumerate(cfg.layers):
            owner = L["weights"]
            m, meta, A, wb = L["mixer"], self.layer_meta[owner], self.arenas[owner], ext(self.buffers[owner])
            ni = meta["n_in"]
            if L["type"] == "latent_attention":
                H, dim, vdim, rank = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
                window = _window(m)
                ops.append(DeviceOp.linear(proj, x, wb, A.off["in"], T, ni, D, wdt))
                cache = pool.buffers[f"l{i}.latent"]
                R = cache.elems // (slots * rank)
                ops.append(DeviceOp.cache_append(ext(cache), proj, ctl, H * dim, 0, T, rank, ni, rank, R, norm_w=wb, norm_off=A.off["dkv.norm"], normed=rank, eps=eps, wdt=wdt))
                att = scratch("att", T * H * vdim)
                sink = dict(sink=wb if meta["sink"] else None, sink_off=A.off.get("sink", 0), sink_wdt=wdt)
                mask = dict(mask="causal" if window is None else "window", mask_size=window or 0)
                if self._expands(T, R, m):
                    # EXPANDED form: keys | values of every ring row per head from ONE tensor-core product over the slot's latents, then
                    # ordinary multi-head attention over them: dim + vdim numbers per (query, key, head) instead of 2 rank
                    kvw = H * (dim + vdim)
                    kv = scratch("latent.kv", R * kvw)
                    ops.append(DeviceOp.linear(kv, ext(cache), wb, A.off["ukv"], R, kvw, rank, wdt, ctl=ctl, src_slot_stride=R * rank))
                    ops.append(DeviceOp.cached_attention(att, proj, kv, kv, ctl, 0, 0, H * dim, T, H, H, 1, dim, vdim, ni, kvw, kvw, R, m["scale"], unslotted=True, **mask, **sink))
                else:
                    # ABSORBED form: q' = W_uk^T q per head, attention of q' over the latent itself (one key head that is also the value), W_uv per head
                    qa = scratch("qa", T * H * rank)
                    ops.append(DeviceOp.head_linear(qa, proj, wb, A.off["ukT"], T, H, rank, dim, wdt, src_hs=dim, src_rs=ni))
                    ctx = scratch("ctx", T * H * rank)
                    ops.append(DeviceOp.cached_attention(ctx, qa, ext(cache), ext(cache), ctl, 0, 0, 0, T, H, 1, 1, rank, rank, H * rank, rank, rank, R, m["scale"], **mask, **sink))
                    ops.append(DeviceOp.head_linear(att, ctx, wb, A.off["uv"], T, H, vdim, rank, wdt))
                ops.append(DeviceOp.linear(y, att, wb, A.off["o"], T, D, H * vdim, wdt))
            elif L["type"] == "parallel":
                l, r = m["left"], m["right"]
                H, G, dim, vdim = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
                Hr, dr, vr = r["heads"], r["dim"], r["vdim"]
                C, taps, window = meta["C"], meta["taps"], _window(l)
                ops.append(DeviceOp.linear(proj, x, wb, A.off["in"], T, ni, D, wdt))
                if taps:
                    qkv, qrs = scratch("conv", T * C), C
                    tail = ext(pool.buffers[f"l{i}.tail"]) if taps > 1 else ctl    # one tap: no carried inputs, the operand is unused
                    ops.append(DeviceOp.causal_conv(qkv, proj, wb, A.off["conv"], tail, ctl, T, C, taps, wdt, "none", src_rs=ni))
                else:
                    qkv, qrs = proj, ni
                rot = l.get("rot")
                cache = pool.buffers[f"l{i}.kv"]
                cw = G * (dim + vdim)
                R = cache.elems // (slots * cw)
                # one launch: every key head turned by its position, brought to unit RMS and written into the ring, values copied, every
                # query head turned and brought to unit RMS in place
                ops.append(DeviceOp.cache_append(ext(cache), qkv, ctl, H * dim, 0, T, cw, qrs, cw, R, norm_w=wb, norm_off=A.off["unit"], normed=G * dim, eps=eps, wdt=wdt,
                                                 norm_group=dim, q_heads=H, q_col=0, q_norm_off=A.off["unit"], rot_layout="halves", head_rot=rot["dims"] if rot else 0,
                                                 rot_base=rot["base"] if rot else 0.0, freqs=ext(self._freqs[i]) if rot else None))
                mw = meta["mix"]
                mix = scratch("mix", T * mw)
                ops.append(DeviceOp.cached_attention(mix, qkv, ext(cache), ext(cache), ctl, 0, 0, G * dim, T, H, G, 1, dim, vdim, qrs, cw, cw, R, l["scale"],
                                                     mask="causal" if window is None else "window", mask_size=window or 0, softcap=float(l.get("softcap") or 0.0),
                                                     out_scale=m["left_scale"], dst_rs=mw, dst_col=0))
                a = scratch("decay", T * Hr * dr)
                ops.append(DeviceOp.linear(a, proj, wb, A.off["a2"], T, Hr * dr, meta["rank_a"], wdt, src_off=meta["ra1"], src_rs=ni))
                ops.append(DeviceOp.delta_rule(mix, proj, None, a, proj, wb, ext(pool.buffers[f"l{i}.gla"]), ctl, meta["rq"], meta["rk"], meta["rv"], 0, 0, A.off["a2.b"],
                                               A.off["gla.norm"], T, Hr, Hr, dr, vr, ni, 0, Hr * dr, ni, wdt, eps, 0.0, dr ** -0.5, gate_off=meta["rg"], plain=True,
                                               decay_tau=r["tau"], silu_gate=True, out_scale=m["right_scale"], dst_rs=mw, dst_col=H * vdim))
                ops.append(DeviceOp.linear(y, mix, wb, A.off["o"], T, D, mw, wdt))
            else:
                W, bw, taps = m["width"], meta["bw"], meta["taps"]
                ops.append(DeviceOp.linear(proj, x, wb, A.off["in"], T, ni, D, wdt, bias=wb, bias_off=A.off["in.b"]))
                if meta.get("conv"):
                    u, u_rs, u_col = scratch("lru.u", T * W), W, 0
                    tail = ext(pool.buffers[f"l{i}.tail"]) if taps > 1 else ctl
                    ops.append(DeviceOp.causal_conv(u, proj, wb, A.off["conv"], tail, ctl, T, W, taps, wdt, "none", src_off=W, src_rs=ni, bias_off=A.off["conv.b"]))
                else:
                    u, u_rs, u_col = proj, ni, W
                gates = scratch("lru.gates", T * 2 * W)
                ops.append(DeviceOp.head_linear(gates, u, wb, A.off["gates"], T, W // bw, 2 * bw, bw, wdt, src_col=u_col, src_hs=bw, src_rs=u_rs))
                rec = scratch("lru.out", T * W)
                ops.append(DeviceOp.rg_lru(rec, u, gates, proj, wb, ext(pool.buffers[f"l{i}.lru"]), ctl, u_col, 0, bw, 0, A.off["ra.b"], A.off["ri.b"], A.off["lam"],
                                           T, W, u_rs, 2 * W, bw, 2 * bw, ni, wdt, rate=LRU_RATE, y_act="gelu_tanh"))
                ops.append(DeviceOp.linear(y, rec, wb, A.off["o"], T, D, W, wdt))
            close(wb, A.off["norm1"])
            if L["mlp"] is not None:
                ff = meta["ff"]
                up = scratch("ff", T * ff)
                ops.append(DeviceOp.linear(up, x, wb, A.off["up"], T, ff, D, wdt, bias=wb, bias_off=A.off["up.b"], act="relu2"))      # the squared ReLU rides in the epilogue
                ops.append(DeviceOp.linear(y, up, wb, A.off["down"], T, D, ff, wdt, bias=wb, bias_off=A.off["down.b"]))
                close(wb, A.off["norm2"])
            if keep_layers:
                layer_bufs.append(x)
        logits, rows = None, 0
        if head != "none":
            rows = T if head == "all" else 1
            if not cfg.layers:
                ops.append(DeviceOp.norm(h, x, gl, GA.off["final.norm"], T, D, eps, wdt, kind="rms"))
            logits = new(rows * cfg.vocab)
            cap = cfg.logit_softcap
            ops.append(DeviceOp.linear(logits, h, gl, GA.off["embed"], rows, cfg.vocab, D, wdt, src_off=0 if head == "all" else (T - 1) * D,
                                       act="softcap" if cap else None, act_param=cap))       # the head is the embedding table; the cap rides in the epilogue
        prog = DeviceProgram(ops, sizes, [], [], externs)
        return LoweredProgram(prog, ctl, logits, rows, layer_bufs if keep_layers else None)

    def close(self):
        for b in list(self.buffers.values()) + list(self._freqs.values()):
            b.free()
        self.buffers, self._freqs = {}, {}


def synthetic_config(width: int, n_layers: int, heads: int, kv_heads: int, dim: int, ff: int, vocab: int, window: int = 1024, kv_rank: int = 512,
                     gla_heads: Optional[int] = None, lru_width: Optional[int] = None, lru_blocks: Optional[int] = None, conv: int = 4) -> dict:
    """config.json contents of a random-init model: layers cycle latent attention, the pair and the recurrent block; every layer
    but the recurrent ones has a dense feed-forward."""
    layers = []
    for i in range(n_layers):
        kind = MIXERS[i % 3]
        if kind == "latent_attention":
            mixer = {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": kv_rank, "mask": {"size": window}, "scale": dim ** -0.5}
        elif kind == "parallel":
            left = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "scale": 8.0 / dim, "softcap": 50.0, "vdim": dim,
                    "rot": {"base": 10000.0, "dims": dim, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 4096}}}
            right = {"dim": dim, "heads": gla_heads or max(1, heads // 2), "tau": 8.0, "vdim": dim}
            mixer = {"left": left, "left_scale": 0.5, "right": right, "right_scale": 0.5}
        else:
            mixer = {"blocks": lru_blocks or heads, "conv": conv, "width": lru_width or width}
        layers.append({"type": kind, "mixer": mixer, "mlp": None if kind == "rglru" else {"kind": "dense", "ff": ff}})
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 50.0, "layers": layers}


def synthetic_tensors(cfg: dict, seed: int = 0, decay_rank: int = 64):
    """Accessor name -> random f32 tensor of the shape the configuration implies (benchmarks and smoke runs; values are scaled like a
    trained model's so that activations stay O(1))."""
    D = cfg["width"]

    def shape_of(name):
        if name == "embed":
            return (cfg["vocab"], D)
        if name == "final.norm":
            return (D,)
        layer, rest = name.split(".", 1)
        L = cfg["layers"][int(layer[1:])]
        m = L["mixer"]
        if rest in ("norm1", "norm2"):
            return (D,)
        if rest.startswith("mlp."):
            ff = L["mlp"]["ff"]
            return {"up": (ff, D), "up.b": (ff,), "down": (D, ff), "down.b": (D,)}[rest[4:]]
        t = rest[len("mix."):]
        if L["type"] == "latent_attention":
            H, d, dv, rk = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            return {"q": (H * d, D), "dkv": (rk, D), "dkv.norm": (rk,), "uk": (H * d, rk), "uv": (H * dv, rk), "sink": (H,), "o": (D, H * dv)}[t]
        if L["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, d, dv, taps = l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["conv"]
            Hr, dr, vr = r["heads"], r["dim"], r["vdim"]
            return {"left.q": (H * d, D), "left.k": (G * d, D), "left.v": (G * dv, D), "left.q.conv": (H * d, taps), "left.k.conv": (G * d, taps), "left.v.conv": (G * dv, taps),
                    "left.o": (D, H * dv), "right.q": (Hr * dr, D), "right.k": (Hr * dr, D), "right.v": (Hr * vr, D), "right.g": (Hr * vr, D), "right.a1": (decay_rank, D),
                    "right.a2": (Hr * dr, decay_rank), "right.a2.b": (Hr * dr,), "right.norm": (vr,), "right.o": (D, Hr * vr)}[t]
        W, B, taps = m["width"], m["blocks"], m["conv"]
        bw = W // B
        return {"y": (W, D), "y.b": (W,), "x": (W, D), "x.b": (W,), "conv": (W, taps), "conv.b": (W,), "ra": (B, bw, bw), "ra.b": (B, bw), "ri": (B, bw, bw), "ri.b": (B, bw),
                "lam": (W,), "o": (D, W)}[t]

    def get(name):
        import zlib
        shp = shape_of(name)
        r = np.random.default_rng([seed, zlib.crc32(name.encode())])
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            return np.ones(shp, np.float32)
        if last == "conv":
            a = (r.random(shp, dtype=np.float32) - 0.5) * 0.5
            a[:, -1] += 1.0
            return a
        if name.endswith("a2.b"):
            return (2.0 + r.random(shp, dtype=np.float32)).astype(np.float32)
        if last == "lam":
            return (-3.0 + 2.0 * r.random(shp, dtype=np.float32)).astype(np.float32)
        if last in ("b", "sink"):
            return (r.random(shp, dtype=np.float32) * 0.2).astype(np.float32)
        a = r.random(shp, dtype=np.float32)
        a -= 0.5
        a *= np.float32(np.sqrt(12.0 / shp[-1]))
        return a

    return get
