"""Model registry: which loader serves a model file or folder.

A folder with `config.json` is looked up by its `architecture` string; a `.gguf` file is a GGUF-direct quantized LLaMA
(host/gguf.py + host/llama.py).  Every entry returns a session with the same surface — `feed(request, tokens, want)`,
`release(request)`, `step(entries, end)`, `generate(prompt, n, sampler)`, `close()` — so the command line, the trace
replayer and the benches do not care which model they drive.
"""
import json
import os
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import numpy as np

from .sampling import Sampler

_ARCHITECTURES: Dict[str, Callable] = {}


def register(architecture: str):
    def deco(fn):
        _ARCHITECTURES[architecture] = fn
        return fn
    return deco


def architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


@register("Lududra")
def _open_lududra(be, path, dtype, n_slots, max_chunk, max_tokens):
    from .lududra import LududraModel
    from .session import SequenceSession
    model = LududraModel.load(be, path, dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk)


@register("Vemepel")
def _open_vemepel(be, path, dtype, n_slots, max_chunk, max_tokens):
    from .session import SequenceSession
    from .vemepel import VemepelModel
    model = VemepelModel.load(be, path, dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, max_context=max_tokens or None)


@register("Pepevik")
def _open_pepevik(be, path, dtype, n_slots, max_chunk, max_tokens):
    from .pepevik import PepevikModel
    from .session import SequenceSession
    model = PepevikModel.load(be, path, dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, max_context=max_tokens or None)


@register("Setirax")
def _open_setirax(be, path, dtype, n_slots, max_chunk, max_tokens):
    from .session import SequenceSession
    from .setirax import SetiraxModel
    model = SetiraxModel.load(be, path, dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, max_context=max_tokens or None)


class LlamaServingSession:
    """The session surface over `DeviceLlamaSession` (one live request, one token per program execution: the reference's
    decode path).  Quantized GGUF weights run in f32 activations, so `dtype` only accepts "float32"-compatible requests."""

    def __init__(self, be, gguf_path: str, max_tokens: Optional[int] = None):
        from .gguf import GGUFFile, config_from_gguf, load_resident
        from .llama import DeviceLlamaSession
        self.be = be
        gf = GGUFFile.open(gguf_path)
        cfg = config_from_gguf(gf)
        self.weights, self._handles = load_resident(be, gf, cfg)
        self.session = DeviceLlamaSession(be, cfg, self.weights, 1)
        self.vocab, self.cfg, self.live = cfg.vocab_size, cfg, None

    def feed(self, request_id, tokens: Sequence[int], want: Iterable[int] = ()) -> np.ndarray:
        if self.live is None:
            self.live = request_id
            self.session.reset()
        elif self.live != request_id:
            raise RuntimeError("the LLaMA session holds one request at a time")
        want = list(want)
        rows = {}
        for i, t in enumerate(tokens):
            logits = self.session.step(int(t))
            if i in want:
                rows[i] = logits.copy()
        return np.stack([rows[w] for w in want]) if want else np.zeros((0, self.vocab), np.float32)

    def release(self, request_id):
        if self.live == request_id:
            self.live = None

    def step(self, entries, end=()):
        out = [self.feed(e["id"], e["tokens"], e.get("want", ())) for e in entries]
        for r in end:
            self.release(r)
        return out

    def generate(self, prompt, max_new_tokens, sampler: Optional[Sampler] = None, request_id="generate", stop=None):
        sampler = sampler or Sampler()
        logits = self.feed(request_id, prompt, [len(prompt) - 1])[0]
        out = []
        try:
            for _ in range(max_new_tokens):
                out.append(sampler(logits))
                if stop is not None and out[-1] == stop:
                    break
                if len(out) < max_new_tokens:
                    logits = self.feed(request_id, [out[-1]], [0])[0]
        finally:
            self.release(request_id)
        return out

    def close(self):
        self.session.close()
        for h in self._handles:
            h.free()


def open_session(be, path: str, dtype: str = "bfloat16", n_slots: int = 1, max_chunk: int = 256, max_tokens: Optional[int] = None):
    """Load the model at `path` onto `be` and return its serving session."""
    if os.path.isdir(path):
        with open(os.path.join(path, "config.json")) as f:
            arch = json.load(f).get("architecture")
        if arch not in _ARCHITECTURES:
            raise ValueError(f"unknown architecture {arch!r}; known: {architectures()}")
        return _ARCHITECTURES[arch](be, path, dtype, n_slots, max_chunk, max_tokens)
    if path.endswith(".gguf"):
        return LlamaServingSession(be, path, max_tokens)
    raise ValueError(f"{path}: neither a model folder with config.json nor a .gguf file")
