"""Prefill and decode throughput of Setirax next to Pepevik, the framework's closest model (a pair of mixers side by side —
attention and a gated recurrent unit — next to a recurrent mixer behind a short convolution, dense squared-ReLU feed-forwards,
layers that share weights), at equal layer sizes (`bench.py --arch setirax`).

Both models are random-init at shapes that resemble a real model's layers, keep bfloat16 weights and run through the same
`SequenceSession`.  Per arm: tokens / s end to end through the session (host control words, token ids and logits cross PCIe
every step) and device-only (the step's CUDA graph replayed with inputs resident), the HBM bytes a decoded token must move
(active weights + the rings and states it reads and writes) as a fraction of the measured copy bandwidth, and the prefill's
matmul FLOPs as a fraction of the measured dense bf16 throughput.
Timing: wall clock around synchronised replays, after warm-up.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for d in (ROOT, HERE):
    if d not in sys.path:
        sys.path.insert(0, d)

from bench_lududra import SIZES as LUDUDRA_SIZES, peaks, timed  # noqa: E402
from bench_pepevik import SIZES as PEPEVIK_SIZES, pepevik_arm  # noqa: E402

# the feed-forward is as wide as the experts a token of the other arm uses
SIZES = {n: dict(width=s["width"], n_layers=s["n_layers"], heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], ff=s["top"] * s["ff"], vocab=s["vocab"],
                 window=s["window"]) for n, s in LUDUDRA_SIZES.items()}
for n in SIZES:        # three kinds of layers: the stack holds each of them the same number of times
    SIZES[n]["n_layers"] = 3 * max(1, (SIZES[n]["n_layers"] + 1) // 3)


def setirax_arm(be, size, prefill_T, context, reps):
    from zgml_b200.host.session import SequenceSession
    from zgml_b200.host.setirax import SetiraxConfig, SetiraxModel, synthetic_config, synthetic_tensors
    cfgd = synthetic_config(**size)
    cfg = SetiraxConfig.from_dict(cfgd)
    model = SetiraxModel(be, cfg, synthetic_tensors(cfgd), "bfloat16")
    s = SequenceSession(be, model, n_slots=1, max_chunk=prefill_T)
    r = np.random.default_rng(0)
    prompt = r.integers(0, cfg.vocab, context).tolist()
    D = cfg.width
    active = state = 0          # weights / ring and state elements one decoded token touches
    attn_flops = walk_flops = 0  # f32 work of the prefill chunk that is not a matmul
    expand_flops = absorbed_only = 0   # tensor-core work of the expanded latent layers (per step, whatever its length); weights only the absorbed form multiplies
    for i, L in enumerate(cfg.layers):
        m, meta = L["mixer"], model.layer_meta[L["weights"]]
        if L["type"] == "latent_attention":
            H, d, dv, rk, w = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["mask"]["size"]
            active += meta["n_in"] * D + H * rk * (d + dv) + D * H * dv
            state += min(w, context) * rk
            expanded = model._expands(prefill_T, w - 1 + prefill_T, m)      # long bfloat16 steps: keys | values per head from a tensor-core product
            attn_flops += 2 * H * ((d + dv) if expanded else 2 * rk) * prefill_T * min(w, prefill_T / 2)
            if expanded:      # the per-head products of the absorbed form are not run; the ring's rows are expanded once per step instead
                expand_flops += 2 * (w - 1 + prefill_T) * rk * H * (d + dv)
                absorbed_only += H * rk * (d + dv)
        elif L["type"] == "parallel":
            l, rt = m["left"], m["right"]
            w = l["mask"]["size"]
            active += meta["n_in"] * D + rt["heads"] * rt["dim"] * meta["rank_a"] + D * meta["mix"]
            state += min(w, context) * l["kv_heads"] * (l["dim"] + l["vdim"]) + 2 * rt["heads"] * rt["dim"] * rt["vdim"]
            attn_flops += 2 * l["heads"] * (l["dim"] + l["vdim"]) * prefill_T * min(w, prefill_T / 2)
            walk_flops += 5 * rt["heads"] * rt["dim"] * rt["vdim"] * prefill_T
        else:
            W = m["width"]
            active += meta["n_in"] * D + 2 * W * meta["bw"] + D * W
            state += 2 * W
        if L["mlp"] is not None:
            active += 2 * D * meta["ff"]
    body = active
    active += cfg.vocab * D
    out = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "active_params_per_token": active, "layers": [L["type"] for L in cfg.layers]}
    toks = prompt[:prefill_T]
    e2e = timed(lambda: (s.feed("p", toks, [prefill_T - 1]), s.release("p")), be.sync, reps)
    handle = s.program(prefill_T, "last")[1]
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, handle.ptr), be.sync, reps)
    out["prefill"] = {"tokens": prefill_T, "tok_s_e2e": round(prefill_T / e2e), "tok_s_device": round(prefill_T / dev), "ms_device": round(dev * 1e3, 3),
                      "matmul_tflops_device": round((2.0 * ((body - absorbed_only) * prefill_T + cfg.vocab * D) + expand_flops) / dev / 1e12, 1), "attention_gflop_f32": round(attn_flops / 1e9, 1),
                      "walk_gflop_f32": round(walk_flops / 1e9, 1), "kernels": be.program_stats(handle)["kernels"],
                      "tensor_core_linears": be.program_stats(handle)["tensor_core_linears"]}
    s.feed("d", prompt, [])
    tok = [1]
    e2e = timed(lambda: s.feed("d", tok, [0]), be.sync, 4 * reps)
    s.release("d")
    s.feed("d", prompt, [])
    handle = s.program(1, "last")[1]
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, handle.ptr), be.sync, 4 * reps)   # replays rewrite position `context`: same work every time
    bytes_tok = 2 * active + 4 * state
    out["decode"] = {"context": context, "tok_s_e2e": round(1 / e2e, 1), "tok_s_device": round(1 / dev, 1), "us_device": round(dev * 1e6, 1),
                     "bytes_per_token": bytes_tok, "hbm_gbs_device": round(bytes_tok / dev / 1e9, 1), "kernels": be.program_stats(handle)["kernels"]}
    out["dense_gemm_timeouts"] = be.program_stats(handle)["dense_gemm_timeouts"]
    s.close()
    model.close()
    return out


def run(args):
    from zgml_b200 import CudaBackend
    hbm, tf, how = peaks()
    be = CudaBackend(0)
    names = [n for n in (args.sizes.split(",") if args.sizes else SIZES)]
    res = {"bench": "setirax_vs_pepevik", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": how}, "data": "synthetic random-init", "sizes": {}}
    for n in names:
        entry = {"shape": SIZES[n]}
        psize = dict(PEPEVIK_SIZES[n], n_layers=SIZES[n]["n_layers"])          # the same number of layers in both arms
        for arm, fn, size in (("setirax", setirax_arm, SIZES[n]), ("pepevik", pepevik_arm, psize)):
            if getattr(args, "arms", "") and arm not in args.arms.split(","):
                continue
            try:
                e = fn(be, size, args.prefill_tokens, args.context, args.steps)
                e["decode"]["frac_of_hbm"] = round(e["decode"]["hbm_gbs_device"] / hbm, 3)
                e["prefill"]["frac_of_bf16"] = round(e["prefill"]["matmul_tflops_device"] / tf, 3)
                entry[arm] = e
            except Exception as ex:   # one arm failing must not hide the other
                entry[arm] = {"error": repr(ex)}
        res["sizes"][n] = entry
    res["gpu_launches"] = be.launch_count()
    be.close()
    print(json.dumps(res))
