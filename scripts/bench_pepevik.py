"""Prefill and decode throughput of Pepevik next to Lududra, the framework's closest model (a hybrid of a recurrent mixer
behind a short convolution and attention, with routed experts), at equal layer sizes (`bench.py --arch pepevik`).

Both models are random-init at shapes that resemble a real model's layers, keep bfloat16 weights and run through the same
`SequenceSession`.  Per arm: tokens / s end to end through the session (host control words, token ids and logits cross PCIe
every step) and device-only (the step's CUDA graph replayed with inputs resident), the HBM bytes a decoded token must move
(active weights + the cache and states it reads and writes) as a fraction of the measured copy bandwidth, and the prefill's
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

from bench_lududra import SIZES as LUDUDRA_SIZES, lududra_arm, peaks, timed  # noqa: E402

SIZES = {n: dict(width=s["width"], n_layers=s["n_layers"], heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], experts=s["experts"], top=s["top"], ff=s["ff"],
                 vocab=s["vocab"]) for n, s in LUDUDRA_SIZES.items()}


def pepevik_arm(be, size, prefill_T, context, reps):
    from zgml_b200.host.pepevik import PepevikConfig, PepevikModel, synthetic_config, synthetic_tensors
    from zgml_b200.host.session import SequenceSession
    cfgd = synthetic_config(**size, max_positions=context + 64)
    cfg = PepevikConfig.from_dict(cfgd)
    model = PepevikModel(be, cfg, synthetic_tensors(cfgd), "bfloat16")
    s = SequenceSession(be, model, n_slots=1, max_chunk=prefill_T, max_context=context + 64)
    r = np.random.default_rng(0)
    prompt = r.integers(0, cfg.vocab, context).tolist()
    D = cfg.width
    active = state = 0          # weights / cache and state elements one decoded token touches
    scan_flops = attn_flops = 0  # f32 work of the prefill chunk that is not a matmul
    for i, L in enumerate(cfg.layers):
        m, mlp, meta = L["mixer"], L["mlp"], model.layer_meta[L["weights"]]
        if L["type"] == "mamba2":
            inner = meta["inner"]
            active += meta["n_in"] * D + D * inner
            state += 2 * inner * m["state"]                  # read and written
            scan_flops += 6 * inner * m["state"] * prefill_T
        else:
            l, W = m["left"], meta["W"]
            active += meta["n_in"] * D + D * l["heads"] * l["vdim"] + D * W
            state += context * l["kv_heads"] * (l["dim"] + l["vdim"]) + 2 * W
            attn_flops += 2 * l["heads"] * (l["dim"] + l["vdim"]) * prefill_T * prefill_T // 2
        if mlp["kind"] == "dense":
            active += 2 * D * meta["ff"]
        else:
            active += meta["E"] * D + meta["top"] * 3 * D * meta["ff"]
    body = active
    active += cfg.vocab * D
    out = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "active_params_per_token": active, "layers": [L["type"] for L in cfg.layers]}
    toks = prompt[:prefill_T]
    e2e = timed(lambda: (s.feed("p", toks, [prefill_T - 1]), s.release("p")), be.sync, reps)
    handle = s.program(prefill_T, "last")[1]
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, handle.ptr), be.sync, reps)
    out["prefill"] = {"tokens": prefill_T, "tok_s_e2e": round(prefill_T / e2e), "tok_s_device": round(prefill_T / dev), "ms_device": round(dev * 1e3, 3),
                      "matmul_tflops_device": round(2.0 * (body * prefill_T + cfg.vocab * D) / dev / 1e12, 1), "attention_gflop_f32": round(attn_flops / 1e9, 1),
                      "scan_gflop_f32": round(scan_flops / 1e9, 1), "kernels": be.program_stats(handle)["kernels"],
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
    res = {"bench": "pepevik_vs_lududra", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": how}, "data": "synthetic random-init", "sizes": {}}
    for n in names:
        entry = {"shape": SIZES[n]}
        for arm, fn, size in (("pepevik", pepevik_arm, SIZES[n]), ("lududra", lududra_arm, LUDUDRA_SIZES[n])):
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
