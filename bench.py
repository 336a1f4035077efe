#!/usr/bin/env python
"""bench.py — BASELINE.json metric on B200: Llama decode tok/s at 1/2/4/8 GPUs (value) and quantized GEMV HBM GB/s (gemv).

Two legs per run, ONE JSON line:

* `value` / `e2e` — greedy decode of the Llama-3-70B-shape Q4_0 model (BASELINE.json configs[4]): batch 1, context 512,
  every linear row-sharded over the N GPUs of the box (2 NVLink peer all-reduces per layer + 1 NCCL all-gather per token
  inside the step's CUDA graph); at N = 1 the same 39 GB model runs on one GPU.  STRONG scaling: the work per token is
  fixed, `value` = tokens/s of the whole job.  A "step" is one decode token.
    value : device-timed graph replays, inputs resident in HBM (CUDA events on the launching stream, max over ranks)
    e2e   : LlamaInferenceSession.step through refresh_program + execute_program with HOST buffers: embedding row, mask
            and RoPE leaves uploaded, logits downloaded, argmax on the host — every token
  `check` carries the correctness evidence: the greedy tokens and a logits probe of the first steps (the synthetic
  model is the same at every N, so they must agree across N) and a 2-layer 70B-width model against the CPU oracle.
* `gemv` / `roofline` — the quantized matvec microbenchmark (configs[1]): for every case (K x N in {4096x4096,
  4096x14336}) x (int8+f32 scale, Q8_0-origin, Q4_0-origin), one batch-1 matvec over EACH of R distinct GPU-resident
  weight copies (R x bytes >= 512 MB > 4 x L2: every weight byte comes from HBM).  `roofline` is its dominant kernel —
  qgemv_kernel, the kernel that also dominates the decode step — against MEASURED_PEAKS.json hbm_gbs.
  Algorithmic bytes per GEMV = (K*N/32)*B_blk + 4K + 4N, B_blk = 36 / 34 / 18.

`cpu_baseline` / `--impl reference`: the oracle executor (reference semantics, oracle/zgml_oracle.c) decoding the same
70B-shape model on the host cores — a bounded sample: 1- and 2-layer models at full width with the full LM head, per-token
time extrapolated linearly to 80 layers (t1 + 79 (t2 - t1)); 1 thread for cpu_baseline (the reference runs its matmul
single-threaded, src/inference_utils.zig:192), all host threads for the reference arm.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 14336)]          # (K, N): zgml rows=K, cols=N
FORMATS = [("i8_f32", 36), ("q8_0", 34), ("q4_0", 18)]
if os.environ.get("ZG_BENCH_SHAPES"):            # kernel-tuning sweeps only (not the default workload)
    SHAPES = [tuple(int(v) for v in t.split("x")) for t in os.environ["ZG_BENCH_SHAPES"].split(",")]
if os.environ.get("ZG_BENCH_FORMATS"):
    FORMATS = [f for f in FORMATS if f[0] in os.environ["ZG_BENCH_FORMATS"].split(",")]
ROTATION_BYTES = 512 << 20
METRIC = "llama_decode_tok_s"
UNIT = "tok/s"
GEMV_METRIC = "quant_gemv_hbm_gbps"
DECODE_CONTEXT = 512
DECODE_KIND = "q4_0"


def alg_bytes(K, N, blk):
    return (K * N // 32) * blk + 4 * K + 4 * N


def host_weight(K, N, fmt, seed):
    """Synthetic weight in the reference's host form (i8 data + f32 scales, bs=32), the quantized-GEMM configuration of the bench."""
    r = np.random.default_rng(seed)
    if fmt == "q4_0":
        data = r.integers(-8, 8, K * N, dtype=np.int8)
    else:
        data = r.integers(-127, 128, K * N, dtype=np.int8)
    scales = r.uniform(1e-3, 1e-2, K * N // 32).astype(np.float32)
    if fmt != "i8_f32":
        scales = scales.astype(np.float16).astype(np.float32)  # GGUF-origin scales are exact f16
    return data, scales


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock + throttle reasons sampled DURING the timed region (NVML; nvidia-smi fallback)."""
    BAD = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
    NOTE = {"sw_power_cap": 0x4}

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _sample(self):
        if self.nv is not None:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            try:
                bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                bits = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            for name, bit in {**self.BAD, **self.NOTE}.items():
                if bits & bit:
                    self.reasons.add(name)
        else:
            out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm,"
                                  "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap",
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True).stdout.strip().split(",")
            if len(out) >= 6:
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
                for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], out[2:6]):
                    if v.strip() == "Active":
                        self.reasons.add(name)

    def _loop(self):
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception:
                pass
            self._stop.wait(0.02 if self.nv is not None else 0.2)

    def start(self):
        self._thr = threading.Thread(target=self._loop, daemon=True)
        self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join()
        try:
            self._sample()
        except Exception:
            pass
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


_CPU_WS = {}


def cpu_leg(threads, budget_s, passes_cap, native=True):
    """Oracle W8·f32 matmul over one GEMV per case; returns (GB/s, seconds per pass, passes, per-case GB/s)."""
    from oracle import oracle
    ws = _CPU_WS
    if not ws:
        for (K, N) in SHAPES:
            for fmt, blk in FORMATS:
                d, s = host_weight(K, N, fmt, 1)
                ws[(K, N, fmt)] = (oracle.QuantizedWeight(d, s, K, N, 32), blk)
        for (K, N, fmt), (qw, blk) in ws.items():  # warm-up pass (llama_smollm_bench.zig:147 does one too)
            qw.matmul(np.zeros(K, np.float32), 1, threads=threads, native=native)
    x = np.random.default_rng(7).standard_normal(4096).astype(np.float32)
    per_case = {k: 0.0 for k in ws}
    passes, t0 = 0, time.perf_counter()
    while passes < passes_cap and (time.perf_counter() - t0 < budget_s or passes < 1):
        for key, (qw, blk) in ws.items():
            t = time.perf_counter()
            qw.matmul(x, 1, threads=threads, native=native)
            per_case[key] += time.perf_counter() - t
        passes += 1
    total = sum(per_case.values())
    total_bytes = sum(alg_bytes(K, N, blk) for (K, N, fmt), (qw, blk) in ws.items()) * passes
    cases = [{"K": K, "N": N, "format": fmt, "gbps": alg_bytes(K, N, ws[(K, N, fmt)][1]) * passes / per_case[(K, N, fmt)] / 1e9}
             for (K, N, fmt) in ws]
    return total_bytes / total / 1e9, total / passes, passes, cases


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def config_dict(n_gpus):
    return {"workload": "Llama-3-70B-shape Q4_0 greedy decode, batch 1, 512-token context (BASELINE.json configs[4]); synthetic "
                        "random-init GGUF blocks generated in HBM, the same model at every N",
            "model_shape": "d_model 8192, d_ff 28672, 64/8 heads, 80 layers, vocab 128256 untied, 69.5 G quantized weights = 39.1 GB of Q4_0 blocks",
            "batch": 1, "context": DECODE_CONTEXT,
            "l2": "inputs larger than L2: 39.1 GB / N of weights stream from HBM every token",
            "parallelism": "1 GPU" if n_gpus == 1 else f"tp{n_gpus}: q/k/v/gate/up column slabs, o/down row slabs + NVLink peer all-reduce, LM head vocab slab + NCCL all-gather",
            "gemv_leg": "quantized matvec microbench 4096x4096 and 4096x14336, each quant.zig block format (36 / 34 / 18 B per 32 weights), "
                        "batch 1, >= 512 MB of distinct weight copies per case (BASELINE.json configs[1]); every rank its own copies"}


def decode_cfg(n_layers=None, vocab=None):
    from zgml_b200.host import llama
    d = dict(llama.LLAMA3_70B.__dict__)
    if n_layers is not None:
        d["n_layers"] = n_layers
    if vocab is not None:
        d["vocab_size"] = vocab
    return llama.LlamaConfig(**d)


def decode_bytes_per_token(cfg, world):
    """Algorithmic HBM bytes one rank streams per decode token: its Q4_0 blocks (18 B / 32 weights) + the f32 KV rows it reads."""
    from zgml_b200.host import llama
    per_layer = sum(k * n for k, n in llama.linear_shapes(cfg).values())
    q = (per_layer * cfg.n_layers + cfg.d_model * cfg.vocab_size) // 32 * 18
    kv = cfg.n_layers * 2 * DECODE_CONTEXT * cfg.kv_dim * 4
    return (q + kv) // world


def cpu_decode_sample(threads, tokens, native=True):
    """Oracle executor on the 70B-shape model, bounded: 1- and 2-layer models at full width with the full LM head, decode from
    DECODE_CONTEXT; returns (t1, t2) seconds per token and the extrapolated 80-layer tok/s."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from llama_reference import OracleBackend
    from oracle import oracle
    from zgml_b200.host import llama
    cfg2 = decode_cfg(n_layers=2)
    w2 = llama.synthetic_model_host(cfg2, DECODE_KIND, seed=0)
    cfg1 = decode_cfg(n_layers=1)
    w1 = llama.LlamaWeights(cfg1, w2.token_embed, w2.layers[:1], w2.norm1[:1], w2.norm2[:1], w2.norm_f, w2.out_proj)
    oracle.set_exec_threads(threads, native=native)
    times = []
    for cfg, w in ((cfg1, w1), (cfg2, w2)):
        sess = llama.DeviceLlamaSession(OracleBackend(native=native), cfg, w, 1)
        sess.pos = DECODE_CONTEXT
        tok = int(np.argmax(sess.step(1)))   # warm-up (llama_smollm_bench.zig:147 does one too)
        t0 = time.perf_counter()
        for _ in range(tokens):
            tok = int(np.argmax(sess.step(tok)))
        times.append((time.perf_counter() - t0) / tokens)
        sess.close()
    oracle.set_exec_threads(1, native=native)
    t1, t2 = times
    full = t1 + 79.0 * max(t2 - t1, 0.0)
    return t1, t2, 1.0 / full


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    thr = host_threads()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from llama_reference import OracleBackend
    from oracle import oracle
    from zgml_b200.host import llama
    cfg2 = decode_cfg(n_layers=2)
    w2 = llama.synthetic_model_host(cfg2, DECODE_KIND, seed=0)
    cfg1 = decode_cfg(n_layers=1)
    w1 = llama.LlamaWeights(cfg1, w2.token_embed, w2.layers[:1], w2.norm1[:1], w2.norm2[:1], w2.norm_f, w2.out_proj)
    oracle.set_exec_threads(thr, native=True)
    s1 = llama.DeviceLlamaSession(OracleBackend(native=True), cfg1, w1, 1)
    s2 = llama.DeviceLlamaSession(OracleBackend(native=True), cfg2, w2, 1)
    s1.pos = s2.pos = DECODE_CONTEXT
    tok1 = tok2 = 1
    for _ in range(max(args.warmup, 1)):
        tok1 = int(np.argmax(s1.step(tok1)))
        tok2 = int(np.argmax(s2.step(tok2)))
    t1 = t2 = 0.0
    for _ in range(args.steps):     # a step = one token of the 2-layer sample model (+ one of the 1-layer model for the extrapolation)
        t = time.perf_counter(); tok1 = int(np.argmax(s1.step(tok1))); t1 += time.perf_counter() - t
        t = time.perf_counter(); tok2 = int(np.argmax(s2.step(tok2))); t2 += time.perf_counter() - t
    s1.close(); s2.close()
    t1 /= args.steps; t2 /= args.steps
    ms = 1e3 * (t1 + 79.0 * max(t2 - t1, 0.0))
    value = 1e3 / ms
    sample = (f"oracle executor (reference.zig / quant.zig semantics), qmatmul columns split over {thr} threads; per step one decode token of a 1-layer "
              f"and of a 2-layer Llama-3-70B-width Q4_0 model with the full LM head ({1e3 * t1:.1f} / {1e3 * t2:.1f} ms), extrapolated to 80 layers: "
              "t1 + 79 (t2 - t1)")
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "f32 (i8 weights x f32 scales x f32 activations)",
                      "data": "synthetic", "config": config_dict(args.gpus),
                      "cpu_baseline": {"value": value, "unit": UNIT, "cores": thr, "kind": "port", "sample": sample},
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


def gemv_leg(args, be, torch, dist, stream, rank, world, barrier):
    """configs[1]: returns the `gemv` object, the `roofline` object and the launch count of its timed region."""
    from zgml_b200 import DeviceOp, DeviceProgram, ProgramIO, QuantizedWeightUpload
    from zgml_b200.backend import _io_array
    rot = args.rotation_mb << 20
    cases = []
    for (K, N) in SHAPES:
        for fmt, blk in FORMATS:
            R = max(2, -(-rot // alg_bytes(K, N, blk)))
            data, scales = host_weight(K, N, fmt, seed=1 + rank)
            qws = [QuantizedWeightUpload(data, scales, K, N, 32) for _ in range(R)]  # R distinct device copies
            ops = [DeviceOp.qmatmul(1, 0, i, 1, N, K, dst_offset=i * N) for i in range(R)]
            prog = DeviceProgram(ops, [K, R * N], [], qws)
            h = be.compile_program(prog)
            if h is None:
                from zgml_b200.backend import last_error
                raise SystemExit(f"compile_program failed: {last_error()}")
            x = torch.randn(K, dtype=torch.float32).pin_memory()
            out = torch.empty(R * N, dtype=torch.float32).pin_memory()
            cases.append({"K": K, "N": N, "format": fmt, "blk": blk, "R": R, "h": h, "prog": prog, "ops": ops,
                          "x": x, "out": out, "xin": _io_array([ProgramIO(0, x.numpy())]), "oout": _io_array([ProgramIO(1, out.numpy())]),
                          "bytes": alg_bytes(K, N, blk) * R})
            be.lib.zg_cuda_execute(be.ctx, h.ptr, cases[-1]["xin"], 1, cases[-1]["oout"], 1)  # uploads x; captures the graph
    step_bytes = sum(c["bytes"] for c in cases)
    lib, ctx = be.lib, be.ctx
    steps = max(args.gemv_steps, 1)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            for c in cases:
                lib.zg_cuda_execute_device(ctx, c["h"].ptr)
        barrier()
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(cases) + 1)] for _ in range(steps)]
        launches0 = be.launch_count()
        barrier()
        for s in range(steps):
            evs[s][0].record(stream)
            for i, c in enumerate(cases):
                lib.zg_cuda_execute_device(ctx, c["h"].ptr)
                evs[s][i + 1].record(stream)
        barrier()
        launches = be.launch_count() - launches0
        total_ms = evs[0][0].elapsed_time(evs[-1][-1])
        case_ms = [sum(evs[s][i].elapsed_time(evs[s][i + 1]) for s in range(steps)) for i in range(len(cases))]
        for _ in range(max(args.warmup, 3)):   # e2e: host buffers, copies inside the timed region
            for c in cases:
                lib.zg_cuda_execute(ctx, c["h"].ptr, c["xin"], 1, c["oout"], 1)
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            for c in cases:  # VTable.execute_program: upload inputs -> run ops -> download outputs, synchronous
                lib.zg_cuda_execute(ctx, c["h"].ptr, c["xin"], 1, c["oout"], 1)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = t.tolist()
    ms_per_step = total_ms / steps
    value = world * step_bytes / (ms_per_step / 1e3) / 1e9
    e2e_value = world * step_bytes / (e2e_ms / steps / 1e3) / 1e9
    peak, peak_kind = peaks()
    case_out = []
    for c, ms in zip(cases, case_ms):
        us = ms * 1e3 / (steps * c["R"])
        gb = alg_bytes(c["K"], c["N"], c["blk"]) / (us * 1e-6) / 1e9
        case_out.append({"K": c["K"], "N": c["N"], "format": c["format"], "copies": c["R"], "us_per_gemv": round(us, 3),
                         "gbps": round(gb, 1), "frac_of_measured_hbm": round(gb / peak, 4), "frac_of_8TBps": round(gb / 8000.0, 4),
                         "share_of_step": round(ms / sum(case_ms), 4)})
    dom_i = max(range(len(cases)), key=lambda i: case_ms[i])
    dom, domc = case_out[dom_i], cases[dom_i]
    per_launch = min(8, domc["R"])   # one launch carries up to 8 same-level same-shape matvecs (csrc/backend.cu gemv_batch)
    traffic, traffic_note = None, None
    tp = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tp):
        try:
            t = json.load(open(tp)).get(f"{domc['K']}x{domc['N']}_{domc['format']}")
            if isinstance(t, dict):
                traffic = t["dram_bytes_per_launch"] if t.get("gemvs_per_launch") == per_launch else int(t["dram_bytes_per_launch"] / max(t.get("gemvs_per_launch", 1), 1) * per_launch)
                traffic_note = f"ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of {t.get('gemvs_per_launch')} matvecs, captured offline (profiles/traffic.json)"
            elif t is not None:
                traffic = int(t) * per_launch
        except Exception:
            traffic = None
    kname = "qgemv_stream_kernel" if be.program_stats(domc["h"])["streamed_matvec_launches"] else "qgemv_kernel"
    roofline = {"bound": "hbm", "kernel": f"{kname}<{domc['format']}> {domc['K']}x{domc['N']} batch 1, {per_launch} matvecs per launch "
                                          "(dominant kernel of the GEMV leg; the same kernel carries the decode step's linears)",
                "achieved": dom["gbps"], "peak": peak, "peak_kind": f"{peak_kind} copy bandwidth (MEASURED_PEAKS.json hbm_gbs)",
                "unit": "GB/s", "frac": round(dom["gbps"] / peak, 4), "frac_all_cases": round(value / world / peak, 4),
                "algorithmic_bytes_per_launch": alg_bytes(domc["K"], domc["N"], domc["blk"]) * per_launch,
                "launch_us": round(dom["us_per_gemv"] * per_launch, 3), "matvecs_per_launch": per_launch,
                "traffic": traffic, "traffic_note": traffic_note}
    gemv = {"metric": GEMV_METRIC, "value": round(value, 1), "unit": "GB/s", "scaling": "weak (every rank its own weight copies, no collective)",
            "steps": steps, "ms_per_step": round(ms_per_step, 4),
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "ms_per_step": round(e2e_ms / steps, 4),
                    "h2d_bytes_per_step": sum(4 * c["K"] for c in cases), "d2h_bytes_per_step": sum(4 * c["R"] * c["N"] for c in cases)},
            "gpu_launches": int(launches), "cases": case_out}
    for c in cases:
        be.free_program(c["h"])
    return gemv, roofline, int(launches)


def w8a8_leg(be, torch, stream, cpu=True):
    """The W8A8 decode path of `session.quantize()` models (quantizeInput + gemvRange, src/quant.zig:320-459; not on the GGUF-direct
    program path): GPU GB/s over more distinct transposed weights than L2 holds, and the CPU port with the GemvPool partitioning
    rule (src/quant.zig:135-196: <= 16 workers, one per 2^20 weight elements) on 1 and min(host threads, 16) workers.
    Bytes per gemv = N*K int8 + 4*N*K/32 scales + 4K + 4N."""
    from oracle import oracle
    from zgml_b200 import QuantizedWeight
    out = []
    r = np.random.default_rng(0)
    for (K, N) in SHAPES:
        nbytes = N * K + N * (K // 32) * 4 + 4 * K + 4 * N
        copies = max(2, -(-384_000_000 // nbytes))
        data = r.integers(-127, 128, K * N, dtype=np.int8)
        scales = r.uniform(1e-3, 1e-2, K * N // 32).astype(np.float32)
        ws = []
        for _ in range(copies):
            w = QuantizedWeight.upload(be, data, scales, K, N, 32)
            w.prepare_transposed()
            ws.append(w)
        x = torch.randn(K, device="cuda")
        y = torch.empty(N, device="cuda")
        iters = 100
        with torch.cuda.stream(stream):
            for w in ws[:3]:
                w.gemv_device(x.data_ptr(), y.data_ptr())
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(iters):
                    ws[i % copies].gemv_device(x.data_ptr(), y.data_ptr())
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / iters * 1e3
        for w in ws:
            w.free()
        peak, _ = peaks()
        row = {"K": K, "N": N, "block_size": 32, "us_per_gemv": round(us, 2), "gbps": round(nbytes / us / 1e3, 1),
               "frac_of_measured_hbm": round(nbytes / us / 1e3 / peak, 4), "launches_per_gemv": 2}
        if cpu:
            o = oracle.QuantizedWeight(data, scales, K, N, 32)
            o.prepare_transposed()
            xh = r.standard_normal(K).astype(np.float32)
            for workers in (1, min(host_threads(), 16)):
                o.gemv_pool(xh, workers, native=True)
                t0, n = time.perf_counter(), 0
                while n < 3 or time.perf_counter() - t0 < 1.0:
                    o.gemv_pool(xh, workers, native=True)
                    n += 1
                row[f"cpu_gbps_{workers}_workers"] = round(nbytes * n / (time.perf_counter() - t0) / 1e9, 2)
        out.append(row)
    return out


def decode_leg(args, be, torch, dist, stream, rank, world, barrier, sampler):
    """configs[4]: strong-scaling Llama-3-70B-shape Q4_0 decode.  Returns the pieces of the contract line."""
    from zgml_b200.host import llama
    cfg = decode_cfg(n_layers=args.decode_layers or None)
    t0 = time.perf_counter()
    w, handles = llama.synthetic_resident_shard(be, cfg, DECODE_KIND, seed=0, rank=rank, world=world)
    be.sync()
    t_load = time.perf_counter() - t0
    dev_bytes = sum(h.device_bytes for h in handles)
    t0 = time.perf_counter()
    sess = llama.DeviceLlamaSession(be, cfg, w, 1)
    t_compile = time.perf_counter() - t0
    lib, ctx = be.lib, be.ctx
    W = max(args.warmup, 3)
    with torch.cuda.stream(stream):
        # correctness evidence first: greedy tokens + a logits probe from a fixed start (same model at every N)
        sess.pos = DECODE_CONTEXT
        tok, toks, probe = 1, [], None
        for i in range(6):
            lg = sess.step(tok)
            if i == 0:
                probe = {"argmax": int(np.argmax(lg)), "max": float(lg.max()), "min": float(lg.min()),
                         "at": [float(lg[j]) for j in (0, 1, 777, 4096, 65536 % cfg.vocab_size, cfg.vocab_size - 1)]}
            tok = int(np.argmax(lg))
            toks.append(tok)
        # e2e: the session's step (host patching, uploads, execute, logits download, argmax), greedy
        for _ in range(W):
            tok = int(np.argmax(sess.step(tok)))
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            tok = int(np.argmax(sess.step(tok)))
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        # device: graph replays with the step's inputs resident
        for _ in range(W):
            lib.zg_cuda_execute_device(ctx, sess.handle.ptr)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = be.launch_count()
        sampler.start()
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            lib.zg_cuda_execute_device(ctx, sess.handle.ptr)
        e1.record(stream)
        barrier()
        clocks = sampler.stop()
        launches = be.launch_count() - launches0
        dev_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    stats = be.program_stats(sess.handle)
    n_ops = sess.n_ops
    h2d = 4 * (cfg.d_model + cfg.max_seq_len + 2 * cfg.d_head * cfg.n_layers)
    d2h = 4 * cfg.vocab_size
    sess.close()
    for h in handles:
        h.free()
    ms_per_step = dev_ms / args.steps
    peak, _ = peaks()
    bpt = decode_bytes_per_token(cfg, world)
    out = {"value": 1e3 / ms_per_step, "ms_per_step": ms_per_step, "e2e_value": 1e3 / (e2e_ms / args.steps), "e2e_ms": e2e_ms / args.steps,
           "h2d": h2d, "d2h": d2h, "launches": int(launches), "clocks": clocks,
           "detail": {"n_layers": cfg.n_layers, "weights_device_bytes_per_rank": int(dev_bytes), "load_s": round(t_load, 1), "compile_s": round(t_compile, 1),
                      "ops_per_token": n_ops, "kernels_per_token": stats["kernels"], "fused_decode_layers": stats["fused_decode_layers"],
                      "comm": be.comm_mode() if world > 1 else "none",
                      "hbm_bytes_per_token_per_rank": int(bpt), "hbm_floor_ms_per_token": round(bpt / (peak * 1e9) * 1e3, 3),
                      "frac_of_hbm_floor": round(bpt / (peak * 1e9) * 1e3 / ms_per_step, 4)},
           "check": {"greedy_tokens": toks, "logits_probe_step0": probe}}
    return out


def oracle_check(args, be, torch, dist, stream, rank, world):
    """A 2-layer Llama-3-70B-width Q4_0 model (vocab 8192), sharded like the benchmark model, against the CPU oracle executor on the
    host form of the same weights: logits 1e-3 relative, greedy tokens identical (the bar of tests/test_gpu_sharded.py)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from zgml_b200.host import llama
    cfg = decode_cfg(n_layers=2, vocab=8192)
    w, handles = llama.synthetic_resident_shard(be, cfg, DECODE_KIND, seed=17, rank=rank, world=world)
    sess = llama.DeviceLlamaSession(be, cfg, w, 1)
    sess.pos = 20
    tok, logs = 1, []
    with torch.cuda.stream(stream):
        for _ in range(3):
            lg = sess.step(tok).copy()
            tok = int(np.argmax(lg))
            logs.append(lg)
    sess.close()
    for h in handles:
        h.free()
    res = None
    if rank == 0:
        from llama_reference import OracleBackend
        from oracle import oracle
        oracle.set_exec_threads(host_threads(), native=True)   # bit-identical to one thread, just faster
        ref = llama.DeviceLlamaSession(OracleBackend(native=True), cfg, llama.synthetic_model_host(cfg, DECODE_KIND, seed=17), 1)
        ref.pos = 20
        tok, want = 1, []
        for _ in range(3):
            lg = ref.step(tok).copy()
            tok = int(np.argmax(lg))
            want.append(lg)
        ref.close()
        oracle.set_exec_threads(1, native=True)
        got, want = np.stack(logs), np.stack(want)
        err = float(np.max(np.abs(got.astype(np.float64) - want)) / np.max(np.abs(want)))
        res = {"model": "2 layers, d_model 8192, d_ff 28672, 64/8 heads, vocab 8192, Q4_0, sharded over the same N ranks",
               "logits_rel_err_vs_oracle": err, "greedy_tokens_match_oracle": bool((np.argmax(got, 1) == np.argmax(want, 1)).all()),
               "within_1e-3": bool(err < 1e-3)}
    if world > 1:
        dist.barrier()
    return res


def run_b200(args):
    import torch
    import torch.distributed as dist
    from zgml_b200 import CudaBackend

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device — the B200 backend has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = CudaBackend(local)
    stream = torch.cuda.Stream()
    be.set_stream(stream.cuda_stream)
    if world > 1:
        be.comm_init_torch()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    gemv, roofline, gemv_launches = gemv_leg(args, be, torch, dist, stream, rank, world, barrier)
    sampler = ClockSampler(local)
    dec = decode_leg(args, be, torch, dist, stream, rank, world, barrier, sampler)
    check = dec["check"]
    if not args.no_check:
        try:
            check["reduced_layers_vs_oracle"] = oracle_check(args, be, torch, dist, stream, rank, world)
        except Exception as e:   # the check never breaks the contract line; its absence is visible
            check["reduced_layers_vs_oracle"] = {"error": repr(e)}
            if world > 1:
                try:
                    dist.barrier()
                except Exception:
                    pass
    roofline["decode_step_frac_of_hbm_floor"] = dec["detail"]["frac_of_hbm_floor"]
    line = {"metric": METRIC, "value": round(dec["value"], 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (i4 weights x f16 block scales x f32 activations, integer-exact products, fp32 accumulate)",
            "data": "synthetic", "config": config_dict(world), "clocks": dec["clocks"],
            "e2e": {"value": round(dec["e2e_value"], 2), "unit": UNIT, "ms_per_step": round(dec["e2e_ms"], 4),
                    "h2d_bytes_per_step": dec["h2d"], "d2h_bytes_per_step": dec["d2h"]},
            "gpu_launches": dec["launches"], "roofline": roofline, "decode": dec["detail"], "check": check, "gemv": gemv}

    if rank == 0 and world == 1 and not args.no_extras:
        with torch.cuda.stream(stream):
            line["extras"] = run_extras(be, torch)
        try:
            line["gemv"]["w8a8"] = w8a8_leg(be, torch, stream, cpu=not args.no_cpu)
        except Exception as e:
            line["gemv"]["w8a8_error"] = repr(e)
    if rank == 0 and world == 1 and not args.no_cpu:
        t1, t2, tok_s = cpu_decode_sample(1, args.cpu_tokens)
        line["cpu_baseline"] = {"value": round(tok_s, 4), "unit": UNIT, "cores": 1, "kind": "port",
                                "sample": f"oracle executor, 1 thread like src/inference_utils.zig:192: {args.cpu_tokens} decode tokens each of a 1-layer and a 2-layer "
                                          f"Llama-3-70B-width Q4_0 model with the full LM head ({1e3 * t1:.0f} / {1e3 * t2:.0f} ms per token), extrapolated to 80 layers",
                                "host_threads_available": host_threads()}
        gb, sec, passes, ccases = cpu_leg(1, args.cpu_seconds, 200)
        line["gemv"]["cpu_baseline"] = {"value": round(gb, 3), "unit": "GB/s", "cores": 1, "kind": "port",
                                        "sample": f"{passes} passes of one batch-1 matvec per case (6 GEMVs/pass, {sec * 1e3:.1f} ms/pass); "
                                                  "oracle port of QuantizedWeight.matmul, single thread",
                                        "cases": [{**c, "gbps": round(c["gbps"], 3)} for c in ccases]}
    be.close()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


def run_extras(be, torch):
    """Bounded side measurements of the other BASELINE.json configs (never part of `value`): the tcgen05 prefill
    GEMM at Llama-3-8B shapes (config 4) and greedy decode of a SmolLM-135M-shape Q8_0 program (config 1)."""
    out = {}
    try:
        from zgml_b200 import QuantizedWeight
        r = np.random.default_rng(3)
        M, gem = 2048, []
        for (K, N) in [(4096, 4096), (4096, 14336)]:
            data = r.integers(-127, 128, K * N, dtype=np.int8)
            scales = r.uniform(1e-3, 1e-2, K * N // 32).astype(np.float16).astype(np.float32)
            ws = [QuantizedWeight.upload(be, data, scales, K, N, 32) for _ in range(2)]
            x = torch.randn(M, K, device="cuda")
            y = torch.empty(M, N, device="cuda")
            for w in ws:
                w.matmul_device(x.data_ptr(), y.data_ptr(), M)
            be.sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st = torch.cuda.current_stream()
            e0.record(st)
            for i in range(10):
                ws[i % 2].matmul_device(x.data_ptr(), y.data_ptr(), M)
            e1.record(st)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            gem.append({"M": M, "K": K, "N": N, "format": "q8_0", "ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)})
            for w in ws:
                w.free()
        issued = round(3 * max(g["tflops"] for g in gem), 1)
        bf16_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops", 0) or 0) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 0.0
        out["prefill_qgemm_tcgen05"] = {"mode": "3xBF16 (hi/lo split of both operands, fp32 accumulate in TMEM)", "cases": gem,
                                        "bf16_mma_tflops_issued": issued,
                                        "frac_of_measured_bf16_peak": round(issued / bf16_peak, 3) if bf16_peak else None}
    except Exception as e:  # extras never break the contract line
        out["prefill_error"] = repr(e)
    try:
        from zgml_b200.host import llama
        cfg = llama.SMOLLM_135M
        sess = llama.DeviceLlamaSession(be, cfg, llama.synthetic_weights(cfg, "q8_0", seed=0), 1)
        tok = int(np.argmax(sess.step(1)))
        t0 = time.perf_counter()
        n = 64
        for _ in range(n):
            tok = int(np.argmax(sess.step(tok)))
        dt = time.perf_counter() - t0
        out["decode_smollm_135m_q8_0"] = {"tok_s": round(n / dt, 1), "ms_per_token": round(1e3 * dt / n, 3), "ops_per_token": sess.n_ops,
                                          "path": "DeviceProgram through execute_program (host copies inside), greedy"}
        sess.close()
    except Exception as e:
        out["decode_error"] = repr(e)
    try:   # config 3: SmolLM-1.7B-shape Q4_0 decode, batch 1, 512-token context
        from zgml_b200.host import llama
        cfg = llama.SMOLLM_1_7B
        w, handles = llama.synthetic_resident_shard(be, cfg, "q4_0", seed=0)
        sess = llama.DeviceLlamaSession(be, cfg, w, 1)
        sess.pos = 512
        tok = int(np.argmax(sess.step(1)))
        n = 64
        t0 = time.perf_counter()
        for _ in range(n):
            tok = int(np.argmax(sess.step(tok)))
        dt = time.perf_counter() - t0
        be.sync()
        t0 = time.perf_counter()
        for _ in range(n):
            be.lib.zg_cuda_execute_device(be.ctx, sess.handle.ptr)
        be.sync()
        dd = time.perf_counter() - t0
        qb = sum(k * m for k, m in llama.linear_shapes(cfg).values()) * cfg.n_layers // 32 * 18 + cfg.vocab_size * cfg.d_model * 4 + cfg.n_layers * 2 * 512 * cfg.kv_dim * 4
        peak, _ = peaks()
        out["decode_smollm_1p7b_q4_0_ctx512"] = {"tok_s": round(n / dt, 1), "device_tok_s": round(n / dd, 1), "ms_per_token_device": round(1e3 * dd / n, 3),
                                                 "hbm_bytes_per_token": int(qb), "frac_of_hbm_floor": round(qb / (peak * 1e9) / (dd / n), 4),
                                                 "kernels_per_token": be.program_stats(sess.handle)["kernels"]}
        # the tied f32 LM head as an argmax-safe f16 copy (zg_cuda_program_promote_dense), same greedy tokens
        toks_f32 = []
        sess.pos = 512
        t = 1
        for _ in range(8):
            t = int(np.argmax(sess.step(t))); toks_f32.append(t)
        be.promote_dense_weights(sess.handle, "f16")
        sess.pos = 512
        t, toks_f16 = 1, []
        for _ in range(8):
            t = int(np.argmax(sess.step(t))); toks_f16.append(t)
        be.sync()
        t0 = time.perf_counter()
        for _ in range(n):
            be.lib.zg_cuda_execute_device(be.ctx, sess.handle.ptr)
        be.sync()
        d16 = time.perf_counter() - t0
        out["decode_smollm_1p7b_q4_0_ctx512"]["f16_lm_head"] = {
            "device_tok_s": round(n / d16, 1), "ms_per_token_device": round(1e3 * d16 / n, 3),
            "head_bytes_saved_per_token": be.program_stats(sess.handle)["dense_bytes_saved_per_execution"],
            "greedy_tokens_equal_f32_head": toks_f16 == toks_f32}
        sess.close()
        for h in handles:
            h.free()
    except Exception as e:
        out["decode_1p7b_error"] = repr(e)
    try:   # config 4: Llama-3-8B-shape Q8_0 prefill of 2048 tokens as ONE program (every linear on the tcgen05 path)
        from zgml_b200.host import llama
        cfg = llama.LLAMA3_8B
        T = 2048
        w, handles = llama.synthetic_resident_shard(be, cfg, "q8_0", seed=0)
        sess = llama.DeviceLlamaSession(be, cfg, w, T)
        toks = [(i + 1) % cfg.vocab_size for i in range(T)]
        sess.execute_at(toks, 0)   # warm-up: captures the graph
        t0 = time.perf_counter()
        sess.execute_at(toks, 0)
        dt = time.perf_counter() - t0
        be.sync()
        t0 = time.perf_counter()
        for _ in range(2):
            be.lib.zg_cuda_execute_device(be.ctx, sess.handle.ptr)
        be.sync()
        dd = (time.perf_counter() - t0) / 2
        lin_flops = 2.0 * T * (sum(k * m for k, m in llama.linear_shapes(cfg).values()) * cfg.n_layers + cfg.d_model * cfg.vocab_size)
        be.set_profiling(True)
        sess.execute_at(toks, 0)
        prof = be.get_runtime_profile(sess.handle)
        names = ["elementwise", "matmul", "qmatmul", "softmax", "layernorm", "rmsnorm", "reduce", "repeat", "slice_assign", "rope", "attention", "fused_elementwise"]
        by_tag = {nm: round(prof.time_ns[i] / 1e6 / max(prof.call_count, 1), 2) for i, nm in enumerate(names) if prof.time_ns[i]}
        be.set_profiling(False)
        bf16_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops", 0) or 0) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 0.0
        out["prefill_llama3_8b_q8_0_2048"] = {"tok_s": round(T / dt, 1), "device_tok_s": round(T / dd, 1), "ms_device": round(1e3 * dd, 2),
                                              "linear_tflops_effective": round(lin_flops / dd / 1e12, 1),
                                              "frac_of_measured_bf16_peak_effective": round(lin_flops / dd / 1e12 / bf16_peak, 3) if bf16_peak else None,
                                              "ms_by_op_tag_one_launch_per_op": by_tag}
        sess.close()
        for h in handles:
            h.free()
    except Exception as e:
        out["prefill_8b_error"] = repr(e)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50, help="timed decode tokens")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rotation-mb", type=int, default=ROTATION_BYTES >> 20)
    ap.add_argument("--cpu-seconds", type=float, default=5.0, help="budget of the GEMV leg's single-thread CPU sample")
    ap.add_argument("--cpu-tokens", type=int, default=3, help="decode tokens per sample model in cpu_baseline")
    ap.add_argument("--gemv-steps", type=int, default=20, help="passes over the GEMV microbench set (its own leg, not `steps`)")
    ap.add_argument("--decode-layers", type=int, default=0, help="override the 80 layers of the decode model (experiments only; the default run uses 80)")
    ap.add_argument("--no-check", action="store_true", help="skip the 2-layer oracle comparison")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--arch", default="", choices=["", "lududra", "vemepel", "pepevik", "setirax"],
                    help="side bench instead of the default workload: prefill / decode throughput of that design next to the framework's closest "
                         "model at equal layer sizes (lududra: a LLaMA; vemepel, pepevik: Lududra; setirax: Pepevik)")
    ap.add_argument("--arms", default="", help="--arch pepevik, setirax: comma-separated arms to run (default: both)")
    ap.add_argument("--sizes", default="", help="--arch: comma-separated size names (default: all)")
    ap.add_argument("--prefill-tokens", type=int, default=1024, help="--arch: tokens of the timed prefill chunk")
    ap.add_argument("--context", type=int, default=1024, help="--arch: tokens in the sequence before the timed decode steps")
    args = ap.parse_args()
    if args.arch:
        sys.path.insert(0, os.path.join(ROOT, "scripts"))
        side = __import__("bench_" + args.arch)
        if args.steps == 50:
            args.steps = 10
        return side.run(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
