#!/usr/bin/env python
"""Decode-throughput benchmark: Q8_0 Llama-3-8B-shape model, batch 1, greedy.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (seeded synthetic weights of the named shape; there are no checkpoints here): 512-token prompt, then
K timed "steps" of TOKENS_PER_STEP greedy tokens each (default 4 x 64 = the 256 decoded tokens of the named
configuration).  `value` is decode tokens/s with everything resident in HBM, timed with CUDA events on the
runtime's stream; `e2e` is the same loop driven token by token through the public API with the token id going
host -> device and the sampled token coming device -> host every token.  Weights (8 GB) are far larger than L2
(126 MB), so every step streams them from HBM.

`--impl reference` times the CPU restatement of the reference's interpreter semantics (oracle/, the reference
itself is Rust and cannot be built here) on the host cores, on a bounded sample of the same workload.
Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS_PER_STEP = 64
PROMPT_LEN = 512
SEED = 20240607
METRIC = "q8_llama3_8b_bs1_decode_tokens_per_s"
UNIT = "tokens/s"
WORKLOAD = "llama3_8b_q8"


def set_workload(name: str, prompt_given: bool):
    """Switch the benchmarked configuration (its own metric name, so lines of different workloads are never compared)."""
    global WORKLOAD, METRIC, PROMPT_LEN
    WORKLOAD = name
    if name == "qwen3_4b_q8":
        METRIC = "q8_qwen3_4b_bs1_decode_tokens_per_s"
        if not prompt_given:
            PROMPT_LEN = 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.05)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ---------------------------------------------------------------------------------------------- CPU arm

def bench_config(world: int, warmup: int, fused: bool):
    """The `config` object of the JSON line — the same for both arms (the CPU arm runs the GPU arm's configuration)."""
    return {"workload": WORKLOAD, "batch": 1, "prompt_len": PROMPT_LEN, "tokens_per_step": TOKENS_PER_STEP,
            "context_at_start": PROMPT_LEN + warmup * TOKENS_PER_STEP,
            "l2": "weights 8.0 GB >> 126 MB L2; every token re-streams them" if WORKLOAD == "llama3_8b_q8" else "weights >> 126 MB L2; every token re-streams them",
            "parallelism": "single GPU" if world == 1 else f"tp{world}: heads/FFN/vocab sharded, " + ("partial sums exchanged through peer memory inside the projection kernels" if fused else "NCCL all-reduce per projection"),
            "seed": SEED}


def cpu_port_tokens_per_s(pkg, steps: int, warmup: int, context: int):
    """Times the oracle (a C++ restatement of the reference's CPU interpreter semantics, all host threads) on a bounded
    sample of the workload: the WHOLE model (every layer, the whole vocabulary), `warmup` + `steps` single-token forward
    passes at positions context, context + 1, ... — the cache rows before `context` hold seeded stand-in values instead
    of a computed prompt (computing it would take the CPU several minutes; the arithmetic per token is the same)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    from oracle import OracleModel, load
    full = pkg.CONFIGS[WORKLOAD]
    steps, warmup = max(1, steps), max(0, warmup)
    d = full.copy(max_seq=context + steps + warmup + 8)
    lib = load()
    threads = lib.orc_threads()
    t_build = time.perf_counter()
    m = OracleModel(d)
    m.synth(SEED)
    m.kv_fill(SEED, context)
    t_build = time.perf_counter() - t_build
    tok, p = 1, context
    for _ in range(warmup):
        tok = m.argmax(m.forward([tok], p)[0]); p += 1
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = m.argmax(m.forward([tok], p)[0]); p += 1
    dt = time.perf_counter() - t0
    sample = (f"whole model ({full.n_layers} layers, vocabulary {full.vocab}), {steps} single-token passes at context {context}.."
              f"{context + steps + warmup - 1} after {warmup} warm-up passes; cache rows below {context} seeded, not computed; "
              f"model set-up {t_build:.0f} s outside the timed region")
    return steps / dt, threads, sample, np.__version__


def run_reference_arm(args, pkg):
    """One "step" of this arm is one decoded token (a bounded sample of the GPU arm's 64-token step)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    context = PROMPT_LEN + args.warmup * TOKENS_PER_STEP
    v, threads, sample, _ = cpu_port_tokens_per_s(pkg, args.steps, args.warmup, min(context, 2048))
    cfg = bench_config(max(1, args.gpus), args.warmup, os.environ.get("LUM_TP_FUSED", "1") != "0")
    cfg["note"] = "CPU restatement of the reference's NativeRuntime semantics; the reference (Rust) cannot be built here"
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------- GPU arm

def kernel_roofline(pkg, torch, peaks, peak_kind):
    """The dominant kernel (q8_gemv_stream) timed alone on the gate+up-sized shape: N = 28672 rows, K = 4096."""
    lib = pkg.load_library()
    n, k, nbuf = 28672, 4096, 8                       # 8 x 125 MB of distinct weights: far larger than L2
    w = [torch.empty(lib.lum_q8_0_packed_bytes(n, k), dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
    for i in range(nbuf):
        assert lib.lum_op_synth_q8_0_packed(SEED, 900 + i, n, k, w[i].data_ptr(), None) == 0
    x = torch.randn(k, dtype=torch.float32, device="cuda")
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    for i in range(4):
        assert lib.lum_op_gemv_q8_0_packed(w[i % nbuf].data_ptr(), n, k, x.data_ptr(), y.data_ptr(), 0, st) == 0
    launches = 40
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(launches):
        lib.lum_op_gemv_q8_0_packed(w[i % nbuf].data_ptr(), n, k, x.data_ptr(), y.data_ptr(), 0, st)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / launches
    bytes_per_launch = n * k * 34 // 32 + k * 4 + n * 4
    achieved = bytes_per_launch / (ms * 1e-3) / 1e9
    del w
    torch.cuda.empty_cache()
    return {"bound": "hbm", "kernel": "q8_gemv_stream", "shape": f"N={n} K={k} (gate+up sized), alone, back to back",
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "peak_kind": f"of {peak_kind} (burst copy)", "us_per_launch": ms * 1000.0, "bytes_per_launch": bytes_per_launch,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this shape under ncu (124.87 MB read + 9.17 MB
            # written): a figure from a profile of this kernel, not measured by this run
            "traffic": 134_049_024, "traffic_from": "ncu capture of this kernel on this shape (profiles/), not this run"}, launches + 4


def kernel_rows_sweep(pkg, torch):
    """The dominant kernel alone at K = 4096 over a range of row counts, launched back to back on distinct weights (each
    set of buffers larger than L2).  Time per launch is close to linear in the rows: the slope is the steady-state cost of
    one ring fill per CTA (8 tiles = 34816 bytes per SM), the intercept what every launch pays besides streaming."""
    lib = pkg.load_library()
    k, sms = 4096, torch.cuda.get_device_properties(0).multi_processor_count
    x = torch.randn(k, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    rows = []
    for n in (4096, 8192, 14336, 28672, 57344, 114688):
        b = lib.lum_q8_0_packed_bytes(n, k)
        nbuf = max(4, int(600e6 // b) + 1)
        w = [torch.empty(b, dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
        for i in range(nbuf):
            assert lib.lum_op_synth_q8_0_packed(SEED, 700 + i, n, k, w[i].data_ptr(), None) == 0
        y = torch.empty(n, dtype=torch.float32, device="cuda")
        reps, best = 3 * nbuf, None
        for _ in range(3):
            for i in range(nbuf):
                assert lib.lum_op_gemv_q8_0_packed(w[i].data_ptr(), n, k, x.data_ptr(), y.data_ptr(), 0, st) == 0
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(reps):
                lib.lum_op_gemv_q8_0_packed(w[i % nbuf].data_ptr(), n, k, x.data_ptr(), y.data_ptr(), 0, st)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            best = us if best is None else min(best, us)
        rows.append({"rows": n, "us_per_launch": best, "fills_per_cta": n / 8 / sms, "gb_per_s": b / best / 1e3})
        del w, y
        torch.cuda.empty_cache()
    a, b = rows[-2], rows[-1]
    slope = (b["us_per_launch"] - a["us_per_launch"]) / (b["fills_per_cta"] - a["fills_per_cta"])
    return {"kernel": "q8_gemv_stream", "k": k, "rows": rows, "us_per_fill_steady": slope,
            "steady_gb_per_s": sms * 34816 / slope / 1e3, "fixed_us_per_launch": b["us_per_launch"] - slope * b["fills_per_cta"]}


def gemm_shapes(pkg, torch, shapes=None):
    """The tensor-core GEMM alone (row quantiser + q8_gemm_tc [+ the K-split sum]) through lum_op_gemm_q8_0_packed on the
    Llama-3-8B layer's shapes, 512 rows (one pass of a prompt) and 32 rows (batched decode): µs per call and useful TFLOP/s
    (2 N K M: the redundant products of the operand split are not counted)."""
    lib = pkg.load_library()
    out = []
    for n, k, m in (shapes or [(28672, 4096, 512), (6144, 4096, 512), (4096, 4096, 512), (4096, 14336, 512),
                               (28672, 4096, 32), (6144, 4096, 32), (4096, 14336, 32), (128256, 4096, 32)]):
        packed = torch.empty(lib.lum_q8_0_packed_bytes(n, k), dtype=torch.uint8, device="cuda")
        assert lib.lum_op_synth_q8_0_packed(SEED, 900, n, k, packed.data_ptr(), None) == 0
        x = torch.randn(m, k, device="cuda")
        y = torch.empty(m, n, device="cuda")
        ws_bytes = lib.lum_op_gemm_q8_0_workspace(n, k, m)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        best = None
        for _ in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); e0.record()
            assert lib.lum_op_gemm_q8_0_packed(packed.data_ptr(), n, k, x.data_ptr(), m, y.data_ptr(), ws.data_ptr(), ws_bytes, None) == 0
            e1.record(); torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3
            best = us if best is None else min(best, us)
        assert lib.lum_op_status(None) == 0
        out.append({"n": n, "k": k, "m": m, "us": best, "tflops": 2.0 * n * k * m / best / 1e6, "weight_gb_per_s": n * k * 34 / 32 / best / 1e3})
        del packed, x, y, ws
        torch.cuda.empty_cache()
    return {"kernel": "rows_quantize + q8_gemm_tc", "shapes": out}


def sampler_times(pkg, torch):
    """The temperature / top-k / top-p sampler alone (lum_op_sample_topk) on rows of random logits of the two vocabularies, and what
    it costs inside the decode loop: the 2-layer cut of the Llama-3-8B shape with the full vocabulary, greedy against sampled."""
    import ctypes as C
    lib = pkg.load_library()
    out = {"kernel": "sample_rows", "alone": []}
    s = pkg.Sampling(temperature=0.8, top_p=0.95, top_k=50, reserved=0, seed=1)
    for rows, vocab in ((1, 128256), (32, 128256), (1, 201088)):
        logits = torch.randn(rows, vocab, device="cuda") * 3.0
        pos = torch.zeros(rows, dtype=torch.int32, device="cuda")
        tok = torch.zeros(rows, dtype=torch.int32, device="cuda")
        best = None
        for _ in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); e0.record()
            assert lib.lum_op_sample_topk(logits.data_ptr(), rows, vocab, C.byref(s), 0, pos.data_ptr(), tok.data_ptr(), None) == 0
            e1.record(); torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3
            best = us if best is None else min(best, us)
        out["alone"].append({"rows": rows, "vocab": vocab, "us": best, "row_bytes": vocab * 4})
    desc = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(vocab=128256, max_seq=1024, max_new_tokens=512)
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        rt.load_model(desc); rt.synth(SEED)
        ext = torch.cuda.ExternalStream(rt.stream())
        res = {}
        for name, temp in (("greedy", 0.0), ("sampled", 0.8)):
            rt.set_sampling(temp, 50, 0.95, 1)
            rt.generate([1, 2, 3, 4, 5, 6, 7, 8], 64)            # warm-up, captures the graph
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(ext)
            rt.decode_greedy(256)
            e1.record(ext)
            rt.synchronize()
            res[name] = e0.elapsed_time(e1) * 1e3 / 256
        out["decode_step_us_2layer_full_vocab"] = res
        out["sampler_cost_per_token_us"] = res["sampled"] - res["greedy"]
    finally:
        rt.close()
    return out


def prompt_two_layers(pkg, torch, n=4096):
    """A 4096-token prompt through a 2-layer cut of the Llama-3-8B shape (vocabulary 4096): the same kernels and shapes as the
    full model's prompt pass, a few hundred MB on the device — the case the profiler captures of the prompt kernels use."""
    desc = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_seq=n + 64)
    rt = pkg.B200Runtime.initialize(device=0)
    rt.load_model(desc); rt.synth(SEED)
    ids = _prompt_tokens(desc.vocab, n)
    ms = []
    for _ in range(3):
        rt.kv_reset(); rt.decode_reset(); rt.synchronize()
        t0 = time.perf_counter()
        rt.set_data(ids); rt.execute({"s": n, "p": 0}); rt.synchronize()
        ms.append((time.perf_counter() - t0) * 1e3)
    rt.close()
    return {"config": "llama3_8b_q8_2layer", "prompt_len": n, "ms_two_layers_and_head": min(ms), "ms_per_32_layers": min(ms) / 2 * 32}


def launch_chain_floor(pkg, torch):
    """The decode step of the benchmark's model with every projection shrunk to almost nothing (hidden 512, 4/1 heads of 128,
    ffn 512, vocabulary 1024; same 32 layers, same launches, same context): what is left is the chain of dependent launches —
    hand-over between kernels, set-up, activation prologue, first accumulator read-back, epilogue — with no weight streaming
    to speak of.  Reported beside the full model on the same box."""
    base = pkg.CONFIGS[WORKLOAD]
    out = {}
    for name, d in (("full", base), ("tiny_projections", base.copy(hidden=512, n_q_heads=4, n_kv_heads=1, ffn=512, vocab=1024))):
        rt = pkg.B200Runtime.initialize(device=0)
        try:
            rt.load_model(d)
            rt.synth(SEED)
            rt.set_data([i % 1000 + 1 for i in range(512)])
            rt.execute({"s": 512, "p": 0})
            rt.decode_greedy(64)
            rt.synchronize()
            st = torch.cuda.ExternalStream(rt.stream())
            best = None
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                rt.decode_greedy(64)
                e1.record(st)
                rt.synchronize()
                us = e0.elapsed_time(e1) / 64 * 1e3
                best = us if best is None else min(best, us)
            n = rt.launches_per_step()
            out[name] = {"us_per_token": best, "launches_per_token": n, "us_per_launch": best / n, "us_per_layer": best / d.n_layers}
        finally:
            rt.close()
    return out


def run_ours(args, pkg):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this runtime has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peak_kind = measured_peaks()

    desc = pkg.CONFIGS[WORKLOAD]
    rt = pkg.B200Runtime.initialize(device=local)
    if world > 1:
        # tensor parallel: heads / FFN columns / vocabulary sharded over the ranks, one all-reduce per projection
        from oneiron_luminal_b200 import tp as T
        T.validate(desc, world)
        uid = T.exchange_unique_id(dist, rank, pkg.B200Runtime.tp_unique_id, device=torch.device("cuda", local))
        rt.tp_init(uid, world, rank)
        desc = desc.copy(tp_size=world, tp_rank=rank)
    rt.load_model(desc)
    fused = world > 1 and os.environ.get("LUM_TP_FUSED", "1") != "0"
    if fused:
        # partial sums of the K-sharded projections travel through peer memory inside the projection kernels
        rt.tp_peer_import(T.exchange_peer_handles(dist, world, rt.tp_peer_export(), device=torch.device("cuda", local)))
    rt.synth(SEED)
    # prompt: 512 seeded ids (same generator as the oracle's: tensor id 2^20, uniform over the vocabulary)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    prompt = _prompt_tokens(desc.vocab, PROMPT_LEN)
    rt.kv_reset()
    rt.decode_reset()
    rt.set_data(prompt)
    rt.execute({"s": len(prompt), "p": 0})
    rt.synchronize()
    # for the output check below: the logits row that follows the prompt (this rank's vocabulary shard) and its greedy token
    prompt_logits = rt.get_f32()
    first_token = rt.get_token()

    ext = torch.cuda.ExternalStream(rt.stream(), device=torch.device("cuda", local))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        rt.decode_greedy(TOKENS_PER_STEP)
    rt.synchronize()
    p_start = PROMPT_LEN + args.warmup * TOKENS_PER_STEP

    sampler = ClockSampler(physical_gpu_index(local))
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    for _ in range(args.steps):
        rt.decode_greedy(TOKENS_PER_STEP)
    e1.record(ext)
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    n_tok = args.steps * TOKENS_PER_STEP
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tok_s_rank = n_tok / (ms * 1e-3)
    value = tok_s_rank                    # tensor parallel: all ranks work on the one sequence
    p_mean = p_start + n_tok / 2.0
    bytes_tok = pkg.decode_bytes_per_token(pkg.CONFIGS[WORKLOAD], p_mean)

    # Output check: the first 32 greedy tokens and the post-prompt logits against the committed oracle fixture of this
    # workload (tests/golden/<workload>_full.npz: whole model, this seed, this prompt), on every rank.
    parity = check_parity(rt, prompt, prompt_logits, first_token, n_decoded=(args.warmup + args.steps) * TOKENS_PER_STEP,
                          world=world, rank=rank, dist=dist if world > 1 else None, torch=torch)

    # end-to-end through the public API, one token at a time, host <-> device every token
    tok = rt.get_token()
    p = p_start + n_tok
    e2e_tokens = max(1, min(n_tok, desc.max_seq - 1 - p))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_tokens):
        rt.set_data([tok])
        rt.execute({"s": 1, "p": p})
        tok = rt.get_token()
        p += 1
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = e2e_tokens / e2e_s

    launches_step = rt.launches_per_step()
    line = None
    if rank == 0:
        roof, extra_launches = kernel_roofline(pkg, torch, peaks, peak_kind)
        step_ach = bytes_tok * tok_s_rank / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            # one sequence, one fixed-size model whatever N: the same experiment at every N
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 accumulate over Q8_0 (int8 x f16-scale) weights", "data": "synthetic",
            "config": bench_config(world, args.warmup, fused),
            "parity": parity,
            "roofline": roof,
            "step_roofline": {"bound": "hbm", "what": "whole decode step, all kernels; bytes are the whole model's, peak is per GPU x n_gpus",
                              "bytes_per_token": bytes_tok, "achieved": step_ach, "peak": peaks["hbm_gbs"] * world, "unit": "GB/s",
                              "frac": step_ach / (peaks["hbm_gbs"] * world), "frac_of_8tbs_nominal": step_ach / (8000.0 * world),
                              "peak_kind": f"of {peak_kind}"},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": 8 * TOKENS_PER_STEP, "d2h_bytes_per_step": 4 * TOKENS_PER_STEP,
                    "tokens": e2e_tokens,
                    "note": "per token: token id + position host->device, sampled token device->host, synchronous"},
            "gpu_launches": launches_step * n_tok,
            "clocks": clocks,
        }
        # the reference bench crate's derived figures (crates/luminal_bench/src/metrics.rs:13-60) for this step
        from oneiron_luminal_b200.metrics import BenchMetricsMap, HardwareSpec, decode_step_metrics
        mm = BenchMetricsMap(HardwareSpec("NVIDIA B200", 180.0, peaks["hbm_gbs"] * world, peaks["bf16_tflops"] * world))
        name = f"decode/{WORKLOAD}/p{p_start}"
        mm.add(name, decode_step_metrics(desc, p_start + n_tok // 2))
        line["mbu_mfu"] = dict(mm.summary(name, 1e6 / value), benchmark=name, peaks=f"of {peak_kind}")
        if args.report:
            with open(args.report, "w") as fh:
                fh.write(mm.to_json())
        if world == 1 and not args.no_cpu:
            try:
                v, threads, sample, _ = cpu_port_tokens_per_s(pkg, 8, 1, min(p_start, 2048))
                line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
            except Exception as exc:  # the GPU number stands on its own
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
    rt.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line))


def check_parity(rt, prompt, prompt_logits, first_token, n_decoded, world, rank, dist, torch):
    """Compares what this run produced with the oracle's committed outputs for the same workload, seed and prompt."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", f"{WORKLOAD}_full.npz")
    if not os.path.exists(path):
        return {"checked": False, "reason": f"no fixture {os.path.relpath(path, ROOT)}"}
    fx = np.load(path)
    if int(fx["seed"]) != SEED or list(fx["prompt"]) != list(prompt):
        return {"checked": False, "reason": "fixture was made for another seed or prompt (this run used non-default sizes)"}
    want = [int(t) for t in fx["tokens"]]
    n = min(len(want), 1 + n_decoded)
    got = [int(first_token)] + ([int(t) for t in rt.get_decoded(n - 1)] if n > 1 else [])
    ref = fx["prompt_logits"].astype(np.float32)
    shard = ref.size // world
    mine = ref[rank * shard:(rank + 1) * shard]
    err = float(np.max(np.abs(prompt_logits - mine)) / np.max(np.abs(ref)))
    equal = got == want[:n]
    if world > 1:
        t = torch.tensor([err, 0.0 if equal else 1.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err, equal = float(t[0].item()), float(t[1].item()) == 0.0
    first_bad = next((i for i in range(n) if got[i] != want[i]), None)
    return {"checked": True, "tokens_equal": bool(equal), "steps": n, "logits_rel_err": err, "logits_tolerance": 1e-2,
            "first_mismatch": first_bad, "min_margin_of_fixture": float(np.min(fx["margins"][:n])),
            "fixture": os.path.relpath(path, ROOT)}


def run_tensor_core_regime(args, pkg, which: str):
    """The Llama-3-8B-shape model in the regime where the work is a matrix-matrix product (one GPU):
    `llama3_8b_q8_bs32`: batched decode, 32 sequences with 2048 cached tokens each, one row per sequence and step; a "step"
    is `--tokens-per-step` tokens of every sequence.  HBM-bound: weights once + every sequence's cache per token step.
    `llama3_8b_q8_prefill4096`: one 4096-token prompt; a "step" is the whole prompt.  Tensor-pipe-bound."""
    import torch
    torch.cuda.set_device(0)
    peaks, peak_kind = measured_peaks()
    base = pkg.CONFIGS["llama3_8b_q8"]
    rt = pkg.B200Runtime.initialize(device=0)
    sampler = ClockSampler(physical_gpu_index(0))
    if which == "llama3_8b_q8_bs32":
        B, ctx, tps = 32, 2048, max(1, min(TOKENS_PER_STEP, 16))
        total = (args.warmup + 2 * args.steps) * tps          # warm-up, the timed steps, then the same number again end to end
        rt.load_model(base.copy(max_batch=B, max_seq=ctx + total + 8, max_new_tokens=total + 8))
        rt.synth(SEED)
        firsts = []
        for sq in range(B):                      # every sequence's context: a seeded random-id prompt, run as rows
            rt.seq_select(sq)
            ids = _prompt_tokens(base.vocab, ctx + sq)[sq:]
            rt.set_data(ids); rt.execute({"s": ctx, "p": 0})
            firsts.append(rt.get_token())
        rt.batch_begin(firsts, [ctx] * B)
        for _ in range(args.warmup):
            rt.batch_decode(tps)
        rt.synchronize()
        ext = torch.cuda.ExternalStream(rt.stream())
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ext)
        for _ in range(args.steps):
            rt.batch_decode(tps)
        e1.record(ext)
        rt.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        n_tok = args.steps * tps * B
        value = n_tok / (ms * 1e-3)
        p_mean = ctx + (args.warmup + args.steps / 2.0) * tps
        bytes_step = pkg.decode_bytes_per_token(base, 0) - 131072 + 131072.0 * (p_mean + 1) * B     # weights once, every sequence's cache
        ach = bytes_step * (args.steps * tps) / (ms * 1e-3) / 1e9
        n_run = (args.warmup + args.steps) * tps
        launches = int(rt.stats().kernel_launches)
        batch_log = rt.batch_get_decoded(n_run)
        batch_logits = {sq: rt.batch_get_logits(sq) for sq in (0, B - 1)}
        # end to end: the same loop with the sampled tokens of every step read back by the host
        t0 = time.perf_counter()
        for _ in range(args.steps * tps):
            rt.batch_decode(1)
            rt.batch_get_decoded(1)
        e2e = args.steps * tps * B / (time.perf_counter() - t0)
        rt.close()
        parity = _batch_parity(pkg, base, ctx, n_run, firsts, batch_log, batch_logits, B)
        line = {"metric": "q8_llama3_8b_bs32_decode_tokens_per_s", "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16 x f16 -> f32 on tcgen05 (weights as two exact binary16 terms, activations as two), f32 sums", "data": "synthetic",
                "config": {"workload": which, "batch": B, "context": ctx, "tokens_per_step": tps, "seed": SEED,
                           "l2": "weights 8.0 GB + caches 8.6 GB >> 126 MB L2"},
                "roofline": {"bound": "hbm", "kernel": "whole batched step (q8_gemm_tc + attn_rows dominate)", "achieved": ach, "peak": peaks["hbm_gbs"],
                             "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind}", "bytes_per_step": bytes_step, "traffic": None},
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4 * B * tps,
                        "note": "every step's sampled tokens device->host; the fed-back tokens stay on the device"},
                "parity": parity, "gpu_launches": launches, "clocks": clocks}
    else:
        n = 4096
        rt.load_model(base.copy(max_seq=n + 8))
        rt.synth(SEED)
        ids = _prompt_tokens(base.vocab, n)
        ext = torch.cuda.ExternalStream(rt.stream())
        for _ in range(max(1, args.warmup)):
            rt.set_data(ids); rt.execute({"s": n, "p": 0})
        rt.synchronize()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ext)
        for _ in range(args.steps):
            rt.set_data(ids); rt.execute({"s": n, "p": 0})
        e1.record(ext)
        rt.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        value = args.steps * n / (ms * 1e-3)
        # linear layers 2 * weights * rows (the vocabulary projection runs for the last row only) + causal attention
        d = base
        w_layers = d.n_layers * (2 * d.hidden * d.n_q_heads * d.head_dim + 2 * d.hidden * d.n_kv_heads * d.head_dim + 3 * d.hidden * d.ffn)
        flops = 2.0 * w_layers * n + 2.0 * d.vocab * d.hidden + d.n_layers * 4.0 * d.n_q_heads * d.head_dim * n * (n + 1) / 2
        ach = flops * args.steps / (ms * 1e-3) / 1e12
        t0 = time.perf_counter()
        rt.set_data(ids); rt.execute({"s": n, "p": 0}); rows_token = rt.get_token()
        e2e = n / (time.perf_counter() - t0)
        rows_logits = rt.get_f32()
        launches = int(rt.stats().kernel_launches)
        rt.close()
        parity = _prefill_parity(pkg, base, ids, rows_token, rows_logits)
        line = {"metric": "q8_llama3_8b_prefill4096_tokens_per_s", "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16 x f16 -> f32 on tcgen05 (weights as two exact binary16 terms, activations as two); attention bf16 x bf16 -> f32 on tcgen05 (two-term queries and weights)", "data": "synthetic",
                "config": {"workload": which, "batch": 1, "prompt_len": n, "seed": SEED},
                "roofline": {"bound": "tensor", "kernel": "whole prompt (q8_gemm_tc 85 %, attn_prompt_tc 11 % of the time)", "achieved": ach, "peak": peaks.get("bf16_tflops_sustained", 1383.9),
                             "unit": "TFLOP/s", "frac": ach / peaks.get("bf16_tflops_sustained", 1383.9), "peak_kind": f"of {peak_kind} (sustained bf16 GEMM)",
                             "flops_per_step": flops, "traffic": None},
                "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": 4,
                        "note": "token ids host->device, the sampled token device->host"},
                "parity": parity, "gpu_launches": launches, "clocks": clocks}
    print(json.dumps(line))


def _prefill_parity(pkg, base, ids, rows_token, rows_logits):
    """Against the oracle's committed fixture for this very prompt (tests/golden/llama3_8b_q8_prefill4096_full.npz: whole model, 4096
    rows, the logits after the last prompt token and the greedy sample) when it is there; otherwise the prompt once more, one
    decode step per token (the path the default workload checks against the oracle's fixture): logits and sample must agree with
    the rows pass."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "llama3_8b_q8_prefill4096_full.npz")
    if os.path.exists(path):
        fx = np.load(path)
        if int(fx["seed"]) == SEED and list(fx["prompt"]) == list(ids):
            ref = fx["prompt_logits"].astype(np.float32)
            err = float(np.max(np.abs(rows_logits - ref)) / np.max(np.abs(ref)))
            return {"checked": True, "tokens_equal": bool(int(fx["tokens"][0]) == int(rows_token)), "steps": 1, "logits_rel_err": err,
                    "logits_tolerance": 1e-2, "min_margin_of_fixture": float(fx["margins"][0]), "fixture": os.path.relpath(path, ROOT)}
    solo = pkg.B200Runtime.initialize(device=0, prefill_min_rows=1 << 30)
    try:
        solo.load_model(base.copy(max_seq=len(ids) + 8))
        solo.synth(SEED)
        solo.set_data(ids); solo.execute({"s": len(ids), "p": 0})
        tok, ref = solo.get_token(), solo.get_f32()
    finally:
        solo.close()
    err = float(np.max(np.abs(rows_logits - ref)) / np.max(np.abs(ref)))
    top2 = np.partition(ref, -2)[-2:]
    return {"checked": True, "against": "the same prompt run one decode step per token on the GPU (that path is checked against the oracle's "
            "full-size fixture by the default workload; the oracle itself would need hours for 4096 rows)",
            "tokens_equal": bool(tok == rows_token), "steps": 1, "logits_rel_err": err, "logits_tolerance": 1e-2,
            "top1_top2_margin": float(top2[1] - top2[0])}


def _batch_parity(pkg, base, ctx, n_run, firsts, batch_log, batch_logits, B):
    """The first and the last sequence of the batch decoded alone, one decode step per token: same tokens for the first 32
    steps; if a sequence agrees to the end of the run, the final logits are compared too."""
    import numpy as np
    n_cmp = min(32, n_run)
    out = {"checked": True, "against": "sequences 0 and %d decoded alone, one decode step per token, on the GPU (that path is checked against the "
           "oracle's full-size fixture by the default workload)" % (B - 1), "steps": n_cmp, "tokens_equal": True, "first_mismatch": None,
           "logits_rel_err": None, "logits_tolerance": 1e-2}
    solo = pkg.B200Runtime.initialize(device=0)
    try:
        solo.load_model(base.copy(max_seq=ctx + n_run + 8, max_new_tokens=n_run + 8))
        solo.synth(SEED)
        for sq in (0, B - 1):
            ids = _prompt_tokens(base.vocab, ctx + sq)[sq:]
            got = [int(firsts[sq])] + [int(t) for t in batch_log[:, sq]]
            want = solo.generate(ids, n_run + 1)
            bad = next((i for i in range(n_cmp) if got[i] != want[i]), None)
            if bad is not None:
                out["tokens_equal"] = False
                out["first_mismatch"] = {"sequence": sq, "step": bad}
            elif got == want:
                ref = solo.get_f32()
                err = float(np.max(np.abs(batch_logits[sq] - ref)) / np.max(np.abs(ref)))
                out["logits_rel_err"] = err if out["logits_rel_err"] is None else max(err, out["logits_rel_err"])
    finally:
        solo.close()
    return out


def run_moe(args, pkg):
    """gpt-oss-20B-shape mixture of experts: every rank decodes its own sequence (batch = number of GPUs), the experts are spread
    over the ranks and every layer's tokens travel to them and back all-to-all (NCCL).  On one GPU: batch 1, all experts local.
    A "step" is `--tokens-per-step` tokens of every sequence; `value` is the tokens/s of all sequences together (weak scaling)."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks, peak_kind = measured_peaks()
    base = pkg.CONFIGS["gpt_oss_20b_q8"]
    n_prompt = PROMPT_LEN if PROMPT_LEN != 512 else 2048
    tps = TOKENS_PER_STEP
    total = (args.warmup + args.steps) * tps
    desc = base.copy(max_seq=n_prompt + total + 8, max_new_tokens=total + 8)
    rt = pkg.B200Runtime.initialize(device=local)
    if world > 1:
        from oneiron_luminal_b200 import tp as T
        T.validate_ep(desc, world)
        uid = T.exchange_unique_id(dist, rank, pkg.B200Runtime.tp_unique_id, device=torch.device("cuda", local))
        rt.tp_init(uid, world, rank)
        desc = desc.copy(ep_size=world, ep_rank=rank)
    rt.load_model(desc)
    rt.synth(SEED)
    prompt = _prompt_tokens(base.vocab, n_prompt + rank)[rank:]
    rt.kv_reset(); rt.decode_reset()
    rt.set_data(prompt); rt.execute({"s": n_prompt, "p": 0})
    rt.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        rt.decode_greedy(tps)
    ext = torch.cuda.ExternalStream(rt.stream(), device=torch.device("cuda", local))
    sampler = ClockSampler(physical_gpu_index(local))
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    for _ in range(args.steps):
        rt.decode_greedy(tps)
    e1.record(ext)
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    n_tok = args.steps * tps
    value = world * n_tok / (ms * 1e-3)
    st = rt.stats()
    parity = _moe_parity(rt, world, dist, torch)
    p_mean = n_prompt + (args.warmup + args.steps / 2.0) * tps
    # a token reads the attention weights, the router, top-4 experts and the vocabulary projection; K/V rows of the full layers up to
    # its position and at most 128 on the windowed layers
    kv_row = st.kv_bytes_per_position / base.n_layers
    kv_bytes = kv_row * (base.n_layers / 2 * (p_mean + 1) + base.n_layers / 2 * min(p_mean + 1, base.sliding_window))
    bytes_tok = st.weight_bytes_per_token + kv_bytes
    ach = bytes_tok * (value / world) / 1e9
    line = None
    if rank == 0:
        line = {"metric": "q8_gpt_oss_20b_decode_tokens_per_s", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32 accumulate over Q8_0 weights", "data": "synthetic",
                "config": {"workload": "gpt_oss_20b_q8", "batch": world, "prompt_len": n_prompt, "tokens_per_step": tps, "seed": SEED,
                           "parallelism": "single GPU, all experts local" if world == 1 else f"ep{world}: one sequence per GPU, {base.n_experts // world} experts per GPU, all-to-all dispatch and combine per layer (NCCL)"},
                "roofline": {"bound": "hbm", "kernel": "whole decode step of one rank", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": ach / peaks["hbm_gbs"], "peak_kind": f"of {peak_kind}", "bytes_per_token": bytes_tok, "traffic": None},
                "e2e": {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "note": "not measured for this workload"},
                "parity": parity, "gpu_launches": int(st.kernel_launches), "clocks": clocks}
    rt.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line))


def _moe_parity(rt, world, dist, torch):
    """The oracle's committed full-size fixture for this model: its 256-token prompt and 32 greedy tokens, run by every rank
    (under expert parallelism all ranks step together, so all decode the fixture's sequence)."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "gpt_oss_20b_q8_full.npz")
    if not os.path.exists(path):
        return {"checked": False, "reason": f"no fixture {os.path.relpath(path, ROOT)}"}
    fx = np.load(path)
    if int(fx["seed"]) != SEED:
        return {"checked": False, "reason": "fixture was made for another seed"}
    prompt, want = [int(t) for t in fx["prompt"]], [int(t) for t in fx["tokens"]]
    if len(prompt) + len(want) + 1 > rt.desc.max_seq or len(want) > rt.desc.max_new_tokens:
        return {"checked": False, "reason": "this run's cache or token log is smaller than the fixture's sequence"}
    rt.kv_reset(); rt.decode_reset()
    rt.set_data(prompt); rt.execute({"s": len(prompt), "p": 0})
    first, logits = rt.get_token(), rt.get_f32()
    rt.decode_greedy(len(want) - 1)
    got = [int(first)] + [int(t) for t in rt.get_decoded(len(want) - 1)]
    ref = fx["prompt_logits"].astype(np.float32)
    err = float(np.max(np.abs(logits - ref)) / np.max(np.abs(ref)))
    equal = got == want
    if world > 1:
        t = torch.tensor([err, 0.0 if equal else 1.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err, equal = float(t[0].item()), float(t[1].item()) == 0.0
    return {"checked": True, "tokens_equal": bool(equal), "steps": len(want), "logits_rel_err": err, "logits_tolerance": 1e-2,
            "first_mismatch": next((i for i in range(len(want)) if got[i] != want[i]), None),
            "min_margin_of_fixture": float(np.min(fx["margins"])), "fixture": os.path.relpath(path, ROOT)}


def _prompt_tokens(vocab: int, n: int):
    """The seeded prompt, generated without the oracle: SplitMix64 counter generator, tensor id 2^20."""
    mask = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    g = 0x9E3779B97F4A7C15
    key = mix((SEED + g * ((1 << 20) + 1)) & mask)
    return [((mix((key + g * (2 * i)) & mask) >> 32) * vocab) >> 32 for i in range(n)]


def main():
    global PROMPT_LEN, TOKENS_PER_STEP
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--report", default=None, help="also write the byte / flop counts of the timed step as a metrics JSON in the reference bench crate's format")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt tokens before the timed decode (profiling runs use a short one)")
    ap.add_argument("--tokens-per-step", type=int, default=TOKENS_PER_STEP)
    ap.add_argument("--workload", default=WORKLOAD, choices=["llama3_8b_q8", "qwen3_4b_q8", "llama3_8b_q8_bs32", "llama3_8b_q8_prefill4096", "gpt_oss_20b_q8"],
                    help="llama3_8b_q8: the configuration the metric is quoted on (default); qwen3_4b_q8: the Qwen3-4B shape; "
                         "llama3_8b_q8_bs32 / llama3_8b_q8_prefill4096: the same model in the tensor-core regime (batched decode / one long prompt)")
    ap.add_argument("--only", default="all", choices=["all", "kernel", "sweep", "floor", "gemm", "gemm512", "gemm32", "prompt2", "sampler"],
                    help="kernel: time only the dominant kernel alone (small, for ncu captures); sweep: the kernel alone over a range of row counts; "
                         "floor: the decode step with all projections shrunk away; gemm: the tensor-core GEMM alone on the layer's shapes "
                         "(gemm512 / gemm32: the gate+up shape only, 512 / 32 rows, for ncu captures); prompt2: a 4096-token prompt through a 2-layer cut; "
                         "sampler: the top-k / top-p sampler alone and its cost inside the decode loop")
    args = ap.parse_args()
    from __graft_entry__ import load_package
    pkg = load_package()
    PROMPT_LEN, TOKENS_PER_STEP = args.prompt_len, args.tokens_per_step
    if args.workload == "gpt_oss_20b_q8":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU arm is timed on the batch-1 dense decode workloads only"}))
            return
        run_moe(args, pkg)
        return
    if args.workload in ("llama3_8b_q8_bs32", "llama3_8b_q8_prefill4096"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the CPU arm is timed on the batch-1 decode workloads only"}))
            return
        run_tensor_core_regime(args, pkg, args.workload)
        return
    if args.workload != WORKLOAD:
        set_workload(args.workload, prompt_given=args.prompt_len != 512)
    if args.only == "kernel":
        import torch
        torch.cuda.set_device(0)
        peaks, kind = measured_peaks()
        roof, _ = kernel_roofline(pkg, torch, peaks, kind)
        print(json.dumps({"roofline": roof}))
        return
    if args.only == "sweep":
        import torch
        torch.cuda.set_device(0)
        print(json.dumps({"rows_sweep": kernel_rows_sweep(pkg, torch)}))
        return
    if args.only in ("gemm", "gemm512", "gemm32"):
        import torch
        torch.cuda.set_device(0)
        shapes = {"gemm": None, "gemm512": [(28672, 4096, 512)], "gemm32": [(28672, 4096, 32)]}[args.only]
        print(json.dumps({"gemm_shapes": gemm_shapes(pkg, torch, shapes)}))
        return
    if args.only == "prompt2":
        import torch
        torch.cuda.set_device(0)
        print(json.dumps({"prompt_two_layers": prompt_two_layers(pkg, torch)}))
        return
    if args.only == "sampler":
        import torch
        torch.cuda.set_device(0)
        print(json.dumps({"sampler": sampler_times(pkg, torch)}))
        return
    if args.only == "floor":
        import torch
        torch.cuda.set_device(0)
        print(json.dumps({"launch_chain_floor": launch_chain_floor(pkg, torch)}))
        return
    if args.impl == "reference":
        run_reference_arm(args, pkg)
    else:
        run_ours(args, pkg)


if __name__ == "__main__":
    main()
