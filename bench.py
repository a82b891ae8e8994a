#!/usr/bin/env python
"""Benchmark of the quantized forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One GPU (the default).  Headline workload: the Llama-3.2-1B-shaped Q4_0 decoder of the benchmark definition - one
"step" is one request: a 1501-token uniform-random prompt through the batched prefill path, then 128 greedy decode
steps at batch 1, fp16 paged KV cache.  Reported metric: decode tok/s (the prefill tok/s of the same requests rides
along under "prefill").  `value` is device time (CUDA events on the library's stream, tokens resident on the GPU);
`e2e` is the same work timed on the host around the C-ABI calls with host buffers in and out.  The line also
carries, under "configs", one sub-record per other benchmark configuration measured in the same process (the
SmolLM2-135M shape, the Qwen2.5-0.5B shape with 64 requests in flight, the Phi-3-mini shape at batch 1 and batch 16,
the Llama-2-7B shape at batch 8), each with its own decode / prefill rates, roofline fraction and host-timed rate.

N GPUs (torchrun, one rank per GPU).  The headline becomes the request-sharded workload of the benchmark definition:
the Qwen2.5-0.5B-shaped Q8_0 decoder, 64 independent requests per GPU with prompt lengths uniform in [64, 2501]
(`default_rng(2).integers(64, 2502, size=64 N)`, partitioned by `parallel.shard_requests`), 64 decode steps each, no
collective on the data path; `value` is the aggregate decode tok/s over max-over-ranks device time ("weak" scaling).
A "tp" sub-record runs the Llama-2-7B-shaped Q4_0 decoder cut over the N ranks (tensor parallel, batch 8 x 2048-token
prompts, 128 decode steps; strong scaling) and checks a two-layer cut of it against the CPU restatement.

Weights are synthetic (N(0, 0.02), seed 0, quantised to GGUF Q8_0 / Q4_0); there is no network for checkpoints.
Generated images are kept under /tmp between runs on the same machine.

`--impl reference` times the reference's CPU path instead: the C++ restatement of the generated x86 code (the Rust
original cannot be built here) on all host cores, each step a bounded sample of the arm's headline workload.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_PROMPT = {"c1": 100, "c2": 1501, "c3": 2501, "c4": 3001, "c5": 2048}
N_DECODE = {"c1": 64, "c2": 128, "c3": 64, "c4": 256, "c5": 128}
C3_REQUESTS_PER_GPU = 64
CACHE_DIR = os.path.join("/tmp", "forge_b200_bench_cache")


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (read-only query)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for (ts, r) in self.rows if t0 <= ts <= t1 + 0.2 and len(r) >= 9] or [r for (_, r) in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            for i, n in enumerate(names):
                if r[5 + i].lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]), "power_w_max": max(float(r[3]) for r in rows),
                "samples": len(rows), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------- synthetic inputs
REPEAT_LAYERS = {"c4", "c5"}   # multi-billion-parameter shapes: layer 0 is drawn, its bytes repeat (host time)


def model_inputs(cfg_key: str, quantize_fn=None, tag: str = "lib", layers: int | None = None, vocab: int | None = None):
    """(config, weights.bin image, prompt tokens) of a benchmark configuration; the image is kept under /tmp."""
    from forge_llm_b200 import configs, synth
    c = configs.CONFIGS[cfg_key] if layers is None else configs.reduced(cfg_key, layers, vocab)
    repeat = cfg_key in REPEAT_LAYERS and layers is None
    toks = synth.prompt_tokens(c, N_PROMPT[cfg_key], seed=1)
    name = hashlib.sha1(json.dumps([c, repeat, tag], sort_keys=True).encode()).hexdigest()[:16]
    path = os.path.join(CACHE_DIR, f"{c['name']}-{name}.npy")
    need = synth.weights_bin_size(c)
    try:
        if os.path.exists(path) and os.path.getsize(path) >= need:
            return c, np.load(path, mmap_mode="r"), toks, repeat
    except Exception:
        pass
    blob = synth.make_weights_bin(c, seed=0, quantize_fn=quantize_fn, repeat_layers=repeat)
    try:
        os.makedirs(CACHE_DIR, exist_ok=True)
        if shutil.disk_usage(CACHE_DIR).free > need + (40 << 30):
            tmp = f"{path}.{os.getpid()}.tmp"
            with open(tmp, "wb") as f:
                np.save(f, blob)
            os.replace(tmp, path)
    except Exception:
        pass
    return c, blob, toks, repeat


def quant_name(c: dict) -> str:
    return "Q4_0" if c["quant"] == 4 else "Q8_0"


def dtype_name(c: dict) -> str:
    return f"f32 x (int{c['quant']} * f16 block scale), f32 accumulate"


# ---------------------------------------------------------------------------- CPU reference arm
def oracle_quantize_fn():
    from oracle import oracle as O
    return lambda quant, w: (O.quantize_q8_0(w) if quant == 8 else O.quantize_q4_0(w, rule="signed"))


def time_oracle(c, blob, toks, n_prefill: int, n_decode: int, repeats: int):
    """Scalar port of the reference's x86 path (kind "port"), all host threads.  One repeat =
    a batched prefill of `n_prefill` prompt tokens followed by `n_decode` greedy steps."""
    from oracle import oracle as O
    O.lib().fo_set_num_threads(os.cpu_count() or 1)   # launchers pin OMP_NUM_THREADS=1 for their workers
    m = O.OracleModel(c, np.ascontiguousarray(blob), kv_mode=O.KV_INT8, fast=False)
    pre, dec = [], []
    for _ in range(repeats):
        m.reset()
        t0 = time.perf_counter()
        logits = m.forward_prefill(toks[:n_prefill])
        t1 = time.perf_counter()
        for _ in range(n_decode):
            logits = m.forward(O.argmax(logits))
        t2 = time.perf_counter()
        pre.append(t1 - t0)
        dec.append(t2 - t1)
    return n_prefill / statistics.median(pre), n_decode / statistics.median(dec), O.lib().fo_num_threads()


def run_reference(args, rank: int):
    if rank != 0:
        return
    key = "c2" if args.gpus <= 1 else "c3"
    c, blob, toks, _ = model_inputs(key, quantize_fn=oracle_quantize_fn(), tag="oracle")   # no CUDA library in this process
    n_pre, n_dec = 16, 2
    sample = (f"{n_pre}-token batched prefill + {n_dec} greedy decode steps (context {n_pre}..{n_pre + n_dec}, not the arm's "
              f"{N_PROMPT[key]}+) per step, int8 KV, scalar x86 loops")
    for _ in range(args.warmup):
        time_oracle(c, blob, toks, n_pre, n_dec, 1)
    t0 = time.perf_counter()
    pre, dec, threads = time_oracle(c, blob, toks, n_pre, n_dec, args.steps)
    wall = time.perf_counter() - t0
    line = {
        "impl": "reference", "metric": "decode_tok_s", "value": dec, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * wall / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype_name(c), "data": "synthetic",
        "config": headline_config(key, c, args.gpus),
        "prefill": {"value": pre, "unit": "tok/s"},
        "cpu_baseline": {"value": dec, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": dec, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def headline_config(key: str, c: dict, gpus: int) -> dict:
    if gpus <= 1:
        work = f"{c['name']}: {N_PROMPT[key]}-token prompt (batched prefill) + {N_DECODE[key]} greedy decode steps, batch 1"
        par = "one GPU"
    else:
        work = (f"{c['name']}: {C3_REQUESTS_PER_GPU} independent requests per GPU, prompt lengths uniform in [64, 2501], "
                f"{N_DECODE[key]} greedy decode steps each")
        par = f"request-sharded over {gpus} GPUs (one model replica per GPU, no collective on the data path)"
    return {"workload": work, "config_key": key, "quant": quant_name(c), "kv_cache": "fp16 paged (64 positions per page)",
            "prompt_tokens": N_PROMPT[key], "decode_steps": N_DECODE[key], "parallelism": par,
            "l2": "inputs larger than L2: every decode step streams the whole weight set (>= 143 MB) once"}


# DRAM bytes moved per algorithmic byte of the streaming GEMV (dram__bytes_read + dram__bytes_write of one captured
# launch, 153.6 MB for 147.75 MB of weights; the capture is summarised under profiles/).  A decode step is one graph
# replay of such kernels; its traffic is scaled from that capture by the bytes it streams.
DRAM_TRAFFIC_RATIO = 1.04
TRAFFIC_NOTE = "scaled from one ncu capture of the GEMV kernel (traffic/algorithmic = 1.04)"
# The prompt's dominant kernel is the gate/up GEMM (tcgen05, SiLU epilogue): one captured launch at m = 1501 read
# 31.5 MB and wrote 6.2 MB of DRAM (weights 18.9 MB + fp16 hi/lo rows 12.3 MB in; most of its output is still in L2 when
# it ends); the capture is summarised under profiles/.  Reported for the headline prompt length only.
PREFILL_GEMM_TRAFFIC = {"c2": (1501, 37.7e6)}
PREFILL_TRAFFIC_NOTE = "dram read + write of one ncu-captured launch of the dominant kernel (gate/up GEMM, m = 1501)"


# ---------------------------------------------------------------------------- GPU workloads
def run_requests(model, c, prompts, n_dec, reps, warm):
    """`len(prompts)` requests in flight on one model: every prompt through the batched prefill into its own sequence of
    one cache, then `n_dec` greedy steps of all sequences together.  Returns device- and host-timed rates."""
    from forge_llm_b200 import configs
    B = len(prompts)
    kv = model.new_cache(max_seq=max(len(p) for p in prompts) + n_dec + 8, batch=B)
    dev_dec, host_dec, host_pre, launches = [], [], [], 0
    ids = None
    for it in range(warm + reps):
        kv.reset()
        t0 = time.perf_counter()
        first = np.empty(B, np.uint32)
        for b, p in enumerate(prompts):
            lg = model.forward_prefill(p, kv, seq=b)                              # H2D prompt, D2H logits
            first[b] = int(np.flatnonzero(lg == lg.max())[-1])                    # host argmax, last index on ties
        t1 = time.perf_counter()
        ids = model.decode_greedy_batch(first, n_dec, kv)                         # H2D first tokens, D2H ids
        t2 = time.perf_counter()
        _, dms, nl = model.last_timing()
        if it >= warm:
            host_pre.append(t1 - t0)
            host_dec.append(t2 - t1)
            dev_dec.append(dms / 1e3)
            launches += nl
    kv.close()
    ptoks = sum(len(p) for p in prompts)
    ctx_mid = [len(p) + n_dec // 2 for p in prompts]
    bytes_step = configs.decode_bytes_per_token(c, 0) + sum(configs.decode_bytes_per_token(c, x) - configs.decode_bytes_per_token(c, 0) for x in ctx_mid)
    return {"batch": B, "ids": ids, "decode_s": sum(dev_dec), "host_decode_s": sum(host_dec), "host_prefill_s": sum(host_pre), "reps": reps,
            "decode_tokens": B * n_dec * reps, "prefill_tokens": ptoks * reps, "bytes_per_step": bytes_step, "launches": launches,
            "prefill_flops": sum(configs.prefill_flops(c, len(p)) for p in prompts) * reps,
            "h2d": int(sum(len(p) for p in prompts) * 4 + B * 4), "d2h": int(B * c["vocab_size"] * 4 + B * n_dec * 4)}


def sub_record(c, r, peaks, note=None):
    step_s = r["decode_s"] / (r["reps"] * (r["decode_tokens"] // (r["reps"] * r["batch"])))
    achieved = r["bytes_per_step"] / step_s / 1e9
    pre_tf = r["prefill_flops"] / r["host_prefill_s"] / 1e12
    out = {"workload": f"{c['name']}: batch {r['batch']}", "quant": quant_name(c), "value": r["decode_tokens"] / r["decode_s"], "unit": "tok/s",
           "us_per_step": step_s * 1e6,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                        "bytes_per_launch": r["bytes_per_step"], "traffic": None, "peak_source": peaks["source"]},
           "prefill": {"value": r["prefill_tokens"] / r["host_prefill_s"], "unit": "tok/s", "timing": "host, around the C-ABI calls",
                       "roofline": {"bound": "tensor", "achieved": pre_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                    "frac": pre_tf / peaks["bf16_tflops"], "traffic": None}},
           "e2e": {"value": r["decode_tokens"] / r["host_decode_s"], "unit": "tok/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
           "reps": r["reps"]}
    if note:
        out["weights"] = note
    return out


def side_configs(device, peaks, log):
    """The other benchmark configurations on one GPU (one warm-up + two timed repetitions each)."""
    from forge_llm_b200 import runtime, synth
    out = {}

    def one(name, key, batch, lens=None):
        t0 = time.time()
        c, blob, toks, repeat = model_inputs(key)
        model = runtime.Model(c, blob, device=device)
        if lens is None:
            prompts = [synth.prompt_tokens(c, N_PROMPT[key], seed=1 + b) for b in range(batch)]
        else:
            prompts = [synth.prompt_tokens(c, int(n), seed=100 + i) for i, n in enumerate(lens)]
        r = run_requests(model, c, prompts, N_DECODE[key], reps=2, warm=1)
        model.close()
        out[name] = sub_record(c, r, peaks, "layer 0 drawn from the seed, its bytes repeated for the other layers" if repeat else None)
        if lens is not None:
            out[name]["workload"] = f"{c['name']}: {len(lens)} requests in flight, prompt lengths uniform in [64, 2501]"
        log(f"{name}: {out[name]['value']:.0f} tok/s decode, frac {out[name]['roofline']['frac']:.3f}, {time.time() - t0:.0f} s")

    one("c1", "c1", 1)
    lens = np.random.default_rng(2).integers(64, 2502, size=C3_REQUESTS_PER_GPU)
    one("c3", "c3", C3_REQUESTS_PER_GPU, lens)
    one("c3_b1", "c3", 1)
    one("c4_b1", "c4", 1)
    one("c4_b16", "c4", 16)
    one("c5", "c5", 8)
    one("c5_b1", "c5", 1)
    return out


# ---------------------------------------------------------------------------- one GPU: the headline
def run_single(args, device: int):
    import torch
    from forge_llm_b200 import configs, runtime

    def log(msg):
        print(f"[bench] {msg}", file=sys.stderr, flush=True)

    key = "c2"
    c, blob, toks, _ = model_inputs(key)
    n_prompt, n_dec = N_PROMPT[key], N_DECODE[key]
    model = runtime.Model(c, blob, device=device)
    kv = model.new_cache(max_seq=n_prompt + n_dec + 8)
    pinned_prompt = torch.from_numpy(toks.astype(np.int32)).pin_memory()  # H2D source of every step
    prompt_np = pinned_prompt.numpy().view(np.uint32)

    def one_step():
        """One request through the public API, token selection on the device."""
        kv.reset()
        out = model.generate_greedy(prompt_np, n_dec, kv)  # host prompt in, host ids out
        pre_ms, dec_ms, launches = model.last_timing()
        return pre_ms, dec_ms, launches, out

    def one_step_e2e():
        """The same request as two host-timed C-ABI calls (prefill, then the decode loop)."""
        kv.reset()
        h0 = time.perf_counter()
        logits = model.forward_prefill(prompt_np, kv)        # H2D prompt, D2H logits
        h1 = time.perf_counter()
        first = np.array([int(np.flatnonzero(logits == logits.max())[-1])], np.uint32)  # host argmax, last index on ties
        h2 = time.perf_counter()
        ids = model.decode_greedy_batch(first, n_dec, kv)    # H2D first token, D2H ids
        h3 = time.perf_counter()
        return h1 - h0, h3 - h2, ids

    n_warm = args.warmup if args.profile else max(args.warmup, 3)
    for _ in range(n_warm):
        one_step()
        if not args.profile:
            one_step_e2e()
    sampler = ClockSampler(device)
    torch.cuda.synchronize()
    t0 = time.time()
    w0 = time.perf_counter()
    pre_ms, dec_ms, launches, ids0 = [], [], 0, None
    for _ in range(args.steps):
        p, d, l, ids = one_step()
        pre_ms.append(p)
        dec_ms.append(d)
        launches += l
        ids0 = ids
    torch.cuda.synchronize()
    w1 = time.perf_counter()
    e2e_pre, e2e_dec = [], []
    for _ in range(args.steps):
        a, b, ids_e = one_step_e2e()
        e2e_pre.append(a)
        e2e_dec.append(b)
    torch.cuda.synchronize()
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    assert np.array_equal(ids_e[:, 0], ids0), "device-side and host-side greedy loops disagree"
    kv.close()
    model.close()

    K = args.steps
    dec_s, pre_s = sum(dec_ms) / 1e3, sum(pre_ms) / 1e3
    peaks = load_peaks()
    ctx_mid = n_prompt + n_dec // 2
    bytes_tok = configs.decode_bytes_per_token(c, ctx_mid)
    step_s = dec_s / (K * n_dec)
    achieved = bytes_tok / step_s / 1e9
    flops = configs.prefill_flops(c, n_prompt)
    pre_tf = flops / (pre_s / K) / 1e12
    line = {
        "metric": "decode_tok_s", "value": K * n_dec / dec_s, "unit": "tok/s", "n_gpus": 1, "steps": K,
        "warmup": n_warm, "ms_per_step": 1e3 * (w1 - w0) / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype_name(c), "data": "synthetic",
        "config": headline_config(key, c, 1),
        "prefill": {"value": K * n_prompt / pre_s, "unit": "tok/s", "gemm": "tcgen05/TMEM, fp16 hi/lo split, 3 tensor-core passes",
                    "roofline": {"bound": "tensor", "achieved": pre_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                 "frac": pre_tf / peaks["bf16_tflops"],
                                 "traffic": PREFILL_GEMM_TRAFFIC[key][1] if PREFILL_GEMM_TRAFFIC.get(key, (0, 0))[0] == n_prompt else None,
                                 "traffic_source": PREFILL_TRAFFIC_NOTE, "peak_source": peaks["source"], "flops_per_step": flops}},
        "roofline": {"bound": "hbm", "kernel": "one decode step (all kernels of forward(), replayed as one CUDA graph)",
                     "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": bytes_tok * DRAM_TRAFFIC_RATIO, "traffic_source": TRAFFIC_NOTE,
                     "peak_source": peaks["source"], "bytes_per_launch": bytes_tok, "ctx": ctx_mid,
                     "us_per_launch": step_s * 1e6},
        "e2e": {"value": K * n_dec / sum(e2e_dec), "unit": "tok/s", "h2d_bytes_per_step": int(prompt_np.nbytes + 4),
                "d2h_bytes_per_step": int(c["vocab_size"] * 4 + n_dec * 4), "prefill_tok_s": K * n_prompt / sum(e2e_pre)},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if args.profile:
        line["note"] = "profiling run (--profile): not a benchmark value"
    if not args.no_side_configs and not args.profile:
        line["configs"] = side_configs(device, peaks, log)
    if not args.no_cpu_baseline and not args.profile:
        pre, dec, threads = time_oracle(c, blob, toks, 16, 2, 2)
        line["cpu_baseline"] = {"value": dec, "unit": "tok/s", "cores": threads, "kind": "port", "prefill_tok_s": pre,
                                "sample": "16-token batched prefill + 2 greedy decode steps (context 16..18), median of 2, int8 KV, scalar x86 loops"}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- N GPUs: request sharding + tensor parallel
def run_multi(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    from forge_llm_b200 import configs, parallel, runtime, synth

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(vals):
        t = torch.tensor(vals, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def reduce_sum(vals):
        t = torch.tensor(vals, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t.tolist()

    peaks = load_peaks()
    # ---- request sharding: rank 0 makes the weights image first (the others then find it under /tmp)
    key = "c3"
    if rank == 0:
        model_inputs(key)
    barrier()
    c, blob, _, _ = model_inputs(key)
    lens_all = np.random.default_rng(2).integers(64, 2502, size=C3_REQUESTS_PER_GPU * world)
    mine = parallel.shard_requests(len(lens_all), rank, world)
    prompts = [synth.prompt_tokens(c, int(lens_all[i]), seed=100 + i) for i in mine]
    model = runtime.Model(c, blob, device=local_rank)
    n_dec = N_DECODE[key]
    run_requests(model, c, prompts, n_dec, reps=1, warm=max(args.warmup, 3) - 1)   # warm-up (the last warm-up is inside the timed call below)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    t0 = time.time()
    w0 = time.perf_counter()
    r = run_requests(model, c, prompts, n_dec, reps=args.steps, warm=0)
    barrier()
    w1 = time.perf_counter()
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if sampler else None
    model.close()
    dec_s, hdec_s, hpre_s, wall = reduce_max([r["decode_s"], r["host_decode_s"], r["host_prefill_s"], w1 - w0])
    dtok, ptok, launches, pflops = reduce_sum([r["decode_tokens"], r["prefill_tokens"], r["launches"], r["prefill_flops"]])
    per_rank = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(world)]
    dist.all_gather(per_rank, torch.tensor([r["decode_tokens"] / r["decode_s"]], dtype=torch.float64, device="cuda"))
    step_s = r["decode_s"] / (args.steps * n_dec)
    achieved = r["bytes_per_step"] / step_s / 1e9
    line = {
        "metric": "decode_tok_s", "value": dtok / dec_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": 1e3 * wall / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype_name(c), "data": "synthetic", "config": headline_config(key, c, world),
        "per_rank_tok_s": [float(x.item()) for x in per_rank],
        "prefill": {"value": ptok / hpre_s, "unit": "tok/s", "timing": "host, around the C-ABI calls, max over ranks",
                    "roofline": {"bound": "tensor", "achieved": pflops / hpre_s / 1e12 / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s per GPU",
                                 "frac": pflops / hpre_s / 1e12 / world / peaks["bf16_tflops"], "traffic": None}},
        "roofline": {"bound": "hbm", "kernel": "one decode step of 64 sequences on rank 0 (weights once + every sequence's K/V)", "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                     "bytes_per_launch": r["bytes_per_step"], "us_per_launch": step_s * 1e6, "peak_source": peaks["source"]},
        "e2e": {"value": dtok / hdec_s, "unit": "tok/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                "prefill_tok_s": ptok / hpre_s},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    # ---- tensor parallel: the Llama-2-7B shape cut over all ranks
    if not args.no_tp:
        try:
            line["tp"] = run_tp(args, rank, world, local_rank, dist, barrier, reduce_max, peaks)
        except Exception as e:  # the headline stands on its own
            line["tp"] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def run_tp(args, rank, world, local_rank, dist, barrier, reduce_max, peaks):
    import torch
    from forge_llm_b200 import configs, runtime, synth

    def tp_model(c, blob, peer_sums=True):
        uid = torch.from_numpy(runtime.Model.tp_unique_id() if rank == 0 else np.zeros(runtime.TP_ID_BYTES, np.uint8)).cuda()
        dist.broadcast(uid, 0)
        m = runtime.Model(c, blob, device=local_rank, tp_rank=rank, tp_world=world)
        m.tp_init(uid.cpu().numpy())
        if peer_sums:   # decode sums over peer memory (NVLink stores); the handles travel over a host channel with a time limit
            from forge_llm_b200 import parallel
            m.tp_exchange_attach(parallel.gather_exchange_handles(m.tp_exchange_handle(), world))
            dist.barrier()
        return m

    out = {"model": configs.CONFIGS["c5"]["name"], "parallelism": f"tensor-parallel over {world} GPUs: q/k/v and gate/up by rows, o and down by input columns",
           "sum": "prompt: NCCL all-reduce after o and down on the model's stream; batch-1 decode: {value, tag} pairs stored into every peer's exchange "
                  "buffer from the projection's epilogue, summed by the next kernel while it stages its input (no collective kernel); batched decode: the "
                  "same, pairs stored from the batched product's epilogue and added by the next product's packing kernel",
           "scaling": "strong"}
    # parity of the cut: two layers, 8192-token vocabulary, against the CPU restatement (rank 0 checks)
    cp, blobp, _, _ = model_inputs("c5", layers=2, vocab=8192) if rank == 0 else (None, None, None, None)
    barrier()
    cp, blobp, _, _ = model_inputs("c5", layers=2, vocab=8192)
    toks = synth.prompt_tokens(cp, 24, seed=7)
    m = tp_model(cp, blobp)
    kv = m.new_cache(max_seq=64)
    lg = m.forward_prefill(toks, kv)
    kv.reset()
    ids = m.generate_greedy(toks, 16, kv)
    kv.close()
    m.close()
    if rank == 0:
        from oracle import oracle as O
        O.lib().fo_set_num_threads(os.cpu_count() or 1)
        om = O.OracleModel(cp, np.ascontiguousarray(blobp), kv_mode=O.KV_F16)
        lo = om.forward_prefill(toks)
        om.reset()
        ref_ids, _ = om.generate_greedy(toks, 16)
        out["tp_parity"] = {"model": cp["name"], "logit_max_abs_err": float(np.abs(lg - lo).max()), "greedy_ids_equal": bool(np.array_equal(ids, ref_ids)),
                            "checked_against": "CPU restatement, fp16 KV stand-in"}
    barrier()
    # timing: batch 8 x 2048-token prompts + 128 steps, and batch 1
    key = "c5"
    if rank == 0:
        model_inputs(key)
    barrier()
    c, blob, _, repeat = model_inputs(key)
    m = tp_model(c, blob)
    for name, batch in (("batch8", 8), ("batch1", 1)):
        prompts = [synth.prompt_tokens(c, N_PROMPT[key], seed=1 + b) for b in range(batch)]
        run_requests(m, c, prompts, N_DECODE[key], reps=1, warm=0)
        barrier()
        r = run_requests(m, c, prompts, N_DECODE[key], reps=2, warm=0)
        barrier()
        dec_s, hpre_s, hdec_s = reduce_max([r["decode_s"], r["host_prefill_s"], r["host_decode_s"]])
        step_s = dec_s / (2 * N_DECODE[key])
        bytes_gpu = r["bytes_per_step"] / world + (1 - 1 / world) * c["hidden_size"] * c["vocab_size"] * 18 / 32   # the head is replicated
        out[name] = {"value": r["decode_tokens"] / dec_s, "unit": "tok/s", "us_per_step": step_s * 1e6,
                     "prefill_tok_s": r["prefill_tokens"] / hpre_s, "e2e_tok_s": r["decode_tokens"] / hdec_s,
                     "roofline": {"bound": "hbm", "achieved": bytes_gpu / step_s / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s per GPU",
                                  "frac": bytes_gpu / step_s / 1e9 / peaks["hbm_gbs"], "bytes_per_launch": bytes_gpu, "traffic": None}}
    m.close()
    if repeat:
        out["weights"] = "layer 0 drawn from the seed, its bytes repeated for the other layers"
    # the library collective on the sizes the sums have (torch's NCCL, the same library): one all-reduce of [8, 4096] f32
    x = torch.zeros(8 * c["hidden_size"], device="cuda")
    for _ in range(10):
        dist.all_reduce(x)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(100):
        dist.all_reduce(x)
    e1.record()
    torch.cuda.synchronize()
    out["nccl_allreduce_us_128KiB"] = reduce_max([e0.elapsed_time(e1) * 10.0])[0]
    out["sums_per_step"] = 2 * c["num_layers"]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="forge", choices=["forge", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side-configs", action="store_true", help="one GPU: only the headline workload")
    ap.add_argument("--no-tp", action="store_true", help="N GPUs: only the request-sharded headline")
    ap.add_argument("--prompt-tokens", type=int, default=None, help="override the headline prompt length (profiling / experiments)")
    ap.add_argument("--decode-steps", type=int, default=None, help="override the headline number of decode steps")
    ap.add_argument("--profile", action="store_true", help="short run for ncu: no side configurations, no CPU baseline; prints a non-benchmark line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    key = "c2" if world == 1 else "c3"
    if args.prompt_tokens:
        N_PROMPT[key] = args.prompt_tokens
    if args.decode_steps:
        N_DECODE[key] = args.decode_steps
    from forge_llm_b200._lib import lib
    if lib.forge_device_count() == 0:
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference for the CPU path)")
    if world != args.gpus and world > 1:
        print(f"bench.py: WORLD_SIZE={world} but --gpus {args.gpus}; using WORLD_SIZE", file=sys.stderr)
    if args.gpus > 1 and world == 1:
        raise SystemExit("bench.py: launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    if world == 1:
        run_single(args, local_rank)
    else:
        run_multi(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
