#!/usr/bin/env python
"""Benchmark of the quantized forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config c2]

Workload (N = 1): the Llama-3.2-1B-shaped Q4_0 decoder of the benchmark definition — one
"step" is one request: a 1501-token uniform-random prompt through the batched prefill path,
then 128 greedy decode steps at batch 1, fp16 paged KV cache.  Weights are synthetic
(N(0, 0.02), seed 0, quantised to GGUF Q4_0); there is no network for checkpoints.

Reported metric: decode tok/s (the prefill tok/s of the same requests rides along under
"prefill").  `value` is device time (CUDA events on the library's stream, tokens resident on
the GPU); `e2e` is the same loop timed on the host around the C-ABI calls with host buffers
in and out.  With N > 1 (torchrun, one rank per GPU) every rank serves its own copy of the
request stream — independent requests, no collective on the data path — and the aggregate
is N * tokens / max-over-ranks time ("weak" scaling).

`--impl reference` times the reference's CPU path instead: the C++ oracle (a port of the
generated x86 code; the Rust original cannot be built here) on all host cores, each step a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
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

N_PROMPT = {"c1": 100, "c2": 1501, "c3": 2501, "c4": 3001, "c5": 2048}
N_DECODE = {"c1": 64, "c2": 128, "c3": 64, "c4": 256, "c5": 128}


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


def make_model_inputs(cfg_key: str):
    from forge_llm_b200 import configs, synth
    c = configs.CONFIGS[cfg_key]
    blob = synth.make_weights_bin(c, seed=0)
    toks = synth.prompt_tokens(c, N_PROMPT[cfg_key], seed=1)
    return c, blob, toks


# ---------------------------------------------------------------------------- CPU reference arm
def time_oracle(c, blob, toks, n_prefill: int, n_decode: int, repeats: int):
    """Scalar port of the reference's x86 path (kind "port"), all host threads.  One repeat =
    a batched prefill of `n_prefill` prompt tokens followed by `n_decode` greedy steps."""
    from oracle import oracle as O
    m = O.OracleModel(c, blob, kv_mode=O.KV_INT8, fast=False)
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
    c, blob, toks = make_model_inputs(args.config)
    n_pre, n_dec = 16, 2
    sample = f"{n_pre}-token batched prefill + {n_dec} greedy decode steps per step, int8 KV, scalar x86 loops"
    for _ in range(args.warmup):
        time_oracle(c, blob, toks, n_pre, n_dec, 1)
    t0 = time.perf_counter()
    pre, dec, threads = time_oracle(c, blob, toks, n_pre, n_dec, args.steps)
    wall = time.perf_counter() - t0
    line = {
        "impl": "reference", "metric": "decode_tok_s", "value": dec, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * wall / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype_name(c), "data": "synthetic",
        "config": workload_config(args.config, c),
        "prefill": {"value": pre, "unit": "tok/s"},
        "cpu_baseline": {"value": dec, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": dec, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def dtype_name(c: dict) -> str:
    return f"f32 x (int{c['quant']} * f16 block scale), f32 accumulate"


def workload_config(key: str, c: dict) -> dict:
    return {"workload": f"{c['name']}: {N_PROMPT[key]}-token prompt (batched prefill) + {N_DECODE[key]} greedy decode steps, batch 1",
            "config_key": key, "quant": "Q4_0" if c["quant"] == 4 else "Q8_0", "kv_cache": "fp16 paged (64 positions per page)",
            "prompt_tokens": N_PROMPT[key], "decode_steps": N_DECODE[key], "parallelism": "request-sharded (one model replica per GPU)",
            "l2": "inputs larger than L2: every step streams the whole weight set (>= 143 MB) once per token"}


# DRAM bytes moved per algorithmic byte of the streaming GEMV (dram__bytes_read + dram__bytes_write of one captured
# launch, 153.6 MB for 147.75 MB of weights; the capture is summarised under profiles/).  A decode step is one graph
# replay of such kernels; its traffic is scaled from that capture by the bytes it streams.
DRAM_TRAFFIC_RATIO = 1.04
TRAFFIC_NOTE = "scaled from one ncu capture of the GEMV kernel (traffic/algorithmic = 1.04)"


# ---------------------------------------------------------------------------- GPU arm
def run_gpu(args, rank: int, world: int, local_rank: int):
    import torch
    from forge_llm_b200 import configs, runtime
    from forge_llm_b200._lib import lib

    if lib.forge_device_count() == 0:
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback (use --impl reference for the CPU path)")
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    c, blob, toks = make_model_inputs(args.config)
    n_prompt, n_dec = N_PROMPT[args.config], N_DECODE[args.config]
    tp = args.tp and world > 1
    if tp:
        # one model cut over all ranks: rank 0's rendezvous id reaches the others through the process group
        uid = torch.from_numpy(runtime.Model.tp_unique_id() if rank == 0 else np.zeros(runtime.TP_ID_BYTES, np.uint8)).cuda()
        dist.broadcast(uid, 0)
        model = runtime.Model(c, blob, device=local_rank, tp_rank=rank, tp_world=world)
        model.tp_init(uid.cpu().numpy())
        if not args.tp_nccl_only:  # decode sums over peer memory (NVLink stores from the GEMV epilogue)
            mine_h = torch.from_numpy(model.tp_exchange_handle()).cuda()
            all_h = [torch.empty_like(mine_h) for _ in range(world)]
            dist.all_gather(all_h, mine_h)
            model.tp_exchange_attach(torch.cat(all_h).cpu().numpy())
            dist.barrier()
    else:
        model = runtime.Model(c, blob, device=local_rank)
    jobs = 1 if tp else world  # independent requests in flight
    kv = model.new_cache(max_seq=n_prompt + n_dec + 8)
    pinned_prompt = torch.from_numpy(toks.astype(np.int32)).pin_memory()  # H2D source of every step
    prompt_np = pinned_prompt.numpy().view(np.uint32)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(timed: bool):
        """One request through the public API.  Returns device and host timings."""
        kv.reset()
        h0 = time.perf_counter()
        out = model.generate_greedy(prompt_np, n_dec, kv)  # host prompt in, host ids out
        h1 = time.perf_counter()
        pre_ms, dec_ms, launches = model.last_timing()
        return pre_ms, dec_ms, launches, h1 - h0, out

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
        one_step(False)
        if not args.profile:
            one_step_e2e()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    t0 = time.time()
    w0 = time.perf_counter()
    pre_ms, dec_ms, launches, ids0 = [], [], 0, None
    for _ in range(args.steps):
        p, d, l, _, ids = one_step(True)
        pre_ms.append(p)
        dec_ms.append(d)
        launches += l
        ids0 = ids
    barrier()
    w1 = time.perf_counter()
    e2e_pre, e2e_dec = [], []
    for _ in range(args.steps):
        a, b, ids_e = one_step_e2e()
        e2e_pre.append(a)
        e2e_dec.append(b)
    barrier()
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if sampler else None
    assert np.array_equal(ids_e[:, 0], ids0), "device-side and host-side greedy loops disagree"

    # max over ranks of the summed device times
    tot = torch.tensor([sum(dec_ms), sum(pre_ms), sum(e2e_dec), sum(e2e_pre), w1 - w0], dtype=torch.float64, device="cuda")
    cnt = torch.tensor([float(launches)], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
        dist.all_reduce(cnt, op=dist.ReduceOp.SUM)
    dec_s, pre_s, e2e_dec_s, e2e_pre_s, wall = (tot[0].item() / 1e3, tot[1].item() / 1e3, tot[2].item(), tot[3].item(), tot[4].item())
    K = args.steps

    if rank == 0:
        peaks = load_peaks()
        ctx_mid = n_prompt + n_dec // 2
        bytes_tok = configs.decode_bytes_per_token(c, ctx_mid)
        step_s = dec_s / (K * n_dec)                       # one decode step on one GPU
        achieved = bytes_tok / step_s / 1e9
        flops = configs.prefill_flops(c, n_prompt)
        pre_tf = flops / (pre_s / K) / 1e12
        line = {
            "metric": "decode_tok_s", "value": jobs * K * n_dec / dec_s, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": n_warm, "ms_per_step": 1e3 * wall / K, "higher_is_better": True, "scaling": "strong" if tp else "weak",
            "vs_baseline": None, "dtype": dtype_name(c), "data": "synthetic",
            "config": dict(workload_config(args.config, c), **({"parallelism": f"tensor-parallel over {world} GPUs (sum after O and down: " + ("NCCL all-reduce" if args.tp_nccl_only else "NCCL in prefill, peer-memory stores fused into the GEMV in decode") + ")"} if tp else {})),
            "prefill": {"value": jobs * K * n_prompt / pre_s, "unit": "tok/s", "gemm": "tcgen05/TMEM, fp16 hi/lo split, 3 tensor-core passes",
                        "roofline": {"bound": "tensor", "achieved": pre_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                     "frac": pre_tf / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"],
                                     "flops_per_step": flops}},
            "roofline": {"bound": "hbm", "kernel": "one decode step (all kernels of forward(), replayed as one CUDA graph)",
                         "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "traffic": bytes_tok * DRAM_TRAFFIC_RATIO, "traffic_source": TRAFFIC_NOTE,
                         "peak_source": peaks["source"], "bytes_per_launch": bytes_tok, "ctx": ctx_mid,
                         "us_per_launch": step_s * 1e6},
            "e2e": {"value": jobs * K * n_dec / e2e_dec_s, "unit": "tok/s", "h2d_bytes_per_step": int(prompt_np.nbytes + 4),
                    "d2h_bytes_per_step": int(c["vocab_size"] * 4 + n_dec * 4), "prefill_tok_s": jobs * K * n_prompt / e2e_pre_s},
            "gpu_launches": int(cnt.item()),
            "clocks": clocks,
        }
        if args.profile:
            line["note"] = "profiling run (--profile): not a benchmark value"
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            pre, dec, threads = time_oracle(c, blob, toks, 16, 2, 2)
            line["cpu_baseline"] = {"value": dec, "unit": "tok/s", "cores": threads, "kind": "port", "prefill_tok_s": pre,
                                    "sample": "16-token batched prefill + 2 greedy decode steps, median of 2, int8 KV, scalar x86 loops"}
        print(json.dumps(line), flush=True)
    kv.close()
    model.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="forge", choices=["forge", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(N_PROMPT))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prompt-tokens", type=int, default=None, help="override the prompt length (profiling / experiments)")
    ap.add_argument("--decode-steps", type=int, default=None, help="override the number of decode steps")
    ap.add_argument("--tp", action="store_true", help="N > 1: cut ONE model over the N GPUs (tensor parallel, strong scaling) instead of N replicas")
    ap.add_argument("--tp-nccl-only", action="store_true", help="with --tp: keep the library all-reduce in the decode step (no peer-memory sums)")
    ap.add_argument("--profile", action="store_true", help="short run for ncu: one warm-up, no CPU baseline; prints a non-benchmark line")
    args = ap.parse_args()
    if args.prompt_tokens:
        N_PROMPT[args.config] = args.prompt_tokens
    if args.decode_steps:
        N_DECODE[args.config] = args.decode_steps
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world > 1:
        print(f"bench.py: WORLD_SIZE={world} but --gpus {args.gpus}; using WORLD_SIZE", file=sys.stderr)
    if args.gpus > 1 and world == 1:
        raise SystemExit("bench.py: launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
