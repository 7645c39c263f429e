#!/usr/bin/env python
"""Benchmark of the batch-1 decode step (tokens/s and fraction of the HBM roofline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one decoded token: forward(token, pos) + fused sampler.  At N=1 the workload is the
Llama-3.2-1B shape (FP16 weights, 128K vocabulary, temperature 0.8, repetition penalty 1.1, 32-token
prompt); for N>1 it is the Llama-3-8B shape tensor-parallel over the N GPUs (one rank per GPU,
all-reduce after o_proj and down_proj).  Weights are seeded random-init tensors of those shapes.
Rank 0 prints ONE JSON line.

--impl reference times the reference's own CPU implementation of the same step (the compiled,
unmodified reference under oracle/_ref when present, else the plain-C port) on the host cores.
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

WORKLOADS = {
    # name: (shape, prompt tokens, temperature, penalty)
    "llama-3.2-1b": ("llama-3.2-1b", 32, 0.8, 1.1),
    "tinyllama-1.1b": ("tinyllama-1.1b", 32, 0.8, 1.1),
    "llama-3-8b": ("llama-3-8b", 64, 0.8, 1.1),
    "stories15m": ("stories15m", 16, 1.0, 1.0),
    # long context: K/V cache pre-filled with 32768 positions of seeded N(0,1) values, then prompt + decode
    "llama-3-8b-32k": ("llama-3-8b-32k", 64, 0.8, 1.1, 32768),
}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU while the timed region runs.

    Read through NVML in a thread of this process (the same counters nvidia-smi prints; a sample every 5 ms from the
    first millisecond on, which matters on an 8-GPU box where an nvidia-smi child needs longer to start than a 90 ms
    timed region lasts); falls back to an nvidia-smi child when the NVML binding is missing.  Nothing is set."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.rows, self.proc, self.index, self.nvml, self.stop, self.source = [], None, index, None, False, None

    def _nvml_loop(self):
        n = self.nvml
        try:
            h = n.nvmlDeviceGetHandleByIndex(self.index)
            mx = float(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM))
            get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop:
                mask = int(get_reasons(h))
                self.rows.append([str(float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM))), str(mx),
                                  str(n.nvmlDeviceGetPowerUsage(h) / 1000.0)] +
                                 ["Active" if mask & bit else "Not Active" for bit in (0x8, 0x40, 0x20, 0x4)])
                time.sleep(0.005)
        except Exception:
            pass

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml, self.source = pynvml, "nvml"
            self.t = threading.Thread(target=self._nvml_loop, daemon=True)
            self.t.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", os.environ.get("LPP_BENCH_LMS", "25")],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.nvml:
            self.stop = True
            self.t.join(timeout=2)
        elif self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        busy = [x for x in sm if x > 0.5 * max(sm)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(sm), "power_w_max": max(float(r[2]) for r in self.rows if len(r) >= 7), "source": self.source}


def gen_device_weights(cfg, dtype, tied, seed, layers=None):
    """Seeded random-init tensors on the current CUDA device: N(0, 0.02) matrices, unit norms."""
    import torch
    from lighterpp_b200.formats import tensor_shapes
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    tdt = torch.float16 if dtype == "f16" else torch.float32
    for name, shape in tensor_shapes(cfg, tied).items():
        stacked = len(shape) == 3 or name in ("rms_att", "rms_ffn")
        for l in (range(cfg.n_layers) if stacked else [-1]):
            shp = shape[1:] if stacked else shape
            if name.startswith("rms"):
                t = torch.ones(shp, device="cuda")
            else:
                t = (torch.randn(shp, device="cuda", generator=g) * 0.02).to(tdt)
            yield name, l, t


CHECK_TOKENS = (11, 4242)  # tp_check: two steps at positions 0 and 1 (they depend on no earlier cache content)


def check_logits(eng):
    return [eng.step_logits(t, pos) for pos, t in enumerate(CHECK_TOKENS)]


def tp1_same_workload(args, cfg, dtype, tied, seed, local, n_prompt, temp, pen, tp_logits=None):
    """tok/s of the N>1 workload on one GPU: same prompt handling, a shorter timed region.  With tp_logits (the
    tensor-parallel engine's logits of the two check steps) it also reports how far they are from this engine's."""
    import torch
    from lighterpp_b200 import engine as E, synth
    steps = max(16, min(args.steps, 64))
    eng = E.Engine(cfg, dtype, "f16" if dtype == "f16" else "f32", device=local, flags=args.flags & ~E.FLAG_TP_NCCL,
                   ring_kb=args.ring_kb)
    for name, l, t in gen_device_weights(cfg, dtype, tied, seed):
        eng.upload(name, t, max(l, 0))
    eng.finalize()
    torch.cuda.empty_cache()
    prompt = synth.prompt_tokens(cfg.vocab_size, n_prompt, seed)
    rs = np.random.default_rng(seed).random(8 + steps).astype(np.float32)
    hist = [int(t) for t in prompt][-64:]
    eng.prefill(prompt[:-1], 0)
    tok, pos = int(prompt[-1]), n_prompt - 1
    out, _ = eng.decode(tok, pos, 8, temp, pen, hist, 64, rs[:8])
    hist = (hist + [int(x) for x in out])[-64:]
    tok, pos = int(out[-1]), pos + 8
    torch.cuda.synchronize()
    out, dev_ms = eng.decode(tok, pos, steps, temp, pen, hist, 64, rs[8:8 + steps])
    torch.cuda.synchronize()
    bytes_per_step = float(np.mean([eng.step_bytes(p) for p in range(pos, pos + steps)]))
    check = None
    if tp_logits is not None:
        mine = check_logits(eng)
        check = {"max_abs": max(float(np.abs(a - b).max()) for a, b in zip(mine, tp_logits)),
                 "min_cosine": min(float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b))) for a, b in zip(mine, tp_logits))}
    eng.close()
    us = dev_ms * 1e3 / steps
    out = {"value": round(steps / (dev_ms / 1e3), 2), "unit": "tok/s", "n_gpus": 1, "steps": steps,
           "ms_per_step": round(dev_ms / steps, 5), "achieved_gbs": round(bytes_per_step / us / 1e3, 1)}
    return out, check


def run_ours(args, rank, world):
    import torch
    import torch.distributed as dist
    from lighterpp_b200 import engine as E, synth
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    shape, n_prompt, temp, pen, *rest = WORKLOADS[args.workload]
    prefill = rest[0] if rest else 0
    cfg, dtype, tied, seed = synth.SHAPES[shape]
    need = prefill + n_prompt + args.warmup + 2 * args.steps + 8
    if need > cfg.seq_len:
        cfg = type(cfg)(**{**cfg.asdict(), "seq_len": need})
    nccl_id = None
    if world > 1:
        ids = [E.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        nccl_id = ids[0]
    eng = E.Engine(cfg, dtype, "f16" if dtype == "f16" else "f32", device=local, tp_rank=rank, tp_size=world,
                   nccl_id=nccl_id, flags=args.flags, ring_kb=args.ring_kb)
    tp_exchange = "none" if world == 1 else "nccl all-reduce"
    if world > 1 and not (args.flags & E.FLAG_TP_NCCL):
        # the o_proj / down exchange fused into the GEMVs over peer memory: map every rank's receive buffer.
        # If any rank cannot map its peers, every rank stays on the NCCL all-reduce.
        handles = [None] * world
        try:
            mine = eng.tp_export()
        except E.LppError:
            mine = None
        dist.all_gather_object(handles, mine)
        ok = all(h is not None for h in handles)
        if ok:
            try:
                eng.tp_connect(handles)
            except E.LppError:
                ok = False
        oks = [None] * world
        dist.all_gather_object(oks, ok)
        if all(oks):
            tp_exchange = "fused into the GEMVs over peer memory"
        else:
            eng.close()
            ids = [E.nccl_unique_id() if rank == 0 else None]  # a communicator id is good for one group only
            dist.broadcast_object_list(ids, src=0)
            nccl_id = ids[0]
            eng = E.Engine(cfg, dtype, "f16" if dtype == "f16" else "f32", device=local, tp_rank=rank, tp_size=world,
                           nccl_id=nccl_id, flags=args.flags | E.FLAG_TP_NCCL, ring_kb=args.ring_kb)
    # the CPU baseline keeps FP32 host copies of all weights: only for shapes where that is a few GB
    small = cfg.dim * cfg.n_layers <= 2048 * 22
    host_copy = {} if (rank == 0 and world == 1 and not args.no_cpu_baseline and small) else None
    for name, l, t in gen_device_weights(cfg, dtype, tied, seed):
        eng.upload(name, t, max(l, 0))
        if host_copy is not None:
            host_copy.setdefault(name, []).append(t.cpu().numpy())
    eng.finalize()
    torch.cuda.empty_cache()

    prompt = synth.prompt_tokens(cfg.vocab_size, n_prompt, seed)
    rs = np.random.default_rng(seed).random(args.warmup + 2 * args.steps + 8).astype(np.float32)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if prefill:
        g = torch.Generator(device="cuda")
        g.manual_seed(seed + 1000)
        for l in range(cfg.n_layers):  # every rank draws the same full-head tensors and keeps its heads
            k = torch.randn((cfg.n_kv_heads, prefill, cfg.head_size), device="cuda", generator=g).half()
            v = torch.randn((cfg.n_kv_heads, prefill, cfg.head_size), device="cuda", generator=g).half()
            eng.kv_prefill(l, k, v, prefill)
        del k, v
    # prompt: one batched pass over the weights (lpp_prefill) on a single GPU with FP16 weights; token by token through
    # the step, as the reference does (src/main.cpp:163-179), on the engines that have no batched path.  Untimed
    # here; the line reports both ways of feeding the same prompt.
    hist = [int(t) for t in prompt][-64:]
    prompt_ms = eng.prefill(prompt[:-1], prefill)
    tok, pos = int(prompt[-1]), prefill + n_prompt - 1
    # the clock sampler starts before the warm-up: nvidia-smi needs a moment to come up, and the short timed region
    # of the larger rank counts would otherwise pass between two samples (idle samples are filtered out)
    with ClockSampler(local) as clk:
        # warm-up (untimed), device-resident loop
        if args.warmup > 0:
            out, _ = eng.decode(tok, pos, args.warmup, temp, pen, hist, 64, rs[:args.warmup])
            hist = (hist + [int(x) for x in out])[-64:]
            tok, pos = int(out[-1]), pos + args.warmup
        # ---- timed region 1: K steps, inputs resident in HBM, CUDA events on the engine's stream
        barrier()
        out, dev_ms = eng.decode(tok, pos, args.steps, temp, pen, hist, 64, rs[args.warmup:args.warmup + args.steps])
        barrier()
    ids_equal = None
    if world > 1:  # every rank must have sampled the same tokens
        all_ids = [None] * world
        dist.all_gather_object(all_ids, [int(x) for x in out])
        ids_equal = all(a == all_ids[0] for a in all_ids)
    t_dev = torch.tensor([dev_ms], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_dev, op=dist.ReduceOp.MAX)
    dev_ms = float(t_dev.item())
    mean_bytes = float(np.mean([eng.step_bytes(p) for p in range(pos, pos + args.steps)]))
    hist = (hist + [int(x) for x in out])[-64:]
    tok, pos = int(out[-1]), pos + args.steps
    # ---- timed region 2 (e2e): the forward(token,pos) call with host buffers, one call per token
    r2 = rs[args.warmup + args.steps:]
    for i in range(min(3, args.warmup)):
        eng.forward(tok, pos, temp, pen, hist, float(r2[-1 - i]))  # same position: warms the host path only
    barrier()
    t0 = time.perf_counter()
    h2d = d2h = 0
    for i in range(args.steps):
        tok = eng.forward(tok, pos, temp, pen, hist, float(r2[i]))
        h2d += 48 + 4 * len(hist)
        d2h += 8
        hist = (hist + [tok])[-64:]
        pos += 1
    barrier()
    e2e_s = time.perf_counter() - t0
    t_e2e = torch.tensor([e2e_s], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    e2e_s = float(t_e2e.item())

    # ---- per-kernel durations (CUDA events inside a replayed graph) for the roofline object
    prof = eng.profile_step(pos - args.steps // 2, 10, temp, pen)
    gemv_kinds = {k: v for k, v in prof.items() if (k.endswith("gemv") or k == "step_kernel") and v["launches"]}
    dom = max(gemv_kinds, key=lambda k: gemv_kinds[k]["bytes"])  # the kernel family that moves most bytes per step
    try:
        # its launches of one step back to back, launched as the step launches them, one event pair around
        dom_run = eng.profile_kind(pos - args.steps // 2, dom, 10)
    except Exception:
        dom_run = None
    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        us = dev_ms * 1e3 / args.steps
        d = gemv_kinds[dom]
        per_launch_bytes = d["bytes"] / d["launches"]
        isolated_us = d["ms"] * 1e3 / d["launches"]
        per_launch_us = dom_run["ms_per_launch"] * 1e3 if dom_run and dom_run["launches"] else isolated_us
        achieved = per_launch_bytes / per_launch_us / 1e3
        step_gbs = mean_bytes / us / 1e3
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
                traffic = json.load(f).get(f"{args.workload}:{dom}")
        except Exception:
            pass
        line = {
            "metric": "batch-1 decode tok/s and % of HBM roofline", "value": round(args.steps / (dev_ms / 1e3), 2),
            "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights, f32 accumulate" if dtype == "f16" else "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "shape": cfg.asdict(), "prefilled_positions": prefill, "prompt_tokens": n_prompt, "temperature": temp,
                       "penalty": pen, "parallelism": f"tp{world}", "tp_exchange": tp_exchange, "positions": [pos - 2 * args.steps, pos - args.steps],
                       "l2": "inputs larger than L2 (every step streams all weights, >> 126 MB)",
                       "timed_with": "CUDA events on the engine stream around K graph launches, max over ranks"},
            "clocks": clk.summary(),
            "e2e": {"value": round(args.steps / e2e_s, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d // args.steps,
                    "d2h_bytes_per_step": d2h // args.steps,
                    "what": "forward(token,pos) through the C ABI per token: host token/history in, sampled id out"},
            "gpu_launches": eng.kernels_per_step * args.steps,
            "step_roofline": {"bytes_per_step": int(mean_bytes), "achieved_gbs": round(step_gbs, 1),
                              "frac_of_measured": round(step_gbs / peak, 4), "frac_of_8tbs": round(step_gbs / 8000.0, 4),
                              "per_gpu": True},
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peak,
                         "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "traffic": traffic, "bytes_per_launch": int(per_launch_bytes),
                         "us_per_launch": round(per_launch_us, 3), "isolated_us_per_launch": round(isolated_us, 3),
                         "timed_with": "one CUDA event pair around the step's launches of this kernel run back to back "
                                       "with the step's launch attributes (each streams its own layer's weights); "
                                       "isolated = event-record nodes around every single launch, no overlap"},
            "kernels": {k: {"us_per_launch": round(v["ms"] * 1e3 / v["launches"], 3), "launches": v["launches"],
                            "gbs": round(v["bytes"] / v["ms"] / 1e6, 1) if v["ms"] else None}
                        for k, v in prof.items() if v["launches"]},
        }
    prompt_info = None
    if world == 1 and not prefill:
        # the prompt again, both ways, on the finished engine (its cache rows are simply rewritten)
        loop_ms = 0.0
        batched = min(eng.prefill(prompt[:-1], 0) for _ in range(3))
        t0 = time.perf_counter()
        for i, t in enumerate(prompt[:-1]):
            eng.step_logits(int(t), i)
        loop_ms = (time.perf_counter() - t0) * 1e3
        prompt_info = {"tokens": int(len(prompt) - 1), "batched_ms": round(batched, 3),
                       "batched_tok_s": round((len(prompt) - 1) / batched * 1e3, 1),
                       "token_by_token_ms": round(loop_ms, 3),
                       "token_by_token_tok_s": round((len(prompt) - 1) / loop_ms * 1e3, 1),
                       "what": "lpp_prefill (device time) against one lpp_step_logits call per prompt token (host time)"}
    tp_logits = check_logits(eng) if world > 1 else None  # outside every timed region; all ranks take part
    if line is not None and prompt_info is not None:
        line["prompt"] = prompt_info
    eng.close()
    if world > 1 and not args.no_tp1:
        # the same workload on ONE GPU (rank 0 alone, the other ranks wait): the number the sharded run is a
        # speed-up over (N=1 of the default run is a different, smaller shape), and the engine the sharded
        # logits are checked against
        torch.cuda.empty_cache()
        if rank == 0:
            try:
                one, check = tp1_same_workload(args, cfg, dtype, tied, seed, local, n_prompt, temp, pen, tp_logits)
                line["tp1_same_workload"] = one
                if prefill:
                    one["note"] = "this one-GPU run has no pre-filled cache: it serves the logits check only"
                if not prefill:  # the one-GPU run has no pre-filled cache: its positions are not the same work
                    line["scaling_vs_tp1"] = {"speedup": round(line["value"] / one["value"], 3),
                                              "efficiency": round(line["value"] / one["value"] / world, 3)}
                line["tp_check"] = {**check, "sampled_ids_equal_on_all_ranks": ids_equal,
                                    "what": "logits of two steps (positions 0, 1) against the same engine on one GPU; "
                                            "bar: max-abs 2e-2, cosine 0.9999"}
            except Exception as ex:  # e.g. a shape that does not fit one GPU
                line["tp1_same_workload"] = {"unavailable": str(ex)[:200]}
        dist.barrier()
    if rank == 0 and host_copy is not None:
        W = {k: (np.stack(v) if len(v) > 1 or k in ("rms_att", "rms_ffn", "wq") else v[0]) for k, v in host_copy.items()}
        line["cpu_baseline"] = cpu_baseline(cfg, W, prompt, temp, pen, budget_s=args.cpu_seconds)
    return line


def cpu_baseline(cfg, W, prompt, temp, pen, budget_s=20.0):
    """Times the reference CPU path on a bounded sample of the same workload (first tokens of the prompt)."""
    from oracle import oracle as O
    Wf = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in W.items()}
    cores = os.cpu_count()
    if O.have_reference():
        m = O.Reference().model(cfg, Wf)
        kind, threads = "reference", 1
        t1 = m.time_steps(prompt[:1], 0, temp, pen)
        n = int(max(2, min(len(prompt) - 1, budget_s / max(t1, 1e-6))))
        t = m.time_steps(prompt[1:1 + n], 1, temp, pen, prompt[:1])
    else:
        orc = O.Oracle()
        m = orc.model(cfg, Wf)
        kind, threads = "port", cores
        t0 = time.perf_counter()
        m.step_logits(int(prompt[0]), 0)
        t1 = time.perf_counter() - t0
        n = int(max(2, min(len(prompt) - 1, budget_s / max(t1, 1e-6))))
        t0 = time.perf_counter()
        for i in range(n):
            lg = m.step_logits(int(prompt[1 + i]), 1 + i)
            orc.sample(lg, temp, pen, prompt[:1], 0.5)
        t = time.perf_counter() - t0
    return {"value": round(n / t, 4), "unit": "tok/s", "cores": threads, "host_cores": cores, "kind": kind,
            "sample": f"{n} teacher-forced steps at positions 1..{n} of the same model (FP32 copies of the same weights)"}


def run_reference(args, rank, world):
    """The reference's own CPU implementation of the step on the host cores (rank 0 only)."""
    if rank != 0:
        return None
    from lighterpp_b200 import synth
    shape, n_prompt, temp, pen = WORKLOADS[args.workload][:4]
    cfg, dtype, tied, seed = synth.SHAPES[shape]
    small = type(cfg)(**{**cfg.asdict(), "seq_len": 256})
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.set_device(0)
            W = {}
            for name, l, t in gen_device_weights(small, dtype, tied, seed):
                W.setdefault(name, []).append(t.float().cpu().numpy())
            W = {k: (np.stack(v) if len(v) > 1 or k in ("rms_att", "rms_ffn", "wq") else v[0]) for k, v in W.items()}
        else:
            raise RuntimeError
    except Exception:
        W = synth.as_f32(synth.gen_model(small, seed, dtype, tied))
    prompt = synth.prompt_tokens(cfg.vocab_size, n_prompt, seed)
    cb = cpu_baseline(small, W, prompt, temp, pen, budget_s=args.cpu_seconds)
    n = int(cb["sample"].split()[0])
    return {"impl": "reference", "metric": "batch-1 decode tok/s and % of HBM roofline", "value": cb["value"],
            "unit": "tok/s", "n_gpus": world, "steps": n, "warmup": 1, "ms_per_step": round(1e3 / cb["value"], 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "shape": cfg.asdict(), "parallelism": "cpu"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--flags", type=int, default=0)
    ap.add_argument("--ring-kb", type=int, default=0)
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp1", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus and world == 1 and args.gpus > 1:
        print(json.dumps({"error": f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks"}))
        sys.exit(2)
    if args.workload is None:
        args.workload = "llama-3.2-1b" if world == 1 else "llama-3-8b"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if world > 1 and args.impl == "ours":
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")
    line = run_reference(args, rank, world) if args.impl == "reference" else run_ours(args, rank, world)
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    if world > 1 and args.impl == "ours":
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
