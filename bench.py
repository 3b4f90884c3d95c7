#!/usr/bin/env python
"""Headline benchmark: HYDRA-250M bf16 inference prefill throughput (tokens/s) on N B200s of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU arm: the reference's own HydraModel.forward on the host cores
                                              # (from oracle/_ref; the CPU restatement when that is absent)

Workload (the HYDRA-250M prefill benchmark configuration): dim 1024, 10 MoR blocks x 4 recursions, CCGQA 4x compression with 8 query /
2 KV heads (head_dim 32), SwiGLU hidden 2816, MoD top-k at 75% capacity in the interior blocks, vocab 50257, tied
output projection; batch 32 x 2048 synthetic token ids PER GPU (weak scaling: every rank is a full replica working
on its own sequences; sequences never cross GPUs and there is no collective inside the timed region).  Weights are
seeded random-init with the reference's distributions (no checkpoint or dataset is involved).

One step = one full forward (embedding -> 10 blocks -> final norm -> all 65536 x 50257 logits).
  value  tokens/s with the ids already resident in HBM (CUDA events, max over ranks)
  e2e    the same through the public call HydraB200Model.prefill(): pinned host ids -> device, forward,
         last-position logits -> host, copies inside the timed region
  roofline  the dominant kernel (tcgen05 gate_up GEMM with the SwiGLU epilogue): FLOPs actually routed to it
            divided by its summed launch time, measured with CUDA events recorded by the executor around every
            launch in a second pass of the same K steps right after the timed one (the recorder costs ~0.7 ms
            per step, so the timed pass runs without it; `breakdown_pass` carries that pass's own step time)
  parity    outside the timed region: sequence 0 of the batch that was timed against the CPU oracle with the GPU's
            routing replayed (sequences are independent bit for bit, so one speaks for the batch)
  ccgqa_block  outside the timed region: the CCGQA-block microbenchmark (8 x 2048 x 1024) and its fused pre-attention
            kernel against their rooflines - the second half of the headline metric
  library_baseline  outside the timed region: the library calls the reference makes on a GPU (cuBLAS F.linear, SDPA,
            cuDNN Conv1d, its bf16 eager model) timed on this GPU beside this package's kernels at the same shapes
  strong    N > 1 only: the same model on a global batch of 32 sequences split over the ranks
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import threading
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "hydra_250m_prefill_tokens_per_s"
ARCH = dict(vocab_size=50257, dim=1024, n_mor_blocks=10, recursions_per_block=4, n_heads=8, n_kv_heads=2,
            compression_factor=4, mlp_ratio=2.67, mod_capacity=0.75)
SEQ = 2048
SEED = 0


def workload_config(batch_per_gpu: int, n_gpus: int) -> dict:
    return {
        "workload": "configs[3]: HYDRA-250M prefill, dim 1024, 10 MoR blocks x 4 recursions, CCGQA 8q/2kv "
                    "(head_dim 32), SwiGLU 2816, MoD top-k 0.75, vocab 50257, all logits computed",
        "batch_per_gpu": batch_per_gpu, "global_batch": batch_per_gpu * n_gpus, "seq_len": SEQ,
        "parallelism": f"replica-per-GPU x{n_gpus}, batch sharded by sequence, no data-path collective",
        "weights": f"seeded random-init (seed {SEED}), reference init distributions",
        "l2": "working set (weights 0.3 GB + activations > 1 GB + logits 6.6 GB) far exceeds the 126 MB L2; no flush needed",
    }


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled while the timed region runs: NVML read every 10 ms from a thread (reads
    only; nothing is set), or, when NVML cannot be opened, an nvidia-smi loop at its 200 ms period."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.proc, self.thread, self.samples, self.reason_mask, self.smax = None, None, [], 0, None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                pr = torch.cuda.get_device_properties(index)
                bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
                h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.reason_mask |= int(reasons(h))
                    except Exception:
                        pass
                    self._stop.wait(0.01)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            sm = self.samples
            reasons = sorted(n for n, bit in self.REASON_BITS.items() if self.reason_mask & bit)
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.smax, "reasons": reasons,
                    "samples": len(sm), "source": "nvml, 10 ms period"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); smax.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi, 200 ms period"}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_forward_tokens_per_s(n_seq: int, steps: int, warmup: int, state_dict=None) -> tuple[float, float, int]:
    """The oracle port of the reference's eager fp32 forward, all host threads; returns (tok/s, s/step, threads)."""
    from oracle import hydra_oracle as O
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    cfg = O.HydraConfig(vocab_size=ARCH["vocab_size"], dim=ARCH["dim"], n_mor_blocks=ARCH["n_mor_blocks"],
                        recursions_per_block=ARCH["recursions_per_block"], n_heads=ARCH["n_heads"],
                        n_kv_heads=ARCH["n_kv_heads"], max_seq_len=SEQ, mod_capacity=ARCH["mod_capacity"])
    w = O.init_params(cfg, seed=SEED) if state_dict is None else {k: v.float().cpu() for k, v in state_dict.items()}
    ids = torch.randint(0, ARCH["vocab_size"], (n_seq, SEQ), generator=torch.Generator().manual_seed(SEED))
    with torch.no_grad():
        for _ in range(warmup):
            O.model_forward(ids, w, cfg)
        t0 = time.perf_counter()
        for _ in range(steps):
            O.model_forward(ids, w, cfg)
        dt = (time.perf_counter() - t0) / max(1, steps)
    return n_seq * SEQ / dt, dt, threads


REF_ARGS = dict(vocab_size=ARCH["vocab_size"], dim=ARCH["dim"], n_mor_blocks=ARCH["n_mor_blocks"],
                recursions_per_block=ARCH["recursions_per_block"], n_heads=ARCH["n_heads"], n_kv_heads=ARCH["n_kv_heads"],
                compression_factor=ARCH["compression_factor"], max_seq_len=SEQ, mod_capacity=ARCH["mod_capacity"])


def reference_available() -> bool:
    from oracle import build_ref
    return build_ref.add_ref_to_path()


def reference_forward_tokens_per_s(n_seq: int, steps: int, warmup: int) -> tuple[float, float, int]:
    """The reference's own eager fp32 HydraModel.forward (hydra/model/framework/model.py:408-506; the unmodified package
    under oracle/_ref) on the host, all host threads; seeded random-init weights of the benchmarked architecture
    (its own initialiser).  Returns (tok/s, s/step, threads)."""
    from oracle import build_ref
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    model = build_ref.reference_model(seed=SEED, **REF_ARGS)
    ids = torch.randint(0, ARCH["vocab_size"], (n_seq, SEQ), generator=torch.Generator().manual_seed(SEED))
    for _ in range(warmup):
        build_ref.reference_forward(model, ids)
    t0 = time.perf_counter()
    for _ in range(steps):
        build_ref.reference_forward(model, ids)
    dt = (time.perf_counter() - t0) / max(1, steps)
    return n_seq * SEQ / dt, dt, threads


def cpu_arm(n_seq: int, steps: int, warmup: int, state_dict=None) -> dict:
    """cpu_baseline record: the reference itself when oracle/_ref is there, else the CPU restatement (labelled)."""
    if reference_available():
        tps, dt, threads = reference_forward_tokens_per_s(n_seq, steps, warmup)
        kind, what = "reference", "the reference's own HydraModel.forward, eager fp32 (unmodified package, oracle/_ref)"
    else:
        tps, dt, threads = cpu_forward_tokens_per_s(n_seq, steps, warmup, state_dict)
        kind, what = "port", "CPU restatement of the reference's eager fp32 forward (oracle/_ref has not been built)"
    return {"value": tps, "unit": "tok/s", "cores": threads, "kind": kind, "s_per_step": dt,
            "sample": f"{n_seq} sequence x {SEQ} tokens of the same workload per step, {steps} timed step(s) after "
                      f"{warmup} warm-up; {what}"}


def cpu_generation_baseline(blocks: int, prompt: int) -> dict:
    """What the reference does to generate one token (its helper re-runs the whole forward on the sequence so far,
    diagnostics/eval_checkpoint.py:127-160), timed with the oracle port on the host cores at the 1.5B shape:
    one eval forward of one sequence of `prompt` tokens, and one cached step of the oracle's own decode for comparison."""
    from oracle import hydra_oracle as O
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    cfg = O.HydraConfig(vocab_size=50257, dim=2048, n_mor_blocks=blocks, recursions_per_block=4, n_heads=32, n_kv_heads=4,
                        max_seq_len=prompt + 8, mod_capacity=0.75)
    w = O.init_params(cfg, seed=SEED)
    ids = torch.randint(0, 50257, (1, prompt), generator=torch.Generator().manual_seed(SEED))
    with torch.no_grad():
        t0 = time.perf_counter()
        logits, cache = O.cached_prefill(ids, w, cfg)
        t_forward = time.perf_counter() - t0
        nxt = logits[:, -1].argmax(-1)
        t0 = time.perf_counter()
        O.cached_decode_step(nxt, w, cfg, cache)
        t_step = time.perf_counter() - t0
    return {"value": 1.0 / t_forward, "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"1 sequence, {blocks} blocks: one eval forward of {prompt} tokens = the reference's cost of one generated "
                      f"token ({t_forward:.2f} s); one cached step of the CPU port: {t_step * 1e3:.0f} ms"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_seq = 1                                   # a bounded sample: one sequence of the workload per step
    warm = min(args.warmup, 1)
    base = cpu_arm(n_seq, args.steps, warm)
    tps, dt = base["value"], base["s_per_step"]
    cfg = workload_config(args.batch, args.gpus)
    cfg["timed_batch"] = n_seq                  # what one step of THIS arm processes (the workload's batch is above)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": getattr(args, "scaling_mode", "weak"),
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": base,
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def routed_flops(records, mlp_rows, T: int) -> dict:
    """FLOPs per kernel kind with the rows each launch really processed (device-counted launches use taps)."""
    fl: dict = {}
    for r in records:
        kd = r["kind"]
        if kd in ("gemm_gate_up", "gemm_down"):
            m = int(mlp_rows[r["block"]][r["rec"]])
        else:
            m = r["m"]
        if kd.startswith("gemm"):
            f = 2.0 * m * r["n"] * r["k"]
        elif kd == "attention":
            f = 4.0 * T * r["n"] * (r["k"] + 1) / 2.0
        else:
            f = 0.0
        fl[kd] = fl.get(kd, 0.0) + f
    return fl


def parity_record(model, ids_dev, timed_logits_seq0, sd) -> dict:
    """Sequence 0 of the batch that was timed, against the CPU oracle with the GPU's own routing replayed; also the
    agreement of the free-running oracle's depth decisions.  Run after the timed region."""
    from oracle import hydra_oracle as O
    solo = model(ids_dev[:1], taps=True)
    tp = model.last_taps
    same = bool(torch.equal(solo[0], timed_logits_seq0))      # sequence alone == the same sequence inside the batch
    w = {k: v.to(torch.bfloat16).float().cpu() for k, v in sd.items()}
    cfg = O.config_from_state_dict(w, n_heads=ARCH["n_heads"], n_kv_heads=ARCH["n_kv_heads"],
                                   mod_capacity=ARCH["mod_capacity"], max_seq_len=SEQ)
    NB, R = cfg.n_mor_blocks, cfg.recursions_per_block
    rt = O.RoutingTaps()
    d = tp.depths.cpu().long().view(NB, 1, SEQ)
    idx = tp.mod_idx.cpu().long()
    for i in range(NB):
        rt.depths.append(d[i])
        for r in range(R):
            rt.mod_indices[(i, r)] = idx[i, r]
    ids_cpu = ids_dev[:1].cpu()
    free = O.RoutingTaps()
    with torch.no_grad():
        ref_free = O.model_forward(ids_cpu, w, cfg, taps=free)
        ref = O.model_forward(ids_cpu, w, cfg, forced=rt)
    lg = solo.float().cpu()
    agree = [float((d[i] == free.depths[i]).float().mean()) for i in range(NB)]
    return {"checked": "sequence 0 of the timed batch vs the CPU oracle, GPU routing replayed",
            "batch_equals_solo_bitwise": same,
            "rel_l2": float((lg - ref).norm() / ref.norm()), "max_abs": float((lg - ref).abs().max()),
            "logit_range": float(ref.abs().max()),
            "free_run_rel_l2": float((lg - ref_free).norm() / ref_free.norm()),
            "depth_agree_min": min(agree), "depth_agree_mean": sum(agree) / len(agree),
            "finite": bool(torch.isfinite(lg).all())}


def ccgqa_block_record(peaks: dict, iters: int = 20) -> dict:
    """The CCGQA-block microbenchmark (B=8, S=2048, dim 1024, 8q/2kv heads of 32, temperature 1.0, Xavier weights from
    seed 1) and its fused pre-attention kernel, timed alone with rotating buffers larger than L2."""
    import microbench
    ns = microbench.argparse_like(batch=8, iters=iters, impl=0)
    blk = microbench.ccgqa_block(ns)
    pre = microbench.pre_attention(ns)
    att = microbench.attention(ns)
    burst, sust, hbm = float(peaks["bf16_tflops"]), float(peaks["bf16_tflops_sustained"]), float(peaks["hbm_gbs"])
    return {"shape": [8, 2048, 1024], "us": blk["ms"] * 1e3, "gflop": blk["algorithmic_flops"] / 1e9,
            "tflops": blk["achieved"], "frac_of_burst": blk["achieved"] / burst, "frac_of_sustained": blk["achieved"] / sust,
            "parts_us": {k: v * 1e3 for k, v in blk["parts_ms"].items()},
            "pre_attention": {"us": pre["ms"] * 1e3, "algorithmic_mb": pre["algorithmic_bytes"] / 1e6,
                              "gbs": pre["achieved"], "frac_of_hbm": pre["achieved"] / hbm,
                              "conv_tflops": pre["conv_tflops"], "conv_frac_of_burst": pre["conv_tflops"] / burst},
            "attention": {"us": att["ms"] * 1e3, "tflops": att["achieved"], "frac_of_burst": att["achieved"] / burst,
                          "exp_floor_us": 8 * 8 * 2048 * (2048 / 2 + 64) / (148 * 16 * 1.965e9) * 1e6,
                          "note": "exp floor = one ex2 per score at 16 per clock per SM, 148 SMs, 1965 MHz"}}


def decode_record(peaks: dict, steps: int = 48) -> dict:
    """Cached greedy decode at the 1.5B shape (dim 2048, 22 blocks x 4 recursions, 32q/4kv heads of 16, SwiGLU 5632),
    batch 64, prompt 1024: ms per step and the weight + cache stream against the HBM peak."""
    import microbench
    ns = microbench.argparse_like(batch=64, blocks=22, prompt=1024, new_tokens=steps + 3, iters=1, impl=0)
    r = microbench.decode(ns)
    return {"shape": "1.5B: dim 2048, 22x4, 32q/4kv x16, F 5632; batch 64, prompt 1024", "ms_per_step": r["ms"],
            "tok_per_s": r["decode_tok_per_s"], "gbs": r["achieved"], "frac_of_hbm": r["achieved"] / float(peaks["hbm_gbs"]),
            "timed_steps": r["timed_steps"], "note": r["note"]}


def run_ours(args) -> None:
    from hydra_b200.model import HydraB200Model, random_state_dict

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback "
                         "(use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    B, K, W = args.batch, args.steps, max(args.warmup, 3)

    sd = random_state_dict(seed=SEED, device=dev, **ARCH)
    model = HydraB200Model(sd, n_heads=ARCH["n_heads"], n_kv_heads=ARCH["n_kv_heads"], max_seq_len=SEQ,
                           mod_capacity=ARCH["mod_capacity"], device=dev, fold_norm=args.fold_norm)
    # every rank draws its own sequences (seed offset by rank): a sharded global batch of world*B sequences
    ids_host = torch.randint(0, ARCH["vocab_size"], (B, SEQ),
                             generator=torch.Generator().manual_seed(SEED + 1 + rank)).pin_memory()
    ids = ids_host.to(dev)
    T = B * SEQ

    def sync_all():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed(fn, steps):
        """K calls bracketed by barrier + synchronize, CUDA events on the launching stream; max over ranks below."""
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        return e0.elapsed_time(e1)

    # routing statistics of this workload (deterministic): rows per (block, recursion); and how many launches one
    # forward makes, which sizes the launch recorder for the K timed steps
    model.enable_profile(4096)
    model(ids, taps=True, reuse_buffer=True)
    torch.cuda.synchronize(dev)
    mlp_rows = model.last_taps.mlp_rows.cpu().tolist()
    launches_per_forward = len(model.read_profile())
    model.disable_profile()
    for _ in range(W):
        model(ids, reuse_buffer=True)
    sync_all()

    # ---- timed region: K forwards, ids resident in HBM, nothing but the forward in it (the per-launch recorder is off: its
    # two event records per launch cost about 0.7 ms per step, and with it off the model replays its launch sequence as a
    # CUDA graph, which is what a caller gets)
    sampler = ClockSampler(local) if rank == 0 else None
    ms_total = timed(lambda: model(ids, reuse_buffer=True), K)
    model.check_device_errors()
    timed_seq0 = model._logits[:SEQ, :ARCH["vocab_size"]].clone()      # sequence 0 of the last timed step

    # ---- the same K forwards once more with the recorder on: per-kernel CUDA-event times for the breakdown / roofline
    model.enable_profile(launches_per_forward * K + 64)
    ms_recorded = timed(lambda: model(ids, reuse_buffer=True), K)
    records = model.read_profile()              # raises if the recorder overflowed
    if len(records) != launches_per_forward * K:
        raise SystemExit(f"launch recorder: {len(records)} records for {K} steps of {launches_per_forward} launches")
    model.check_device_errors()
    model.disable_profile()

    # ---- e2e: pinned host ids -> device, forward, last-position logits -> host, every step
    out_host = torch.empty((B, ARCH["vocab_size"]), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        model.prefill(ids_host, out_host)
    ms_e2e = timed(lambda: model.prefill(ids_host, out_host), K)
    clocks = sampler.stop() if sampler is not None else None

    t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = float(t[0]), float(t[1])
    tokens_all = world * T * K
    value = tokens_all / (ms_total * 1e-3)
    e2e = tokens_all / (ms_e2e * 1e-3)

    # ---- N > 1: the strong-scaling form of the same workload (a global batch of 32 sequences split over the ranks)
    strong = None
    if dist is not None and args.scaling_mode == "weak" and 32 % world == 0:
        Bs = 32 // world
        ids_s = ids[:Bs].contiguous() if Bs <= B else torch.randint(0, ARCH["vocab_size"], (Bs, SEQ), device=dev)
        for _ in range(3):
            model(ids_s, reuse_buffer=True)
        ms_s = timed(lambda: model(ids_s, reuse_buffer=True), K)
        ts = torch.tensor([ms_s], dtype=torch.float64, device=dev)
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        ms_s = float(ts[0])
        strong = {"global_batch": 32, "batch_per_gpu": Bs, "ms_per_step": ms_s / K, "value": 32 * SEQ * K / (ms_s * 1e-3),
                  "unit": "tok/s", "scaling": "strong"}

    # outside the timed region: gather the last-position logits of every rank (NCCL over NVLink)
    if dist is not None:
        last = model(ids, reuse_buffer=True)[:, -1, :].contiguous()
        gathered = torch.empty((world * B, ARCH["vocab_size"]), dtype=last.dtype, device=dev)
        dist.all_gather_into_tensor(gathered, last)
        torch.cuda.synchronize(dev)
        assert torch.isfinite(gathered.float()).all()

    if rank == 0:
        peaks, peak_src = measured_peaks()
        by_kind: dict = {}
        for r in records:
            d = by_kind.setdefault(r["kind"], {"launches": 0, "ms": 0.0})
            d["launches"] += 1
            d["ms"] += r["ms"]
        tot = sum(d["ms"] for d in by_kind.values()) or 1.0
        fl = routed_flops(records, mlp_rows, T)
        breakdown = {k: {"launches_per_step": d["launches"] / K, "ms_per_step": d["ms"] / K, "share": d["ms"] / tot,
                         "tflops": (fl.get(k, 0.0) / (d["ms"] * 1e-3) / 1e12) if fl.get(k) else None}
                     for k, d in sorted(by_kind.items(), key=lambda kv: -kv[1]["ms"])}
        dom = "gemm_gate_up"
        dom_ms = by_kind.get(dom, {"ms": 0.0})["ms"]
        achieved = fl.get(dom, 0.0) / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else 0.0
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        # DRAM traffic of one gate_up launch, scaled from the ncu capture of the same kernel at M = 8192 rows
        # (N = 5632, K = 1024: 28.40 MB read of which 11.53 MB is the weight, 5.02 MB written before the launch ended):
        # the weight is read once per launch whatever M is, everything else grows with the rows of the launch.
        cap_rows, cap_read, cap_write, cap_weight = 8192.0, 28.40e6, 5.02e6, 2.0 * 5632 * 1024
        n_dom = max(1, by_kind.get(dom, {"launches": 0})["launches"])
        dom_nk = next((r["n"] * r["k"] for r in records if r["kind"] == dom), 0)
        avg_rows = fl.get(dom, 0.0) / (2.0 * dom_nk) / n_dom if dom_nk else 0.0
        traffic = cap_weight + (cap_read - cap_weight + cap_write) / cap_rows * avg_rows
        all_fl = sum(v for k, v in fl.items())
        # the pre-attention convolutions are tensor work too (6 * (lat*hd + lat^2 + kvd*hd + kvd^2) FLOP per token and block)
        lat, hd = ARCH["dim"] // ARCH["compression_factor"], ARCH["dim"] // ARCH["compression_factor"] // ARCH["n_heads"]
        kvd = ARCH["n_kv_heads"] * hd
        all_fl += 6.0 * (lat * hd + lat * lat + kvd * hd + kvd * kvd) * T * ARCH["n_mor_blocks"] * K
        routed_per_token = all_fl / (T * K)
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": getattr(args, "scaling_mode", "weak"),
            "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(B, world),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": world * B * SEQ * 8,
                    "d2h_bytes_per_step": world * B * ARCH["vocab_size"] * 2, "ms_per_step": ms_e2e / K,
                    "api": "HydraB200Model.prefill(pinned int64 ids [B,S]) -> last-position logits [B,V] bf16 on the host"},
            "gpu_launches": launches_per_forward * K,
            "launches_per_step": launches_per_forward,
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<256> (gate_up + SwiGLU epilogue)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                         "peak_source": f"bf16_tflops_sustained, {peak_src}", "traffic": traffic,
                         "traffic_unit": "B/launch (DRAM read + write, scaled by rows from the ncu capture at M=8192)",
                         "avg_rows_per_launch": avg_rows,
                         "launches_per_step": by_kind.get(dom, {"launches": 0})["launches"] / K},
            "model_tflops": {"routed_flops_per_token": routed_per_token,
                             "dense_flops_per_token": 823.4e6,
                             "achieved_routed": routed_per_token * T * K / (ms_total * 1e-3) / 1e12,
                             "frac_of_sustained_peak_routed": routed_per_token * T * K / (ms_total * 1e-3) / 1e12 / peak},
            "breakdown": breakdown, "breakdown_ms_sum": tot / K,
            "breakdown_pass": {"ms_per_step": ms_recorded / K,
                               "note": "breakdown, roofline and model_tflops.per-kernel figures come from a second pass of the "
                                       "same K forwards with the per-launch event recorder on (direct launches); value and "
                                       "ms_per_step from the pass before it with the recorder off (graph replay)"},
            "mlp_rows": mlp_rows, "clocks": clocks,
        }
        if strong is not None:
            line["strong"] = strong
        if not args.no_parity:      # rank 0's first sequence, at every N (the other ranks wait at the final barrier)
            line["parity"] = parity_record(model, ids, timed_seq0, sd)
        if world == 1:
            del timed_seq0
            model._logits = None
            torch.cuda.empty_cache()
            if not args.no_cpu_baseline:
                cpu_sd = {k: v.to(torch.bfloat16).float().cpu() for k, v in sd.items()}
                line["cpu_baseline"] = cpu_arm(1, 2, 1, cpu_sd)
            if not args.no_extras:
                line["ccgqa_block"] = ccgqa_block_record(peaks)
                line["library_baseline"] = microbench_library_baseline(avg_rows)
                del model, sd
                torch.cuda.empty_cache()
                line["decode"] = decode_record(peaks)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def microbench_library_baseline(avg_rows: float) -> dict:
    import microbench
    try:
        return microbench.library_baseline(avg_rows, ROOT, REF_ARGS if reference_available() else None)
    except Exception as e:   # the comparator must never take the headline line down with it
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=None, help="sequences per GPU (default 32; the microbenchmarks default "
                    "to their own configuration: 8 sequences, 64 for decode)")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="weak (default): --batch sequences on every GPU; strong: --batch sequences in total, split over the GPUs")
    ap.add_argument("--fold-norm", dest="fold_norm", action="store_true",
                    help="pre-MLP norm folded into the first MLP contraction (rows gathered by the GEMM itself)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the post-timing comparison with the CPU oracle")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the records measured after the headline: ccgqa_block, library_baseline, decode")
    ap.add_argument("--micro", default=None, help="run one single-kernel microbenchmark instead of the model "
                    "(gemm, gemm_skinny, ccgqa_block, pre_attention, attention, rms_norm, rope, swiglu_ffn, swiglu_act, "
                    "model_hidden, decode, sample_rows)")
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=5632)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--epilogue", default="swiglu", choices=["store", "resid", "swiglu", "scatter"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=22, help="--micro decode: MoR blocks of the 1.5B shape")
    ap.add_argument("--prompt", type=int, default=1024, help="--micro decode: prompt length")
    ap.add_argument("--new-tokens", dest="new_tokens", type=int, default=256, help="--micro decode: tokens to generate")
    ap.add_argument("--gemm-impl", dest="impl_gemm", type=int, default=0)
    args = ap.parse_args()
    if args.micro is not None:
        import microbench
        if args.batch is None:
            args.batch = 64 if args.micro == "decode" else (32 if args.micro in ("gemm", "gemm_skinny", "model_hidden") else 8)
        args.impl = args.impl_gemm
        names = [n for n in microbench.CASES if n not in ("model_hidden", "decode", "gemm_skinny")] if args.micro == "all" else [args.micro]
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        dist = None
        if world > 1:
            # replicas: every rank runs the same microbenchmark on its own GPU (sequences are sharded by rank, nothing
            # is exchanged); the slowest rank's time is reported, tokens/s summed over the ranks
            import torch.distributed as dist
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        for nm in names:
            res = microbench.run(nm, args, ROOT)
            if dist is not None:
                t = torch.tensor([res["ms"]], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res["ms"] = float(t.item())
                res["n_gpus"] = world
                if "decode_tok_per_s" in res:
                    res["decode_tok_per_s"] = world * args.batch / (res["ms"] * 1e-3)
                    res["scaling"] = "weak"
            if nm == "decode" and not args.no_cpu_baseline and rank == 0:
                res["cpu_baseline"] = cpu_generation_baseline(args.blocks, args.prompt)
            if rank == 0:
                print(json.dumps(res), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    args.scaling_mode = args.scaling
    if args.batch is None:
        args.batch = 32
    if args.scaling == "strong":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if args.batch % world != 0:
            sys.exit(f"--scaling strong needs --batch ({args.batch}) divisible by the number of ranks ({world})")
        args.batch //= world
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
