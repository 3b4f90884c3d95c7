#!/usr/bin/env python
"""Headline benchmark: HYDRA-250M bf16 inference prefill throughput (tokens/s) on N B200s of one node.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU arm: the oracle port of the reference's eager forward

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
            divided by its summed launch time, both measured in the timed steps with CUDA events recorded by
            the executor around every launch
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
    n_seq = 1
    tps, dt, threads = cpu_forward_tokens_per_s(n_seq, args.steps, min(args.warmup, 1))
    cfg = workload_config(args.batch, args.gpus)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": getattr(args, "scaling_mode", "weak"),
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{n_seq} sequence x {SEQ} tokens of the same workload per step "
                                   "(CPU port of the reference's eager fp32 forward; the Python reference itself "
                                   "cannot travel to the GPU box)"},
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
                           mod_capacity=ARCH["mod_capacity"], device=dev)
    # every rank draws its own sequences (seed offset by rank): a sharded global batch of world*B sequences
    ids_host = torch.randint(0, ARCH["vocab_size"], (B, SEQ),
                             generator=torch.Generator().manual_seed(SEED + 1 + rank)).pin_memory()
    ids = ids_host.to(dev)
    T = B * SEQ
    model.enable_profile(2048)

    def sync_all():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # routing statistics of this workload (deterministic): rows per (block, recursion)
    model(ids, taps=True)
    torch.cuda.synchronize(dev)
    mlp_rows = model.last_taps.mlp_rows.cpu().tolist()
    model.read_profile()
    for _ in range(W):
        model(ids)
    sync_all()
    model.read_profile()

    # ---- timed region: K forwards, ids resident in HBM
    sampler = ClockSampler(local) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per_step_records = []
    ev0.record()
    for _ in range(K):
        model(ids)
    ev1.record()
    sync_all()
    ms_total = ev0.elapsed_time(ev1)
    records = model.read_profile()
    launches_per_step = len(records) // max(1, K)
    model.check_device_errors()

    # ---- e2e: pinned host ids -> device, forward, last-position logits -> host, every step
    out_host = torch.empty((B, ARCH["vocab_size"]), dtype=torch.bfloat16).pin_memory()
    model.disable_profile()
    for _ in range(2):
        model.prefill(ids_host, out_host)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        model.prefill(ids_host, out_host)
    e1.record()
    sync_all()
    ms_e2e = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler is not None else None

    t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = float(t[0]), float(t[1])
    tokens_all = world * T * K
    value = tokens_all / (ms_total * 1e-3)
    e2e = tokens_all / (ms_e2e * 1e-3)

    # outside the timed region: gather the last-position logits of every rank (NCCL over NVLink)
    if dist is not None:
        last = model(ids)[:, -1, :].contiguous()
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
        breakdown = {k: {"launches_per_step": d["launches"] // K, "ms_per_step": d["ms"] / K, "share": d["ms"] / tot,
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
        all_gemm_fl = sum(v for k, v in fl.items())
        routed_per_token = all_gemm_fl / (T * K)
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": getattr(args, "scaling_mode", "weak"),
            "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(B, world),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": world * B * SEQ * 8,
                    "d2h_bytes_per_step": world * B * ARCH["vocab_size"] * 2, "ms_per_step": ms_e2e / K,
                    "api": "HydraB200Model.prefill(pinned int64 ids [B,S]) -> last-position logits [B,V] bf16 on the host"},
            "gpu_launches": launches_per_step * K,
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel<256> (gate_up + SwiGLU epilogue)",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if peak else None,
                         "peak_source": f"bf16_tflops_sustained, {peak_src}", "traffic": traffic,
                         "traffic_unit": "B/launch (DRAM read + write, scaled by rows from the ncu capture at M=8192)",
                         "avg_rows_per_launch": avg_rows,
                         "launches_per_step": by_kind.get(dom, {"launches": 0})["launches"] // K},
            "model_tflops": {"routed_flops_per_token": routed_per_token,
                             "dense_flops_per_token": 823.4e6,
                             "achieved_routed": routed_per_token * T * K / (ms_total * 1e-3) / 1e12 / 1.0,
                             "frac_of_sustained_peak_routed": routed_per_token * T * K / (ms_total * 1e-3) / 1e12 / peak},
            "breakdown": breakdown, "mlp_rows": mlp_rows, "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu_sd = {k: v.to(torch.bfloat16).float().cpu() for k, v in sd.items()}
            tps, dt, threads = cpu_forward_tokens_per_s(1, 1, 0, cpu_sd)
            line["cpu_baseline"] = {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                                    "sample": f"1 sequence x {SEQ} tokens of the same workload and weights, one timed "
                                              f"forward ({dt:.1f} s), CPU port of the reference's eager fp32 forward"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=32, help="sequences per GPU")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="weak (default): --batch sequences on every GPU; strong: --batch sequences in total, split over the GPUs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
        from hydra_b200 import microbench
        if args.micro == "decode":
            args.batch = 64 if args.batch == 32 else args.batch
        elif args.micro not in ("gemm", "gemm_skinny", "model_hidden"):
            args.batch = 8 if args.batch == 32 else args.batch
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
