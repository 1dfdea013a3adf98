#!/usr/bin/env python
"""Benchmark of the compressed tensor-swap hot path.

One "step" = ZFP fixed-rate compress + decompress of one float32 tensor
(default 256 MiB, rate 8, values tanh(N(0,1)), viewed 32 x 32 x numel/1024) on
each GPU.  Prints ONE JSON line:

  value     uncompressed GB/s through the round trip, all GPUs together:
            n_gpus * 2 * 4N bytes / (time of K steps / K), inputs resident in HBM
  roofline  the slower of the two kernels: algorithmic bytes (4N + N*rate/8) per
            launch / its CUDA-event duration, against the measured HBM peak
  e2e       the same round trip through the reference-named entry points
            cuda_compress / cuda_decompress with pinned HOST buffers
            (host->device and device->host copies inside the timed region)
  cpu_baseline  the CPU codec (oracle port, OpenMP over blocks) on a bounded
            sample of the same data, on this host's cores
  extra     sparse codec GB/s at 50/75/90 % zeros, swap-manager link numbers

`--impl reference` times the CPU implementation alone (the reference ships no
CPU codec, so this is the oracle port pinned against the reference's headers).

Multi-GPU: one process per GPU (torchrun), every rank codes its own tensor,
no collective on the data path; time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
# stdout carries exactly one JSON line: keep NCCL's version banner off it
if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
    os.environ["NCCL_DEBUG"] = "WARN"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mib", type=int, default=256, help="tensor size in MiB (float32)")
    ap.add_argument("--rate", type=int, default=8, help="ZFP bits per value")
    ap.add_argument("--workload", default="zfp", choices=["zfp", "vgg16", "bert"],
                    help="zfp: codec round trip (headline); vgg16 / bert: one swapped training step")
    ap.add_argument("--batch", type=int, default=0, help="batch size of the model workloads (0: 128 / 32)")
    ap.add_argument("--no-extra", action="store_true", help="skip the sparse / swap-link side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    return ap.parse_args()


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# clocks while the timed region runs (read-only NVML queries)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._active = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.t = threading.Thread(target=self._run, daemon=True)
            self.t.start()
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            if self._active:
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                    for bit, name in self.REASONS.items():
                        if r & bit and name != "gpu_idle":
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(0.002)

    def start(self):
        self._active = True

    def stop(self):
        self._active = False

    def summary(self):
        self._stop.set()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------
# CPU leg (oracle port); only place outside tests that runs oracle/
# ---------------------------------------------------------------------------
def cpu_codec_sample(mib_total: int, rate: int, budget_s: float = 12.0):
    """Round-trip GB/s of the CPU codec on a bounded sample of the workload."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    threads = O.max_threads()
    sample_mib = min(mib_total, max(8, 4 * threads))
    n = sample_mib * 262144
    rng = np.random.default_rng(0)
    a = np.tanh(rng.standard_normal(n, dtype=np.float32))
    nz = n // 1024
    best = None
    t_start = time.perf_counter()
    reps = 0
    while reps < 3 and (time.perf_counter() - t_start < budget_s or reps == 0):
        t0 = time.perf_counter()
        s = O.zfp_encode(a, 32, 32, nz, 64 * rate, threads=threads)
        O.zfp_decode(s, 32, 32, nz, 64 * rate, threads=threads)
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
        reps += 1
    gbs = 2 * 4 * n / best / 1e9
    return gbs, threads, f"{sample_mib} MiB slice of the {mib_total} MiB tensor, best of {reps} round trips"


def run_reference(args):
    """The reference arm: the CPU implementation of the path on this host."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np  # noqa: F401
    from oracle import oracle as O
    O.build()
    threads = O.max_threads()
    import numpy as np
    sample_mib = min(args.mib, max(8, 2 * threads))
    n = sample_mib * 262144
    a = np.tanh(np.random.default_rng(0).standard_normal(n, dtype=np.float32))
    nz = n // 1024

    def step():
        s = O.zfp_encode(a, 32, 32, nz, 64 * args.rate, threads=threads)
        O.zfp_decode(s, 32, 32, nz, 64 * args.rate, threads=threads)

    for _ in range(min(args.warmup, 2)):
        step()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    gbs = 2 * 4 * n / dt / 1e9
    sample = f"{sample_mib} MiB slice per step, {steps} timed steps (of {args.steps} requested), {threads} OpenMP threads"
    line = {
        "impl": "reference", "metric": "zfp_roundtrip_uncompressed_GBps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32->i32/u64", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU codec (zfp.c is stripped); this is the CPU restatement of its GPU "
                "algorithm, pinned against a host build of the reference's own headers",
    }
    print(json.dumps(line))


def max_over_ranks(values, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity on one rank)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def whole_job_gbps(world: int, bytes_per_rank_per_step: float, seconds_per_step: float) -> float:
    """Every rank codes its own tensor (weak scaling): the job's throughput is
    all ranks' bytes over the slowest rank's time."""
    return world * bytes_per_rank_per_step / seconds_per_step / 1e9


def workload_config(args):
    n = args.mib * 262144
    return {"workload": f"ZFP fixed-rate round trip (compress + decompress), float32 {args.mib} MiB tensor "
                        f"viewed 32x32x{n // 1024}, rate {args.rate} bits/value, values tanh(N(0,1))",
            "tensor_mib": args.mib, "rate": args.rate, "maxbits": 64 * args.rate,
            "cache": "inputs larger than L2 (no flush needed)" if args.mib > 126 else "L2 flushed between steps",
            "parallelism": f"{args.gpus} independent replica(s), no collective"}


def bind_host_threads_near_gpu(index: int) -> bool:
    """Run this process on the CPUs next to its GPU (NVML's affinity for the
    device), so that the pinned host buffers it allocates land in the memory
    of that socket.  With several ranks per host the end-to-end numbers
    otherwise share one socket's memory.  A property of this process only."""
    try:
        import pynvml
        pynvml.nvmlInit()
        pynvml.nvmlDeviceSetCpuAffinity(pynvml.nvmlDeviceGetHandleByIndex(index))
        return True
    except Exception:
        return False


def run_model_workload(args):
    """Swapped training step (VGG16 batch 128 on 3x32x32, or BERT-base-shaped
    encoder batch 32 x seq 512): step latency without swapping, with raw swap of
    every activation (vDNN-style), with the reference's hard-wired split and
    with the cost model's per-tensor choice, plus the bytes each puts on the
    host link."""
    import torch
    import torch.distributed as dist
    import cswap_b200 as cs
    from cswap_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1 + rank)
    if args.workload == "vgg16":
        batch = args.batch or 128
        model = W.VGG16().to(dev).train()
        hx = torch.randn(batch, 3, 32, 32).pin_memory()
        hy = torch.randint(0, 10, (batch,)).pin_memory()
        maxbits, pinned, staging, nids = 512, 2 << 30, 512 << 20, 64
        name = f"VGG16 CIFAR-10-shaped training step, fp32, batch {batch}, synthetic 3x32x32 inputs"
    else:
        batch = args.batch or 32
        model = W.BertEncoder().to(dev).train()
        hx = torch.randint(0, 30522, (batch, 512)).pin_memory()
        hy = torch.randint(0, 2, (batch,)).pin_memory()
        maxbits, pinned, staging, nids = 1024, 24 << 30, 4 << 30, 400
        name = f"BERT-base-shaped encoder training step, fp32, batch {batch}, seq 512, 12 layers"
    mgr = cs.SwapManager(pinned_bytes=pinned, staging_bytes=staging, zfp_maxbits=maxbits)
    make_batch = lambda: (hx, hy)
    steps, warmup = max(1, min(args.steps, 20)), max(3, min(args.warmup, 5))

    def fresh(policy_fn):
        exe = cs.Execution(mgr=mgr)
        exe.init_(nids)
        policy_fn(exe)
        return exe

    def all_raw(exe):
        for i in range(nids):
            exe.begin_stage[i] = i + 1
            exe.policy[i] = cs.POLICY_RAW

    results = {}
    results["no_swap"] = W.timed_steps(model, fresh(lambda e: None), make_batch, steps, warmup)
    results["raw_swap"] = W.timed_steps(model, fresh(all_raw), make_batch, steps, warmup)

    def all_zfp(exe):
        for i in range(nids):
            exe.begin_stage[i] = i + 1
            exe.policy[i] = cs.POLICY_ZFP

    results["zfp_everywhere"] = W.timed_steps(model, fresh(all_zfp), make_batch, steps, warmup)
    if args.workload == "vgg16":
        results["reference_split_zfp8"] = W.timed_steps(model, fresh(W.vgg16_reference_policy), make_batch, steps,
                                                        warmup)
        # the baseline planners of the reference's drivers (policy_ 3 and 4)
        results["vdnn_baseline"] = W.timed_steps(model, fresh(lambda e: W.vgg16_baseline_policy(e, 3)), make_batch,
                                                 steps, warmup)
        results["superneurons_baseline"] = W.timed_steps(model, fresh(lambda e: W.vgg16_baseline_policy(e, 4)),
                                                         make_batch, steps, warmup)
    # self-tuning: profile one step, fit the cost model on this GPU, decide per tensor
    exe = fresh(lambda e: None)
    exe.profile = True
    x, y = hx.to(dev), hy.to(dev)
    if x.is_floating_point():
        x.requires_grad_(True)
    model.forward_with(exe, x, y).backward()
    prof = exe.finish_profile()
    cm = cs.CostModel.fit(mgr, maxbits)
    def run_under(e):
        def run(k):
            r = W.timed_steps(model, e, make_batch, k, 0)
            return r["ms_per_step"] * k * 1e-3
        return run

    # the cost model's table, then a short measured run-off against its ZFP-eager neighbour
    lossy = None if args.workload == "vgg16" else [i for i, p in prof.items() if p["float32"]]
    cands = exe.policy_candidates(prof, cm, lossy_ids=lossy)
    chosen = exe.refine_policy(cands, run_under(exe))
    policy = list(exe.policy)
    results["self_tuned"] = W.timed_steps(model, exe, make_batch, steps, warmup)
    counts = {str(k): policy.count(k) for k in (0, 2, 3, 6)}
    counts["chosen"] = chosen
    if args.workload == "vgg16":
        # swap-or-recompute table in the manner of the Capuchin baseline (policy_ 2)
        exe_cap = fresh(lambda e: None)
        cap = exe_cap.make_policy_capuchin(prof, cm)
        results["capuchin_style_baseline"] = W.timed_steps(model, exe_cap, make_batch, steps, warmup)
        results["capuchin_style_baseline"]["policy_counts"] = {str(k): cap.count(k) for k in (0, 1, 2)}
    # the same decision when loss is acceptable on every float activation
    exe_all = fresh(lambda e: None)
    cands_all = exe_all.policy_candidates(prof, cm, lossy_ids=[i for i, p in prof.items() if p["float32"]])
    chosen_all = exe_all.refine_policy(cands_all, run_under(exe_all))
    policy_all = list(exe_all.policy)
    results["self_tuned_lossy_everywhere"] = W.timed_steps(model, exe_all, make_batch, steps, warmup)
    counts_all = {str(k): policy_all.count(k) for k in (0, 2, 3, 6)}
    counts_all["chosen"] = chosen_all
    t_tuned, t_raw, t_none = (max_over_ranks([results[k]["ms_per_step"]], dev)[0]
                              for k in ("self_tuned", "raw_swap", "no_swap"))
    raw, tuned = results["raw_swap"], results["self_tuned"]
    if rank == 0:
        line = {
            "metric": f"{args.workload}_swapped_step_ms", "value": t_tuned, "unit": "ms/step", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": t_tuned, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "parallelism": f"{world} independent replica(s), no collective",
                       "zfp_maxbits": maxbits, "policy_counts": counts,
                       "policy_counts_lossy_everywhere": counts_all},
            "step_ms": {"no_swap": t_none, "raw_swap": t_raw, "self_tuned": t_tuned,
                        "self_tuned_lossy_everywhere": results["self_tuned_lossy_everywhere"]["ms_per_step"],
                        **{k: results[k]["ms_per_step"]
                           for k in ("zfp_everywhere", "reference_split_zfp8", "vdnn_baseline",
                                     "superneurons_baseline", "capuchin_style_baseline")
                           if k in results}},
            "peak_device_mib": {k: round(v["peak_device_bytes"] / 2**20, 1) for k, v in results.items()},
            "raw_swap": raw, "self_tuned": tuned,
            "activation_bytes_per_link_byte": {
                k: v["activation_bytes_per_step"] / max(v["link_bytes_out_per_step"], 1)
                for k, v in results.items() if v["link_bytes_out_per_step"] > 0},
            "cost_model": cm.as_dict(),
        }
        print(json.dumps(line))
    mgr.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "zfp":
        run_model_workload(args)
        return

    import torch
    import torch.distributed as dist
    import cswap_b200 as cs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the codec has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        bind_host_threads_near_gpu(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = cs.lib()

    n = args.mib * 262144
    maxbits = 64 * args.rate
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.tanh(torch.randn(n, device=dev, generator=g))
    stream_bytes = cs.zfp_max_bytes(32, 32, n // 1024, maxbits)
    comp = torch.empty(stream_bytes, dtype=torch.uint8, device=dev)
    y = torch.empty_like(x)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev) if args.mib <= 126 else None

    def step():
        cs.zfp_compress(x, maxbits, out=comp)
        cs.zfp_decompress(comp, n, maxbits, out=y)
        if flush is not None:
            flush.fill_(1)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record()
    for k in range(args.steps):
        evs[k][0].record()
        cs.zfp_compress(x, maxbits, out=comp)
        evs[k][1].record()
        cs.zfp_decompress(comp, n, maxbits, out=y)
        evs[k][2].record()
        if flush is not None:
            flush.fill_(1)
    e_end.record()
    torch.cuda.synchronize()
    sampler.stop()
    if world > 1:
        dist.barrier()
    t_enc = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps * 1e-3
    t_dec = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps * 1e-3
    if flush is None:
        t_total = e_begin.elapsed_time(e_end) * 1e-3
    else:
        t_total = (t_enc + t_dec) * args.steps  # the flush is not part of the step
    assert L.csw_device_status(None) == 0, "a kernel reported a bounded-wait timeout"
    t_total, t_enc, t_dec = max_over_ranks([t_total, t_enc, t_dec], dev)
    ms_per_step = t_total / args.steps * 1e3
    value = whole_job_gbps(world, 2 * 4 * n, t_total / args.steps)

    # ---- end to end through the reference-named entry points, host buffers ----
    import ctypes as C
    from cswap_b200._lib import Bitstream, ZfpField, ZfpStream
    h_field = torch.empty(n, dtype=torch.float32).pin_memory()
    h_field.copy_(x)
    h_stream = torch.empty(stream_bytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n, dtype=torch.float32).pin_memory()
    fld_in = ZfpField(3, 32, 32, n // 1024, 0, 0, 0, 0, 0, h_field.data_ptr())
    fld_out = ZfpField(3, 32, 32, n // 1024, 0, 0, 0, 0, 0, h_out.data_ptr())

    def e2e_step():
        sp = h_stream.data_ptr()
        bs = Bitstream(0, 0, sp, sp, sp + stream_bytes)
        zs = ZfpStream(maxbits, maxbits, 32, -1074, C.pointer(bs))
        got = L.cuda_compress(C.byref(zs), C.byref(fld_in))
        assert got == stream_bytes
        bs2 = Bitstream(0, 0, sp, sp, sp + stream_bytes)
        zs2 = ZfpStream(maxbits, maxbits, 32, -1074, C.pointer(bs2))
        L.cuda_decompress(C.byref(zs2), C.byref(fld_out))

    e2e_steps = max(1, min(args.steps, 10))
    torch.cuda.synchronize()
    for _ in range(2):
        e2e_step()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()  # blocking calls, as the reference's are
    t_e2e = (time.perf_counter() - t0) / e2e_steps
    t_e2e = max_over_ranks([t_e2e], dev)[0]
    e2e_ok = bool(torch.equal(h_out, y.cpu()))
    e2e = {"value": whole_job_gbps(world, 2 * 4 * n, t_e2e), "unit": "GB/s", "h2d_bytes_per_step": 4 * n + stream_bytes,
           "d2h_bytes_per_step": 4 * n + stream_bytes, "ms_per_step": t_e2e * 1e3, "steps": e2e_steps,
           "matches_device_path": e2e_ok,
           "path": "cuda_compress + cuda_decompress with pinned host field and stream buffers"}

    # ---- roofline of the slower kernel ----
    peak, peak_kind = load_peaks()
    alg = 4 * n + n * args.rate // 8
    name, t_k = ("zfp_encode_slab_kernel", t_enc) if t_enc >= t_dec else ("zfp_decode_slab_kernel", t_dec)
    # DRAM read + write bytes of one launch from the committed ncu capture of this exact
    # workload (profiles/zfp_slab_kernels_256MiB_rate8.md); unknown for other sizes / rates
    ncu_traffic = {("zfp_encode_slab_kernel", 256, 8): 317.7e6, ("zfp_decode_slab_kernel", 256, 8): 276.2e6}
    roofline = {"bound": "hbm", "kernel": name, "achieved": alg / t_k / 1e9, "peak": peak, "unit": "GB/s",
                "frac": alg / t_k / 1e9 / peak, "peak_kind": f"of {peak_kind}", "traffic": ncu_traffic.get((name, args.mib, args.rate)),
                "algorithmic_bytes_per_launch": alg,
                "encode": {"ms": t_enc * 1e3, "GBps_algorithmic": alg / t_enc / 1e9, "frac": alg / t_enc / 1e9 / peak},
                "decode": {"ms": t_dec * 1e3, "GBps_algorithmic": alg / t_dec / 1e9, "frac": alg / t_dec / 1e9 / peak},
                "roundtrip_frac": 2 * alg / (t_enc + t_dec) / 1e9 / peak}

    extra = {}
    if not args.no_extra:
        extra = side_measurements(cs, torch, dev, peak)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, cores, sample = cpu_codec_sample(args.mib, args.rate)
        cpu = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}

    clocks = sampler.summary()
    if rank == 0:
        line = {
            "metric": "zfp_roundtrip_uncompressed_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32->i32/u64", "data": "synthetic",
            "config": workload_config(args), "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": 2 * args.steps, "clocks": clocks, "extra": extra,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def side_measurements(cs, torch, dev, peak):
    """Sparse codec throughput per sparsity (16 MiB and 256 MiB tensors) and the
    swap manager's host-link numbers.  Reported beside the headline, not in it."""
    out = {"sparse": [], "swap": {}, "zfp_rates": []}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn, reps=10):
        fn()
        ts = []
        for _ in range(reps):
            flush.fill_(0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2]

    for mib in (16, 256):
        n = mib * 262144
        for zf, mu in ((0.5, 0.0), (0.75, -0.6745), (0.9, -1.2816)):
            g = torch.Generator(device=dev).manual_seed(int(zf * 100))
            t = torch.relu(torch.randn(n, device=dev, generator=g) + mu)
            packed, nnz_t = cs.sparse_compress(t)
            nnz = int(nnz_t.item())
            back = torch.empty_like(t)
            tc = timeit(lambda: cs.sparse_compress(t, out=packed, nnz_out=nnz_t))
            t1 = timeit(lambda: cs.sparse_compress(t, out=packed, nnz_out=nnz_t, onepass=True))
            td = timeit(lambda: cs.sparse_decompress(packed, n, out=back))
            alg = 4 * n + 4 * nnz + n // 8
            out["sparse"].append({
                "tensor_mib": mib, "zero_fraction": round(1 - nnz / n, 4),
                "ratio": 4 * n / cs.sparse_packed_bytes(n, nnz),
                "compress_GBps_uncompressed": 4 * n / tc / 1e9, "decompress_GBps_uncompressed": 4 * n / td / 1e9,
                "onepass_compress_GBps_uncompressed": 4 * n / t1 / 1e9,
                "compress_frac_hbm": alg / tc / 1e9 / peak, "onepass_compress_frac_hbm": alg / t1 / 1e9 / peak,
                "decompress_frac_hbm": alg / td / 1e9 / peak,
                "exact": bool(torch.equal(back.view(torch.int32), t.view(torch.int32)))})
            del t, packed, back
    # the ZFP kernels at the other two rates the reference's drivers use (256 MiB tensor)
    n = 256 * 262144
    t = torch.tanh(torch.randn(n, device=dev))
    back = torch.empty_like(t)
    for rate in (4, 8, 16):
        mb = 64 * rate
        comp = torch.empty(cs.zfp_max_bytes(32, 32, n // 1024, mb), dtype=torch.uint8, device=dev)
        te = timeit(lambda: cs.zfp_compress(t, mb, out=comp))
        td = timeit(lambda: cs.zfp_decompress(comp, n, mb, out=back))
        alg = 4 * n + n * rate // 8
        out["zfp_rates"].append({"tensor_mib": 256, "rate": rate, "encode_ms": te * 1e3, "decode_ms": td * 1e3,
                                 "encode_frac_hbm": alg / te / 1e9 / peak, "decode_frac_hbm": alg / td / 1e9 / peak})
        del comp
    del t, back
    # swap link: raw vs ZFP-8 swap-out + swap-in of a 64 MiB tensor through the manager
    mgr = cs.SwapManager(pinned_bytes=512 << 20, staging_bytes=256 << 20)
    n = 64 * 262144
    t = torch.tanh(torch.randn(n, device=dev))
    dst = torch.empty_like(t)
    for name, pol in (("raw", cs.POLICY_RAW), ("zfp8", cs.POLICY_ZFP)):
        def trip():
            tk = mgr.swap_out(t, pol)
            mgr.swap_in(tk, out=dst)
            torch.cuda.synchronize()
            tk.release()
        trip()
        t0 = time.perf_counter()
        for _ in range(5):
            trip()
        dt = (time.perf_counter() - t0) / 5
        out["swap"][name] = {"tensor_mib": 64, "out_plus_in_ms": dt * 1e3, "uncompressed_GBps": 2 * 4 * n / dt / 1e9}
    mgr.close()
    return out


if __name__ == "__main__":
    main()
