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
  extra     reference_cuda (the reference's own CUDA kernels on the same tensors,
            when their build is present), link (plain pinned-copy ceiling with
            all ranks copying at once), zfp_sweep (64 KiB .. 512 MiB x rates x
            distributions), sparse codec at 50/75/90 % zeros, swap-manager
            trips, vgg16 (swapped training step and the activation bytes that
            can be swapped within a stated stretch of the step)

`--impl reference` times the CPU implementation on the whole tensor (the
reference ships no CPU codec, so this is the oracle port, pinned against the
reference's headers and against the output of its CUDA kernels) and, where a
GPU and the reference's CUDA build are present, reports the reference's own
kernels beside it.

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


# Standard output carries exactly one JSON line.  Libraries print there too (NCCL's
# version banner, the reference's timing lines), so file descriptor 1 is pointed at
# standard error for the run and the line goes to the descriptor saved here.
_REAL_STDOUT = None


def guard_stdout():
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line) -> None:
    data = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    if _REAL_STDOUT is None:
        os.write(1, data)
    else:
        os.write(_REAL_STDOUT, data)


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
    ap.add_argument("--no-vgg", action="store_true", help="skip the swapped VGG16 step in the side measurements")
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
def host_threads() -> int:
    """CPU threads this process may run on.  Counted from the affinity mask:
    launchers such as torchrun export OMP_NUM_THREADS=1, which must not decide
    how many cores the CPU codec gets."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_codec_sample(mib_total: int, rate: int, budget_s: float = 12.0):
    """Round-trip GB/s of the CPU codec on a bounded sample of the workload."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    threads = host_threads()
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


def reference_cuda_times(mib: int, rate: int, device=None):
    """The reference's own CUDA kernels (cuZFP.cu / compression.cu compiled for
    sm_100a, oracle/_ref/libcswap_ref_cuda.so) on this GPU: ZFP encode / decode
    of the benchmark tensor and the sparse codec on config 2's tensor, timed
    with CUDA events on the legacy default stream they run on.  None where the
    build or a GPU is missing.  The calls include what the reference's entry
    points do around the kernel (a cudaMemset of the stream and two device
    synchronisations, cuZFP.cu:392-399, encode3.cuh:152)."""
    try:
        import torch
        from oracle import oracle as O
        if not (torch.cuda.is_available() and O.have_ref_cuda()):
            return None
        R = O.ref_cuda()
    except Exception:
        return None
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())

    def best_ms(fn, reps=3):
        fn()
        out = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return min(out)

    n = mib * 262144
    nz, maxbits = n // 1024, 64 * rate
    with torch.cuda.device(dev):
        x = torch.tanh(torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(1234)))
        nbytes = n * rate // 8
        buf = torch.zeros(nbytes + 4096, dtype=torch.uint8, device=dev)
        y = torch.empty_like(x)
        te = best_ms(lambda: R.refcuda_zfp_compress(x.data_ptr(), 32, 32, nz, maxbits, buf.data_ptr(), buf.numel()))
        td = best_ms(lambda: R.refcuda_zfp_decompress(buf.data_ptr(), buf.numel(), 32, 32, nz, maxbits, y.data_ptr()))
        res = {"zfp": {"tensor_mib": mib, "rate": rate, "encode_ms": te, "decode_ms": td,
                       "roundtrip_uncompressed_GBps": 2 * 4 * n / ((te + td) * 1e-3) / 1e9},
               "sparse": []}
        del x, y, buf
        ns = 128 * 128 * 16 * 16
        P = 512 * 32
        chunk = -(-ns // P)
        begin = torch.zeros(P, dtype=torch.int32, device=dev)
        num = torch.zeros(1, dtype=torch.int32, device=dev)
        bitmap = torch.zeros(P * (-(-chunk // 32)), dtype=torch.int32, device=dev)
        values = torch.zeros(ns, device=dev)
        out = torch.zeros(ns, device=dev)
        for zf, mu in ((0.5, 0.0), (0.75, -0.6745), (0.9, -1.2816)):
            t = torch.relu(torch.randn(ns, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) + mu)
            tc = best_ms(lambda: R.refcuda_sparse_compress(t.data_ptr(), ns, 512, 32, begin.data_ptr(), num.data_ptr(),
                                                           bitmap.data_ptr(), values.data_ptr()))
            tdd = best_ms(lambda: R.refcuda_sparse_decompress(values.data_ptr(), out.data_ptr(), ns, 512, 32,
                                                              bitmap.data_ptr(), begin.data_ptr()))
            # the reference's scatter leaves the positions after a word's last set bit unwritten
            # (compression.cu:281-292): check it on a zeroed destination, as its caller provides
            out.zero_()
            torch.cuda.synchronize()
            R.refcuda_sparse_decompress(values.data_ptr(), out.data_ptr(), ns, 512, 32, bitmap.data_ptr(),
                                        begin.data_ptr())
            torch.cuda.synchronize()
            res["sparse"].append({"tensor_mib": 16, "zero_fraction": zf, "compress_ms": tc, "decompress_ms": tdd,
                                  "exact": bool(torch.equal(out, t))})
    res["what"] = ("the reference's cuda_compress / cuda_decompress and PreGPUcompression+PreAcc+GPUcompression / "
                   "GPUdecompression, device pointers, compiled for sm_100a from its own sources")
    return res


def run_reference(args):
    """The reference arm: the CPU implementation of the path on this host's
    cores, whole tensor per step, every step and warm-up asked for; plus, where
    possible, the reference's own CUDA kernels on this GPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O
    O.build()
    threads = host_threads()
    n = args.mib * 262144
    a = np.tanh(np.random.default_rng(0).standard_normal(n, dtype=np.float32))
    nz = n // 1024

    def step():
        s = O.zfp_encode(a, 32, 32, nz, 64 * args.rate, threads=threads)
        O.zfp_decode(s, 32, 32, nz, 64 * args.rate, threads=threads)

    for _ in range(args.warmup):
        step()
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    gbs = 2 * 4 * n / dt / 1e9
    sample = f"the whole {args.mib} MiB tensor per step, {steps} timed steps, {threads} OpenMP threads"
    line = {
        "impl": "reference", "metric": "zfp_roundtrip_uncompressed_GBps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32->i32/u64", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "reference_cuda": reference_cuda_times(args.mib, args.rate),
        "note": "the reference has no CPU codec (zfp.c is stripped); `value` is the CPU restatement of its GPU "
                "algorithm, pinned against a host build of the reference's own headers and against the output "
                "of its CUDA kernels; reference_cuda times those kernels themselves on this GPU",
    }
    emit(line)


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
    mgr.close()
    del model
    torch.cuda.empty_cache()
    # the same workload through the C++ host side; every rank runs it, rank 0 reports
    cpp = vgg16_cpp_block(torch, dev, world, rank, local) if args.workload == "vgg16" else \
        cpp_step_block(torch, dev, world, rank, local, "bert_step", ["--steps", str(steps), "--warmup", str(warmup)])
    if rank == 0:
        line["cpp_host_side"] = cpp
    if rank == 0:
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def hidden_bytes_sweep(W, cs, torch, model, mgr, make_batch, prof, policy_of, t_no_swap_ms, eps_list,
                       steps=6, warmup=2):
    """How many activation bytes can be swapped out and back within a stated
    stretch of the step.  Candidates are the activations autograd keeps for
    backward, largest first; the k largest are swapped under `policy_of(id)`,
    for k = 0, 1, 2, ...; a point is "hidden" at eps when its median step time
    stays within (1 + eps) of the no-swap step.  Returns, per eps, the largest
    swapped activation bytes among the hidden points, and the measured curve."""
    ids = [i for i, p in prof.items() if p["saved"] and p["float32"] and p["has_grad"] and not p["omit"]
           and p["numel"] >= 1 << 18]
    consumer = {}
    for idx in sorted(prof):
        for tid in prof[idx]["inputs"]:
            consumer.setdefault(tid, idx)
    ids = [i for i in ids if i in consumer]
    ids.sort(key=lambda i: -prof[i]["numel"])
    nids = max(prof) + 2
    curve = []
    ks = list(range(0, len(ids) + 1))
    for k in ks:
        exe = cs.Execution(mgr=mgr)
        exe.init_(nids)
        for tid in ids[:k]:
            exe.policy[tid] = policy_of(tid)
            exe.begin_stage[tid] = consumer[tid]
        r = W.timed_steps(model, exe, make_batch, steps, warmup)
        # bytes that went out AND came back through the link (a lossless tensor taken back
        # before it had left the device is not counted)
        curve.append({"k": k, "ms_median": r["ms_median"], "activation_bytes": r["activation_bytes_back_per_step"],
                      "link_bytes_out": r["link_bytes_out_per_step"], "link_bytes_in": r["link_bytes_in_per_step"]})
    hidden = {}
    for eps in eps_list:
        ok = [c["activation_bytes"] for c in curve if c["ms_median"] <= (1 + eps) * t_no_swap_ms]
        hidden[f"{eps:g}"] = max(ok) if ok else 0.0
    return {"candidates": len(ids), "hidden_activation_bytes": hidden, "curve": curve}


def cpp_step_block(torch, dev, world, rank, local, name, extra_args):
    """Launch tests/cpp/<name> --bench on this rank's GPU (all ranks behind one
    barrier), parse its JSON line and add the slowest rank's time to every row."""
    import subprocess
    import torch.distributed as dist
    exe = os.path.join(ROOT, "tests", "cpp", name)
    if not os.path.exists(exe):
        return {"unavailable": f"tests/cpp/{name} has not been built (python -m cswap_b200.build --cpp)"}
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    r = subprocess.run([exe, "--bench", "--device", str(local), "--seed", str(1 + rank)] + list(extra_args),
                       capture_output=True, text=True, timeout=1500)
    if r.returncode != 0:
        return {"unavailable": f"{name} exited {r.returncode}: {r.stderr[-300:]}"}
    d = json.loads(r.stdout.strip().splitlines()[-1])
    names = sorted(d["rows"])
    worst = max_over_ranks([d["rows"][k]["ms_per_step_median"] for k in names], dev)
    for k, w in zip(names, worst):
        d["rows"][k]["ms_per_step_median_slowest_rank"] = w
    d["ranks_running"] = world
    return d


def vgg16_cpp_block(torch, dev, world, rank, local):
    """The swapped VGG16 step through the C++ host side (cswap::Execution over
    libtorch, tests/cpp/vgg16_step.cpp, the driver laid out like the
    reference's vgg16-cifar10.cpp): every rank launches the binary on its own
    GPU behind one barrier, so the ranks share the host link while they run.
    Rank 0's line is reported, with each row's step time also given for the
    slowest rank."""
    return cpp_step_block(torch, dev, world, rank, local, "vgg16_step", [])


def vgg16_block(args, cs, torch, dev, world, rank):
    """The swapped VGG16 training step (batch 128, 3x32x32 synthetic inputs,
    CSWAP+/vgg16-cifar10.cpp:135-245) on every rank at once: step time, link
    bytes and peak device memory without swapping, with raw swap of every
    kept activation, with the reference's hard-wired split, self-tuned, and
    with ZFP-8 on everything; then the activation bytes each of raw swap and
    compressed swap can move within a stated stretch of the no-swap step."""
    from cswap_b200 import workloads as W
    torch.manual_seed(1 + rank)
    batch = 128
    model = W.VGG16().to(dev).train()
    hx = torch.randn(batch, 3, 32, 32).pin_memory()
    hy = torch.randint(0, 10, (batch,)).pin_memory()
    mgr = cs.SwapManager(pinned_bytes=2 << 30, staging_bytes=512 << 20, zfp_maxbits=512)
    make_batch = lambda: (hx, hy)
    nids, steps, warmup = 64, 10, 3

    def fresh(policy_fn):
        exe = cs.Execution(mgr=mgr)
        exe.init_(nids)
        policy_fn(exe)
        return exe

    def every(pol):
        def f(exe):
            for i in range(nids):
                exe.begin_stage[i] = i + 1
                exe.policy[i] = pol
        return f

    rows = {}
    rows["no_swap"] = W.timed_steps(model, fresh(lambda e: None), make_batch, steps, warmup)
    rows["raw_swap"] = W.timed_steps(model, fresh(every(cs.POLICY_RAW)), make_batch, steps, warmup)
    rows["reference_split_zfp8"] = W.timed_steps(model, fresh(W.vgg16_reference_policy), make_batch, steps, warmup)
    rows["zfp8_everywhere"] = W.timed_steps(model, fresh(every(cs.POLICY_ZFP)), make_batch, steps, warmup)
    # self-tuned: profile one step, fit the cost model on this GPU with the other ranks busy too, decide
    exe = fresh(lambda e: None)
    exe.profile = True
    x, y = hx.to(dev).requires_grad_(True), hy.to(dev)
    model.forward_with(exe, x, y).backward()
    prof = exe.finish_profile()
    cm = cs.CostModel.fit(mgr, 512)
    cands = exe.policy_candidates(prof, cm)
    chosen = exe.refine_policy(cands, lambda k: W.timed_steps(model, exe, make_batch, k, 0)["ms_per_step"] * k * 1e-3)
    tuned_policy = list(exe.policy)
    rows["self_tuned"] = W.timed_steps(model, exe, make_batch, steps, warmup)
    t0 = rows["no_swap"]["ms_median"]
    eps_list = (0.1, 0.25, 0.5, 1.0)
    lossless = {tid: (cs.POLICY_SPARSE if p["zero_fraction"] >= 0.3 else cs.POLICY_RAW) for tid, p in prof.items()}
    mgr.keep_staged(False)  # strict for the sweeps: whatever comes back crosses the link again
    sweeps = {
        "raw": hidden_bytes_sweep(W, cs, torch, model, mgr, make_batch, prof, lambda tid: cs.POLICY_RAW, t0, eps_list),
        # the reference's rule for where loss is allowed: ZFP-8 on conv inputs, lossless elsewhere
        "compressed_reference_rule": hidden_bytes_sweep(
            W, cs, torch, model, mgr, make_batch, prof,
            lambda tid: cs.POLICY_ZFP if tid in W.VGG_CONV_INPUT_IDS else lossless.get(tid, cs.POLICY_RAW), t0,
            eps_list),
        "compressed_zfp8_everywhere": hidden_bytes_sweep(W, cs, torch, model, mgr, make_batch, prof,
                                                         lambda tid: cs.POLICY_ZFP, t0, eps_list),
    }
    ratios = {}
    for name in ("compressed_reference_rule", "compressed_zfp8_everywhere"):
        ratios[name] = {e: (sweeps[name]["hidden_activation_bytes"][e] / sweeps["raw"]["hidden_activation_bytes"][e]
                            if sweeps["raw"]["hidden_activation_bytes"][e] > 0 else None)
                        for e in sweeps["raw"]["hidden_activation_bytes"]}
    # the slowest rank's step time per row
    names = list(rows)
    worst = max_over_ranks([rows[k]["ms_median"] for k in names], dev)
    out = {"batch": batch, "ranks_running": world, "host_side": "python saved-tensor hooks (cswap_b200/execution.py)",
           "steps": steps, "warmup": warmup,
           "rows": {k: {"ms_per_step_median": rows[k]["ms_median"], "ms_per_step_median_slowest_rank": w,
                        "activation_bytes_swapped": rows[k]["activation_bytes_per_step"],
                        "link_bytes_out": rows[k]["link_bytes_out_per_step"],
                        "link_bytes_in": rows[k]["link_bytes_in_per_step"],
                        "peak_device_mib": round(rows[k]["peak_device_bytes"] / 2**20, 1)}
                    for k, w in zip(names, worst)},
           "self_tuned_policy_counts": {str(c): tuned_policy.count(c) for c in (0, 2, 3, 6)},
           "self_tuned_chosen": chosen,
           "hidden_activation_bytes": {
               "definition": "uncompressed activation bytes swapped out and back per step by the configuration "
                             "that swaps the most while the median step stays within (1 + eps) of the no-swap "
                             "step; candidates are the kept activations, largest first",
               "eps": list(eps_list), "no_swap_ms": t0,
               "per_policy": {k: v["hidden_activation_bytes"] for k, v in sweeps.items()},
               "ratio_to_raw": ratios, "target_ratio": 2.0,
               "curves": {k: v["curve"] for k, v in sweeps.items()}},
           "cost_model": cm.as_dict()}
    mgr.close()
    del model
    torch.cuda.empty_cache()
    return out


def main():
    args = parse()
    guard_stdout()
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

    # A second, longer region of the same step (at least half a second of device time), so that
    # the clock samples show what the step does to the clocks; the headline stays the K steps asked for.
    per_step = max(t_total / args.steps, 1e-6)
    long_steps = max(args.steps, int(0.6 / per_step) + 1)
    sampler.start()
    l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    l0.record()
    for _ in range(long_steps):
        cs.zfp_compress(x, maxbits, out=comp)
        cs.zfp_decompress(comp, n, maxbits, out=y)
        if flush is not None:
            flush.fill_(1)
    l1.record()
    torch.cuda.synchronize()
    sampler.stop()
    t_long = max_over_ranks([l0.elapsed_time(l1) * 1e-3], dev)[0]

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
    # DRAM read + write bytes of one launch, from an ncu capture of this exact workload
    # (256 MiB tensor, rate 8); unknown for other sizes / rates
    ncu_traffic = {("zfp_encode_slab_kernel", 256, 8): 320.7e6, ("zfp_decode_slab_kernel", 256, 8): 276.4e6}
    roofline = {"bound": "hbm", "kernel": name, "achieved": alg / t_k / 1e9, "peak": peak, "unit": "GB/s",
                "frac": alg / t_k / 1e9 / peak, "peak_kind": f"of {peak_kind}", "traffic": ncu_traffic.get((name, args.mib, args.rate)),
                "algorithmic_bytes_per_launch": alg,
                "encode": {"ms": t_enc * 1e3, "GBps_algorithmic": alg / t_enc / 1e9, "frac": alg / t_enc / 1e9 / peak},
                "decode": {"ms": t_dec * 1e3, "GBps_algorithmic": alg / t_dec / 1e9, "frac": alg / t_dec / 1e9 / peak},
                "roundtrip_frac": 2 * alg / (t_enc + t_dec) / 1e9 / peak}

    extra = {}
    if not args.no_extra:
        extra = side_measurements(cs, torch, dev, peak, world, args)
        extra["speedup_over_reference_cuda"] = against_reference_cuda(extra.get("reference_cuda"), t_enc, t_dec,
                                                                     extra["sparse"])
        # The two calls block, as the reference's do, so they cannot overlap each other: each is
        # bound by its larger direction (the field in, then the field out).  Against the measured
        # one-direction copy rates with every rank copying at once.
        lk = extra["link"]
        t_floor = max(4 * n / lk["h2d_GBps_per_gpu"], stream_bytes / lk["d2h_GBps_per_gpu"]) / 1e9 + \
            max(stream_bytes / lk["h2d_GBps_per_gpu"], 4 * n / lk["d2h_GBps_per_gpu"]) / 1e9
        e2e["link_floor_ms_per_step"] = t_floor * 1e3
        e2e["fraction_of_link_ceiling"] = t_floor / t_e2e
        if not args.no_vgg:
            extra["vgg16"] = vgg16_cpp_block(torch, dev, world, rank, local)
            extra["vgg16_python_engine"] = vgg16_block(args, cs, torch, dev, world, rank)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, cores, sample = cpu_codec_sample(args.mib, args.rate)
        cpu = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}

    clocks = sampler.summary()
    sustained = {"steps": long_steps, "seconds": t_long, "ms_per_step": t_long / long_steps * 1e3,
                 "value": whole_job_gbps(world, 2 * 4 * n, t_long / long_steps), "unit": "GB/s",
                 "ms_per_step_x_median_sm_mhz": (t_long / long_steps * 1e3 * clocks["sm_mhz"]) if clocks["sm_mhz"]
                 else None}
    if rank == 0:
        line = {
            "metric": "zfp_roundtrip_uncompressed_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32->i32/u64", "data": "synthetic",
            "config": workload_config(args), "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": 2 * args.steps, "clocks": clocks, "sustained": sustained, "extra": extra,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def link_ceiling(torch, dev, world):
    """What the host link gives a plain copy: pinned device-to-host only,
    host-to-device only and both directions at once, 256 MiB per copy by
    cudaMemcpyAsync, with every rank of the job starting behind one barrier -
    the ceiling for anything that swaps (the raw-swap copy of
    CSWAP+/Execution.h:70-85 run by all replicas at once).  GB/s per GPU is the
    slowest rank's; the job's aggregate is that times the rank count."""
    import torch.distributed as dist
    nbytes = 256 << 20
    d_a = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    d_b = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    h_a = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_b = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_b.copy_(d_a)  # both host buffers have been written before they are read
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def run(kind, reps=6):
        best = float("inf")
        for r in range(reps + 1):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            s1.wait_event(e0)
            s2.wait_event(e0)
            if kind in ("d2h", "both"):
                with torch.cuda.stream(s1):
                    h_a.copy_(d_a, non_blocking=True)
            if kind in ("h2d", "both"):
                with torch.cuda.stream(s2):
                    d_b.copy_(h_b, non_blocking=True)
            e1.record(s1)
            e2.record(s2)
            torch.cuda.synchronize()
            dt = max(e0.elapsed_time(e1), e0.elapsed_time(e2)) * 1e-3
            if r:
                best = min(best, dt)
        return max_over_ranks([best], dev)[0]

    t_out, t_in, t_both = run("d2h"), run("h2d"), run("both")
    return {"bytes_per_copy": nbytes, "ranks_copying": world,
            "d2h_GBps_per_gpu": nbytes / t_out / 1e9, "h2d_GBps_per_gpu": nbytes / t_in / 1e9,
            "both_GBps_per_gpu_each_way": nbytes / t_both / 1e9,
            "both_GBps_aggregate_both_ways": 2 * world * nbytes / t_both / 1e9}


def zfp_sweep(cs, torch, dev, peak, flush):
    """Encode and decode time of every point of the size sweep: 64 KiB .. 512 MiB
    (nx = ny = 32, nz scaled) x rates 4 / 8 / 16 x values N(0,1) and U[-1,1].
    L2 is flushed before every timed call; `frac` is algorithmic bytes
    (4N + N*rate/8) over time against the measured HBM peak."""
    rows = []

    def med(fn, reps):
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

    for dist_name in ("normal", "uniform"):
        g = torch.Generator(device=dev).manual_seed(99)
        big = torch.randn(512 * 262144, device=dev, generator=g) if dist_name == "normal" else \
            torch.rand(512 * 262144, device=dev, generator=g) * 2 - 1
        back = torch.empty_like(big)
        comp = torch.empty(cs.zfp_max_bytes(32, 32, big.numel() // 1024, 1024), dtype=torch.uint8, device=dev)
        kib = 64
        while kib <= 512 * 1024:
            n = kib * 256
            t = big[:n]
            reps = 7 if kib <= 65536 else 3
            for rate in (4, 8, 16):
                mb = 64 * rate
                te = med(lambda: cs.zfp_compress(t, mb, out=comp), reps)
                td = med(lambda: cs.zfp_decompress(comp, n, mb, out=back[:n]), reps)
                alg = 4 * n + n * rate // 8
                rows.append({"kib": kib, "rate": rate, "dist": dist_name, "encode_us": te * 1e6, "decode_us": td * 1e6,
                             "encode_GBps_uncompressed": 4 * n / te / 1e9, "decode_GBps_uncompressed": 4 * n / td / 1e9,
                             "encode_frac_hbm": alg / te / 1e9 / peak, "decode_frac_hbm": alg / td / 1e9 / peak})
            kib *= 2
        del big, back, comp
    return rows


def swap_trips(cs, torch, dev):
    """One tensor out to pinned host memory and back through the swap manager,
    per policy: raw, ZFP rate 8 and sparse at 50 / 75 / 90 % zeros (64 MiB
    tensor).  The trip waits for the copy out and gives the staging copy up
    before it asks for the tensor back, so every policy crosses the link in
    both directions; link bytes each way are the manager's own counters."""
    out = {}
    mgr = cs.SwapManager(pinned_bytes=512 << 20, staging_bytes=256 << 20)
    n = 64 * 262144
    g = torch.Generator(device=dev).manual_seed(5)
    dense = torch.tanh(torch.randn(n, device=dev, generator=g))
    dst = torch.empty_like(dense)
    cases = [("raw", cs.POLICY_RAW, dense), ("zfp8", cs.POLICY_ZFP, dense)]
    for zf, mu in ((50, 0.0), (75, -0.6745), (90, -1.2816)):
        cases.append((f"sparse_{zf}", cs.POLICY_SPARSE, torch.relu(torch.randn(n, device=dev, generator=g) + mu)))
        cases.append((f"raw_of_sparse_{zf}", cs.POLICY_RAW, cases[-1][2]))
    for name, pol, t in cases:
        def trip():
            tk = mgr.swap_out(t, pol)
            mgr.sync()             # the copy out has landed and the staging copy is given up
            mgr.swap_in(tk, out=dst)
            torch.cuda.synchronize()
            tk.release()
        trip()
        mgr.reset_stats()
        reps = 5
        t0 = time.perf_counter()
        for _ in range(reps):
            trip()
        dt = (time.perf_counter() - t0) / reps
        st = mgr.stats()
        exact = bool(torch.equal(dst.view(torch.int32), t.view(torch.int32)))
        out[name] = {"tensor_mib": 64, "out_plus_in_ms": dt * 1e3, "uncompressed_GBps": 2 * 4 * n / dt / 1e9,
                     "link_bytes_out": st["moved_bytes_out"] // reps, "link_bytes_in": st["moved_bytes_in"] // reps,
                     "link_GBps": (st["moved_bytes_out"] + st["moved_bytes_in"]) / reps / dt / 1e9,
                     "bit_exact": exact}
        if pol == cs.POLICY_SPARSE:
            # The sparse payload's size is only known on the device, so it leaves through a small copy
            # kernel that writes mapped pinned memory instead of the copy engine.  Its way out alone
            # (compress + copy), beside the copy engine moving the same number of bytes as a raw swap.
            def out_only(tensor, policy):
                best = float("inf")
                for _ in range(4):
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    tk = mgr.swap_out(tensor, policy)
                    mgr.sync()
                    best = min(best, time.perf_counter() - t0)
                    tk.release()
                return best
            link_bytes = st["moved_bytes_out"] // reps
            same = dense[:max(link_bytes // 4, 1)]
            t_sparse, t_engine = out_only(t, pol), out_only(same, cs.POLICY_RAW)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            packed, cnt = cs.sparse_compress(t, onepass=True)
            a.record()
            cs.sparse_compress(t, out=packed, nnz_out=cnt, onepass=True)
            b.record()
            torch.cuda.synchronize()
            t_codec = a.elapsed_time(b) * 1e-3
            out[name]["way_out"] = {"link_bytes": link_bytes, "compress_ms": t_codec * 1e3,
                                    "compress_plus_copy_kernel_ms": t_sparse * 1e3,
                                    "copy_kernel_GBps": link_bytes / max(t_sparse - t_codec, 1e-9) / 1e9,
                                    "copy_engine_same_bytes_ms": t_engine * 1e3,
                                    "copy_engine_GBps": link_bytes / t_engine / 1e9}
            del packed, cnt
    mgr.close()
    return out


def side_measurements(cs, torch, dev, peak, world=1, args=None):
    """Measurements reported beside the headline, not in it."""
    out = {"link": link_ceiling(torch, dev, world), "sparse": [], "swap": {}, "zfp_rates": []}
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
    out["zfp_sweep"] = zfp_sweep(cs, torch, dev, peak, flush)
    out["zfp_rates"] = [r for r in out["zfp_sweep"] if r["kib"] == 256 * 1024 and r["dist"] == "normal"]
    del flush
    out["swap"] = swap_trips(cs, torch, dev)
    try:
        out["reference_cuda"] = reference_cuda_times(args.mib if args else 256, args.rate if args else 8, dev)
    except Exception as err:  # the checker's build is optional
        out["reference_cuda"] = {"unavailable": repr(err)}
    return out


def against_reference_cuda(ref, t_enc, t_dec, sparse_rows):
    """This library's kernels over the reference's own on the same GPU and
    tensors (time ratios, > 1 means faster here)."""
    if not ref or "zfp" not in ref:
        return None
    z = ref["zfp"]
    out = {"zfp_encode": z["encode_ms"] * 1e-3 / t_enc, "zfp_decode": z["decode_ms"] * 1e-3 / t_dec,
           "zfp_roundtrip": (z["encode_ms"] + z["decode_ms"]) * 1e-3 / (t_enc + t_dec)}
    mine = {round(r["zero_fraction"], 1): r for r in sparse_rows if r["tensor_mib"] == 16}
    n = 16 * 262144
    for r in ref.get("sparse", []):
        m = mine.get(round(r["zero_fraction"], 1))
        if m:
            key = f"sparse_{int(r['zero_fraction'] * 100)}"
            out[key + "_compress"] = r["compress_ms"] * 1e-3 / (4 * n / m["onepass_compress_GBps_uncompressed"] / 1e9)
            out[key + "_decompress"] = r["decompress_ms"] * 1e-3 / (4 * n / m["decompress_GBps_uncompressed"] / 1e9)
    return out


if __name__ == "__main__":
    main()
