#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

Workload (config 5 of the baseline: the one the metric is quoted on): FP8 E4M3 Linear, K = 8192, N = 28672,
weights N(0, 0.02) quantised per tensor, activations N(0, 1).  One "step" is one decode-shaped (M = 1) linear
call over the whole weight; `value` is the algorithmic HBM GB/s of that step with everything resident in HBM.
The dense M = 4096 TFLOP/s figure of the same metric, the INT8 variants and the decode sweep are reported in
`extra`, measured outside the timed steps.  Two weight sets (2 x 235 MB > 126 MB of L2) are rotated so no
step finds its weights in L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 (under torchrun): the weight is column-sharded across the ranks, each rank computes its slice and one
NCCL all-gather assembles the 1-byte outputs (strong scaling: total work is fixed).
`--impl reference` times the reference's own x86 kernel for the same configuration on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K, N = 8192, 28672
L2_BYTES = 126 * 1024 * 1024
SEED = 0xFEA70005
METRIC = "quant Linear HBM GB/s at M=1 & TFLOP/s at M=4096 (% B200 peak), 1/2/4/8 GPU"


def measured_peaks():
    """HBM GB/s and dense bf16 TFLOP/s measured on this pool (MEASURED_PEAKS.json), else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def e4m3_codes_torch(torch, x, scale):
    """float32 tensor → E4M3 codes (uint8 view) through torch's own float8 cast (synthetic-data plumbing)."""
    return (x / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons through NVML while the timed regions run (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag = index, [], set(), False
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in names.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def synth(torch, shape, std, seed, device):
    """Seeded N(0, std) tensor quantised to E4M3 with an absmax per-tensor scale → (codes uint8, scale)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std
    scale = float(x.abs().max().item() / 448.0)
    return e4m3_codes_torch(torch, x, scale), scale


def event_time_ms(torch, fn, steps, warmup, barrier=None):
    """W untimed warm-up calls, then exactly `steps` calls between two CUDA events on the launching stream,
    with a barrier + synchronize on both sides.  Returns total milliseconds."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1)


def algorithmic_bytes(m, n, per_channel=False):
    """Minimum bytes one linear call must move: weights + activations + outputs (+ channel scales)."""
    return K * n + m * K + m * n + (4 * n if per_channel else 0)


# ------------------------------------------------------------------------------------------------------------
# reference arm: the reference's own x86 kernel on the host cores
# ------------------------------------------------------------------------------------------------------------
def cpu_reference_kernel(torch, m=1):
    """(kernel handle, description) of the reference x86 FP8 Linear on the C5 weight: the unmodified reference
    library when it was built here (kind "reference"), else this repo's C restatement (kind "port")."""
    import oracle as O
    w, sw = synth(torch, (K, N), 0.02, SEED, "cpu")
    a, sa = synth(torch, (m, K), 1.0, SEED + 1, "cpu")
    w, a = w.numpy(), a.numpy()
    so = float(np.float32(0.02 * np.sqrt(K) * 4.0 / 448.0))
    if O.have_ref():
        kern = O.fp8_linear(O.OP_MATMUL, O.E4M3, a, sa, w, sw, so, impl="ref", device=O.X86, return_kernel=True)
        t0 = time.time()
        if kern.prepare() != 0:
            raise RuntimeError("reference Prepare() failed")
        prep = time.time() - t0
        threads = min(4, os.cpu_count() or 1)  # src/kernel/x86/linear_fp8.cc:45-70 caps FP8 at 4 OpenMP threads
        return (lambda reps: kern.time_compute(reps)), dict(kind="reference", cores=threads, prepare_s=round(prep, 2))
    threads = os.cpu_count() or 1

    def run(reps):
        best = 1e9
        for _ in range(reps):
            t0 = time.time()
            O.fp8_linear(O.OP_MATMUL, O.E4M3, a, sa, w, sw, so)
            best = min(best, time.time() - t0)
        return best
    return run, dict(kind="port", cores=threads, prepare_s=0.0)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the reference kernel should have the host cores it can use
    # (its own cap is 4 threads for this path), so the variable is lifted before any OpenMP runtime is loaded
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import torch
    run, info = cpu_reference_kernel(torch, 1)
    for _ in range(max(args.warmup, 1)):
        run(1)
    t0 = time.time()
    for _ in range(args.steps):
        run(1)
    total = time.time() - t0
    ms = total / args.steps * 1e3
    gbs = algorithmic_bytes(1, N) / (ms * 1e-3) / 1e9
    sample = f"full C5 M=1 FP8-E4M3 weight ({K}x{N}) per step, {args.steps} steps; Prepare() {info['prepare_s']} s once, untimed"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"C5 FP8-E4M3 Linear M=1 K={K} N={N}", "host_cpus": os.cpu_count()},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": info["cores"], "kind": info["kind"], "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import infer_b200 as B
    from infer_b200.sharded import ShardedLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    barrier = (lambda: dist.barrier()) if dist else None
    dev = torch.device("cuda", local_rank)
    B.lib()  # fails loudly if the CUDA library is missing
    peaks = measured_peaks()
    stream = B.current_stream()
    fp8_call = B.lib().fth_b200_fp8_linear
    int8_call = B.lib().fth_b200_int8_linear

    # ---- this rank's column shard of two weight sets (rotated so steps never hit L2-resident weights) ----
    shard = ShardedLinear(N, world, rank, compute=None, dist=dist)
    n0, n1 = shard.n0, shard.n1
    n_local, width = n1 - n0, shard.width
    out_scale = float(np.float32(0.02 * np.sqrt(K) * 4.0 / 448.0))
    # enough weight sets that one rotation moves at least twice the L2 capacity through the GPU (a 29 MB shard
    # on 8 GPUs needs 9 of them; the full 235 MB weight needs 2)
    n_sets = max(2, -(-2 * L2_BYTES // (K * n_local)))
    weights, w_scales = [], []
    for i in range(n_sets):
        if world == 1:
            w_part, sw = synth(torch, (K, N), 0.02, SEED + 10 * i, dev)
        else:  # this rank's columns of weight set i, drawn directly (the same distribution; no 235 MB detour per set)
            w_part, sw = synth(torch, (K, n_local), 0.02, SEED + 10 * i + 1000 * (rank + 1), dev)
        weights.append(w_part.contiguous())
        w_scales.append(sw)
        del w_part
    a_dev, sa = synth(torch, (1, K), 1.0, SEED + 1, dev)
    local_out = torch.zeros((1, width), dtype=torch.uint8, device=dev)

    def make_desc(m, w, sw, a, out, ldo=0):
        d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=K, n=w.shape[1], a=a, w=w, out=out, a_scale=sa,
                              w_scale=sw, out_scale=out_scale, ldo=ldo, weights_static=True)
        ws = B.linear_workspace(torch, d)
        return d, ws

    descs = [make_desc(1, weights[i], w_scales[i], a_dev, local_out, ldo=width) for i in range(n_sets)]
    counter = [0]

    # N > 1: every rank's kernel stores its columns into all ranks' output buffers (peer-mapped) and a signal / wait
    # kernel ends the step; no collective library on the data path.
    gather = None
    if world > 1:
        from infer_b200.sharded import PeerGather, ShardedLinear, forward_peer
        from infer_b200.sharded import point_at_step_buffers
        shard = ShardedLinear(N, world, rank, compute=None, dist=dist)
        call_desc = lambda desc, s: fp8_call(C.byref(desc), s)  # noqa: E731
        try:
            gather = PeerGather(B.lib(), dist, world, rank, 1, N)  # raises on every rank or on none
            # per weight set, one descriptor per step parity, pointed at that parity's buffers once
            prepared = [tuple(point_at_step_buffers(shard, gather, type(d).from_buffer_copy(d), parity) for parity in (0, 1)) for d, _ in descs]
        except RuntimeError as exc:
            # no peer mapping on this box: the gather falls back to one NCCL all-gather of the 1-byte outputs
            gather = None
            if rank == 0:
                print(f"[bench] {exc}; using NCCL all_gather_into_tensor", file=sys.stderr)
    nccl_gathered = torch.zeros((world, width), dtype=torch.uint8, device=dev) if world > 1 and gather is None else None

    def step():
        i = counter[0] % n_sets
        counter[0] += 1
        if gather is not None:
            forward_peer(shard, gather, descs[i][0], call_desc, stream, prepared[i])
            return
        rc = fp8_call(C.byref(descs[i][0]), stream)
        if rc != 0:
            raise RuntimeError(f"fth_b200_fp8_linear failed: {rc}")
        if world > 1:
            dist.all_gather_into_tensor(nccl_gathered, local_out)

    # N > 1: a sharded step is a few microseconds of GPU time, less than the host needs to issue it, so the steps are
    # replayed from a CUDA graph of one full rotation (every weight set, both buffer parities); the gather's step
    # numbers live on the device for that.  Steps that do not fill a whole rotation are issued one by one.
    timed_step, steps_per_call = step, 1
    if gather is not None:
        rotation = n_sets * (2 if n_sets % 2 else 1)  # an even number of steps: the buffer parity repeats
        for _ in range(rotation):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        main_stream = stream
        epoch_before, counter_before = gather.epoch, counter[0]
        captured = True
        try:
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                    for _ in range(rotation):
                        step()
        except Exception as exc:  # capture is an optimisation of the issue rate, never a requirement
            captured = False
            gather.epoch, counter[0] = epoch_before, counter_before
            print(f"[bench] rank {rank}: CUDA-graph capture failed ({type(exc).__name__}: {exc}); issuing steps one by one", file=sys.stderr)
        stream = main_stream
        verdict = torch.tensor([1 if captured else 0], device=dev)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)  # all ranks replay, or none does
        if int(verdict.item()) == 1:
            # the capture ran the host-side counters forward without running a step: put them back
            gather.epoch, counter[0] = epoch_before, counter_before

            def replay():
                graph.replay()
                gather.epoch += rotation
                counter[0] += rotation
            timed_step, steps_per_call = replay, rotation

    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- timed region: exactly K steps, device-timed, max over ranks ----
    B.lib().fth_b200_reset_launch_count()
    if steps_per_call == 1:
        total_ms = event_time_ms(torch, step, args.steps, args.warmup, barrier)
        launches_total = B.lib().fth_b200_launch_count()
        launches = launches_total * args.steps // (args.steps + args.warmup)
    else:
        calls, rest = divmod(args.steps, steps_per_call)
        B.lib().fth_b200_reset_launch_count()
        step()
        per_step_launches = B.lib().fth_b200_launch_count()  # kernels one step launches (counted outside the graph)
        step_odd = gather.epoch & 1
        if step_odd:
            step()  # keep the parity the graph was captured with

        def timed_block():
            for _ in range(calls):
                timed_step()
            for _ in range(rest):
                step()
        # warm-up: W steps one by one, then the timed block once: exactly K steps between the events
        for _ in range(args.warmup + (args.warmup & 1)):
            step()
        total_ms = event_time_ms(torch, timed_block, 1, 0, barrier)
        launches = per_step_launches * args.steps
    variant = B.last_variant()
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    bytes_step = algorithmic_bytes(1, N)
    value = bytes_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer plan API: H2D of the activation, launch, D2H of the result ----
    a_host = torch.empty((1, K), dtype=torch.uint8).pin_memory()
    a_host.copy_(a_dev.cpu())
    out_host = torch.empty((1, width), dtype=torch.uint8).pin_memory()
    plans = []
    for i in range(2 if world == 1 else 0):
        hd = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=1, k=K, n=n_local, a=None, w=None, out=None, a_scale=sa,
                               w_scale=w_scales[i], out_scale=out_scale, ldo=width)
        w_host = weights[i].cpu()
        hd.w = w_host.data_ptr()
        plans.append(B.Plan(hd))
        del w_host
    pc = [0]

    a_stage = torch.empty((1, K), dtype=torch.uint8, device=dev)
    full_host = torch.empty((1, N), dtype=torch.uint8).pin_memory()
    e2e_descs = [make_desc(1, weights[i], w_scales[i], a_stage, local_out, ldo=width) for i in range(n_sets)] if world > 1 else []

    def e2e_step():
        if world == 1:
            plans[pc[0] & 1].run(a_host, out_host, stream)
            pc[0] += 1
            return
        # N > 1: pinned-host activation in, sharded kernels with peer stores, the gathered row back to the host
        a_stage.copy_(a_host, non_blocking=True)
        d, _ = e2e_descs[pc[0] % n_sets]
        pc[0] += 1
        if gather is not None:
            parity = forward_peer(shard, gather, d, call_desc, stream)
            full_host.copy_(gather.view(torch, parity), non_blocking=True)
        else:
            if fp8_call(C.byref(d), stream) != 0:
                raise RuntimeError("fth_b200_fp8_linear failed")
            dist.all_gather_into_tensor(nccl_gathered, local_out)
            full_host.copy_(nccl_gathered.view(1, -1)[:, :N], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(args.steps, 500)
    e2e_ms = event_time_ms(torch, e2e_step, e2e_steps, max(args.warmup, 3), barrier) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = bytes_step / (e2e_ms * 1e-3) / 1e9
    for p in plans:
        p.close()

    extra = {}
    cpu_baseline = None
    if rank == 0 and not args.quick:
        extra = extra_measurements(torch, B, dev, peaks, fp8_call, int8_call, stream, sa, out_scale, weights[0], w_scales[0])
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    if rank == 0 and world == 1:
        cpu_baseline = cpu_baseline_measurement(torch)

    if rank == 0:
        achieved = value if world == 1 else value / world
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"C5 FP8-E4M3 Linear M=1 K={K} N={N}" + ((f", N column-sharded over {world} GPUs, " + ("outputs stored to all ranks over NVLink (peer stores + flag wait)" if gather is not None else "NCCL all-gather")) if world > 1 else ""),
                       "l2": f"inputs larger than L2: {n_sets} weight sets of {K * n_local / 1e6:.0f} MB rotated", "kernel": variant,
                       "algorithmic_bytes_per_step": bytes_step, "seed": SEED},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
                         "peak_source": peaks["source"], "note": "per GPU; step = tcgen05 GEMV + split-K reduce kernel"},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": K, "d2h_bytes_per_step": width if world == 1 else N,
                    "ms_per_step": round(e2e_ms, 5),
                    "api": "fth_b200_plan_run (pinned host activation in, host result out)" if world == 1 else
                           "pinned host activation in, fth_b200_fp8_linear with peer stores + fth_b200_gather_sync, gathered row out"},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
            "cpu_baseline": cpu_baseline,
            "extra": extra,
        }
        print(json.dumps(line))
    if dist:
        dist.barrier()
        if gather is not None:
            gather.close()
        dist.destroy_process_group()
    return 0


# dram__bytes_read.sum + dram__bytes_write.sum of one tcgen05 GEMV launch on the bench workload, from the ncu
# capture summarised in profiles/ (per launch, bytes).
TRAFFIC_BYTES_PER_LAUNCH = 239648512


def extra_measurements(torch, B, dev, peaks, fp8_call, int8_call, stream, sa, out_scale, w, sw):
    """The rest of the metric on one GPU, outside the timed steps: decode sweep and dense M=4096, FP8 and INT8."""
    out = {}
    n = w.shape[1]
    w_i8 = w.view(torch.int8)
    scales = torch.empty(n, dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2)
    w2 = torch.roll(w, 1, 0)  # a second weight set for the rotation
    for kind in ("fp8_e4m3", "int8"):
        for m in (1, 16, 256, 4096):
            if kind == "fp8_e4m3":
                a = torch.randint(0, 0x7E, (m, K), dtype=torch.uint8, device=dev)
                o = torch.empty((m, n), dtype=torch.uint8, device=dev)
                ds = [B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=m, k=K, n=n, a=a, w=ww, out=o, a_scale=sa, w_scale=sw,
                                        out_scale=out_scale * 4, weights_static=True) for ww in (w, w2)]
                call = fp8_call
            else:
                a = torch.randint(-127, 128, (m, K), dtype=torch.int8, device=dev)
                o = torch.empty((m, n), dtype=torch.int8, device=dev)
                ds = [B.int8_linear_desc(op=B.OP_MATMUL, m=m, k=K, n=n, a=a, w=ww.view(torch.int8), out=o, a_scale=0.02, a_zp=0,
                                         w_scales=scales, w_zps=None, w_params=n, out_scale=2.0, out_zp=0, weights_static=True)
                      for ww in (w, w2)]
                call = int8_call
            keep = [B.linear_workspace(torch, d) for d in ds]
            i = [0]

            def fn():
                rc = call(C.byref(ds[i[0] & 1]), stream)
                i[0] += 1
                if rc != 0:
                    raise RuntimeError(f"linear call failed: {rc}")
            iters = 200 if m <= 256 else 20
            ms = event_time_ms(torch, fn, iters, 3) / iters
            gbs = algorithmic_bytes(m, n, kind == "int8") / (ms * 1e-3) / 1e9
            tfl = 2.0 * m * K * n / (ms * 1e-3) / 1e12
            out[f"{kind}_m{m}"] = {"us": round(ms * 1e3, 2), "GB/s": round(gbs, 1), "TFLOP/s": round(tfl, 2),
                                   "hbm_frac": round(gbs / peaks["hbm_gbs"], 3),
                                   "tensor_frac": round(tfl / (2.0 * peaks["bf16_tflops"]), 3), "kernel": B.last_variant()}
            del keep
    out["config4_decode_step"] = config4_decode_step(torch, B, dev, fp8_call, stream)
    out["config3_conv"] = config3_conv(torch, B, dev, stream)
    out["peaks"] = {"hbm_gbs": peaks["hbm_gbs"], "fp8_int8_dense_tflops": 2.0 * peaks["bf16_tflops"],
                    "note": "8-bit dense peak taken as twice the measured bf16 burst figure", "source": peaks["source"]}
    return out


def config4_decode_step(torch, B, dev, fp8_call, stream):
    """Config 4: the 168 projections of a 24-layer decode step (hidden 1024, intermediate 3584, FP8 E5M2, BF16 in and
    out — Cast -> MatMul -> Cast fused per projection), replayed as one CUDA graph.  Synthetic weights and inputs."""
    hidden, inter, layers = 1024, 3584, 24
    shapes = [(hidden, hidden)] * 4 + [(hidden, inter), (hidden, inter), (inter, hidden)]
    result = {}
    for m in (1, 16):
        descs, keep = [], []
        for _ in range(layers):
            for k, n in shapes:
                w = torch.randint(0, 120, (k, n), dtype=torch.uint8, device=dev)
                a = torch.randn((m, k), device=dev).to(torch.bfloat16)
                o = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
                d = B.fp8_linear_desc(dtype=B.E5M2, op=B.OP_MATMUL, m=m, k=k, n=n, a=a, w=w, out=o, a_scale=2.0 ** -9, w_scale=2.0 ** -20,
                                      out_scale=2.0 ** -9, a_dtype=B.BF16, out_dtype=B.BF16, weights_static=True)
                keep += [w, a, o, B.linear_workspace(torch, d)]
                descs.append(d)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            s2 = C.c_void_p(side.cuda_stream)
            for d in descs:
                fp8_call(C.byref(d), s2)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for d in descs:
                    if fp8_call(C.byref(d), C.c_void_p(torch.cuda.current_stream().cuda_stream)) != 0:
                        raise RuntimeError("linear call failed during capture")
        ms = event_time_ms(torch, graph.replay, 20, 3) / 20
        wbytes = layers * sum(k * n for k, n in shapes)
        result[f"m{m}"] = {"us": round(ms * 1e3, 1), "projections": len(descs), "weight_GB/s": round(wbytes / (ms * 1e-3) / 1e9, 1),
                           "kernel": B.last_variant()}
        del keep, graph
    return result


def config3_conv(torch, B, dev, stream):
    """Config 3: INT8 3x3 conv 1x64x160x160 (*) 64x64x3x3, pad 1, per-channel scales, int32 bias, fused ReLU table."""
    x = torch.randint(-128, 128, (1, 64, 160, 160), dtype=torch.int8, device=dev)
    w = torch.randint(-128, 128, (64, 64, 3, 3), dtype=torch.int8, device=dev)
    bias = torch.randint(-(1 << 15), 1 << 15, (64,), dtype=torch.int32, device=dev)
    ws = torch.empty(64, dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2)
    out = torch.empty((1, 64, 160, 160), dtype=torch.int8, device=dev)
    so = 0.4
    lut = torch.from_numpy(B.int8_relu_table(so, 0, so, 0)).to(dev)
    d = B.int8_conv2d_desc(batch=1, ic=64, ih=160, iw=160, oc=64, kh=3, kw=3, x=x, w=w, out=out, x_scale=0.02, x_zp=0, w_scales=ws, w_zps=None,
                           w_params=64, out_scale=so, out_zp=0, bias=bias, relu_lut=lut, bias_max_abs=1 << 15)
    need = B.lib().fth_b200_int8_conv2d_workspace_bytes(C.byref(d))
    wsb = torch.empty(max(int(need), 16), dtype=torch.uint8, device=dev)
    d.workspace, d.workspace_bytes = wsb.data_ptr(), need
    call = B.lib().fth_b200_int8_conv2d

    def fn():
        if call(C.byref(d), stream) != 0:
            raise RuntimeError("conv call failed")
        d.weights_packed = 1
    fn()
    ms = event_time_ms(torch, fn, 100, 3) / 100
    return {"us": round(ms * 1e3, 2), "TOP/s": round(2.0 * 160 * 160 * 64 * 576 / (ms * 1e-3) / 1e12, 1), "kernel": B.last_variant()}


def cpu_baseline_measurement(torch):
    """The reference's x86 kernel for the same workload on this box's host cores (a reported baseline)."""
    try:
        run, info = cpu_reference_kernel(torch, 1)
        run(1)
        reps = 10 if info["kind"] == "reference" else 2
        best = run(reps)
        gbs = algorithmic_bytes(1, N) / best / 1e9
        return {"value": round(gbs, 3), "unit": "GB/s", "cores": info["cores"], "kind": info["kind"],
                "sample": f"full C5 M=1 weight ({K}x{N}), best of {reps} compute() calls after Prepare() ({info['prepare_s']} s, untimed); "
                          f"host has {os.cpu_count()} CPUs", "ms": round(best * 1e3, 3)}
    except Exception as exc:  # the baseline is reported, never required
        return {"value": None, "unit": "GB/s", "cores": 0, "kind": "unavailable", "sample": f"{type(exc).__name__}: {exc}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--quick", action="store_true", help="skip the extra sweep (decode / dense / INT8)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        args.quick = True
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
