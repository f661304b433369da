#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

Workload (config 5 of the baseline: the one the metric is quoted on): FP8 E4M3 Linear, K = 8192, N = 28672,
weights N(0, 0.02) quantised per tensor, activations N(0, 1).  One "step" is one decode-shaped (M = 1) linear
call over the whole weight; `value` is the algorithmic HBM GB/s of that step with everything resident in HBM.
The K timed steps are run as a block, the block is repeated (`blocks` in the JSON line) and the median block is
reported, so that the clock ramp of a GPU that was idle a moment ago does not set the number.  Enough weight sets
are rotated that no step finds its weights in L2.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--quick]

N > 1 (under torchrun): the weight is column-sharded across the ranks; every rank's kernel stores its columns into
all ranks' output buffers over NVLink (peer stores from the epilogue) and a small signal / wait kernel ends the step
(strong scaling: total work is fixed).  There is no collective library on the data path; NCCL is used for set-up
and is the fallback gather on a box without peer mapping.

Checks outside the timed regions (any failure makes the run exit non-zero):
  * N = 1: the output row of the timed kernel is compared with the CPU oracle (`parity` in the JSON line);
  * N > 1: with one seeded weight shared by all ranks, every rank compares the gathered [M, N] result with the
    result of its own single-GPU run (`gather_mismatch_bytes`), FP8 and INT8;
  * every rank reads the device status word after the timed and the end-to-end regions (`device_status`).

`extra` carries the rest of the metric: FP8 and INT8 at M = 1, 16, 256, 4096 (at N > 1 on the column shards, step
time including the gather), the config-4 decode step, the config-3 conv, and the reference's x86 kernels timed on
the host cores for configs 2, 3, 4 and 5-INT8.  `--impl reference` times the reference's own x86 kernel for the
headline configuration on the host cores.
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
WORKLOAD = f"C5 FP8-E4M3 Linear M=1 K={K} N={N}"
BLOCKS = 7
# dram__bytes_read.sum + dram__bytes_write.sum of one tcgen05 GEMV launch on the bench workload, from the ncu
# capture summarised in profiles/ (per launch, bytes).
TRAFFIC_BYTES_PER_LAUNCH = 239427328


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


def synth_int8(torch, shape, seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randint(-127, 128, shape, generator=g, device=device, dtype=torch.int8)


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


FP8_OUT_SCALE = float(np.float32(0.02 * np.sqrt(K) * 4.0 / 448.0))


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
    so = FP8_OUT_SCALE
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


def bench_config(world, extra=None):
    """`config` of the JSON line; both arms carry the same keys."""
    cfg = {"workload": WORKLOAD, "gpus": world, "host_cpus": os.cpu_count(), "seed": SEED, "algorithmic_bytes_per_step": algorithmic_bytes(1, N),
           "sharding": None, "l2": None, "kernel": None}
    if extra:
        cfg.update(extra)
    return cfg


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
        "config": bench_config(args.gpus, {"kernel": "reference x86 MatMulKernel<X86,FP8E4M3> (packed BF16 GEMV)"}),
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": info["cores"], "kind": info["kind"], "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------
class Ctx:
    """What every measured case needs: torch, the library, this rank's place in the job and its column shard."""

    def __init__(self, torch, B, dist, world, rank, dev):
        from infer_b200.sharded import ShardedLinear
        self.torch, self.B, self.dist, self.world, self.rank, self.dev = torch, B, dist, world, rank, dev
        self.local_rank = dev.index or 0
        self.shard = ShardedLinear(N, world, rank, compute=None, dist=dist)
        self.n0, self.n1 = self.shard.n0, self.shard.n1
        self.n_local = self.n1 - self.n0
        self.stream = B.current_stream()
        self.fp8_call = B.lib().fth_b200_fp8_linear
        self.int8_call = B.lib().fth_b200_int8_linear
        self.peer_ok = world > 1  # cleared on the first failure to map peer buffers

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max_over_ranks(self, value):
        if not self.dist:
            return value
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, value):
        if not self.dist:
            return value
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.int64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return int(t.item())


class LinearCase:
    """One (kind, M) linear over this rank's columns of the C5 weight, with rotating weight sets.

    world == 1: the kernel writes a local [M, N] buffer.  world > 1: the output goes to every rank's [M, N] buffer
    (peer stores) and fth_b200_gather_sync ends the step; steps are replayed from a CUDA graph of one rotation
    because a sharded decode step is less GPU time than the host needs to issue it.  Without peer mapping the
    gather is one NCCL all-gather of the 1-byte outputs."""

    def __init__(self, ctx, kind, m, weights=None, seed=SEED, rotate_bytes=2 * L2_BYTES, use_graph=None, graph_steps=None):
        torch, B = ctx.torch, ctx.B
        self.ctx, self.kind, self.m = ctx, kind, m
        self.int8 = kind == "int8"
        n_local = ctx.n_local
        if weights is None:
            n_sets = max(2, -(-rotate_bytes // (K * n_local)))
            weights = []
            for i in range(n_sets):
                if self.int8:
                    weights.append((synth_int8(torch, (K, n_local), seed + 10 * i + 1000 * (ctx.rank + 1), ctx.dev), None))
                elif ctx.world == 1:
                    weights.append(synth(torch, (K, N), 0.02, seed + 10 * i, ctx.dev))
                else:  # this rank's columns of weight set i, drawn directly (same distribution; no 235 MB detour per set)
                    weights.append(synth(torch, (K, n_local), 0.02, seed + 10 * i + 1000 * (ctx.rank + 1), ctx.dev))
        self.weights = weights
        self.n_sets = len(weights)
        if self.int8:
            g = torch.Generator(device=ctx.dev)
            g.manual_seed(seed + 77)
            full_scales = torch.empty(N, dtype=torch.float32, device=ctx.dev).uniform_(1e-3, 1e-2, generator=g)
            self.scales = full_scales[ctx.n0:ctx.n1].contiguous()
            self.a = synth_int8(torch, (m, K), seed + 1, ctx.dev)
            self.sa = 0.02
            sigma = 73.3 ** 2 * np.sqrt(K) * self.sa * 5.5e-3
            self.so = float(np.float32(2.33 * sigma / 127.0))
        else:
            self.a, self.sa = synth(torch, (m, K), 1.0, seed + 1, ctx.dev)
            self.so = FP8_OUT_SCALE
        self.call = ctx.int8_call if self.int8 else ctx.fp8_call
        self.local_out = torch.zeros((m, N if ctx.world > 1 else n_local), dtype=torch.uint8, device=ctx.dev)
        self.keep = []
        self.descs = [self._desc(w, sw, self.a, self.local_out, ldo=self.local_out.shape[1]) for (w, sw) in weights]
        self.counter = 0
        self.gather = None
        self.graph = None
        self.graph_is_block = False
        self.rotation = 0
        self.stream = ctx.stream
        self.nccl_gathered = None
        if ctx.world > 1:
            self._setup_gather()
            if self.gather is not None and (use_graph if use_graph is not None else True):
                self._capture(graph_steps)

    # ---- descriptors ----
    def _desc(self, w, sw, a, out, ldo=0):
        B, torch = self.ctx.B, self.ctx.torch
        n = w.shape[1]
        if self.int8:
            d = B.int8_linear_desc(op=B.OP_MATMUL, m=self.m, k=K, n=n, a=a, w=w, out=out, a_scale=self.sa, a_zp=0, w_scales=self.scales,
                                   w_zps=None, w_params=n, out_scale=self.so, out_zp=0, ldo=ldo, weights_static=True)
        else:
            d = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=self.m, k=K, n=n, a=a, w=w, out=out, a_scale=self.sa,
                                  w_scale=sw, out_scale=self.so, ldo=ldo, weights_static=True)
        self.keep.append(B.linear_workspace(torch, d))
        return d

    def _call_desc(self, desc, stream):
        return self.call(C.byref(desc), stream)

    def _setup_gather(self):
        from infer_b200.sharded import PeerGather, forward_peer, point_at_step_buffers
        self._forward_peer = forward_peer
        ctx = self.ctx
        if ctx.peer_ok:
            try:
                # symmetric memory first (it brings an NVLink multicast address where the box has NVLS), CUDA IPC otherwise;
                # FTH_B200_NO_MULTICAST=1 keeps to the IPC buffers (A/B).  Raises on every rank or on none.
                self.gather = PeerGather(ctx.B.lib(), ctx.dist, ctx.world, ctx.rank, self.m, N,
                                         torch=None if os.environ.get("FTH_B200_NO_MULTICAST") == "1" else ctx.torch)
                if ctx.rank == 0 and not getattr(ctx, "gather_reported", False):
                    ctx.gather_reported = True
                    print(f"[bench] gather buffers: {'torch symmetric memory' if self.gather._symmetric is not None else 'CUDA IPC'}, "
                          f"NVLink multicast address {'present' if self.gather.multicast else 'absent'}", file=sys.stderr)
                # the kernels do the step signalling themselves (gather_world in the descriptors): no extra launch per step
                self.prepared = [tuple(point_at_step_buffers(ctx.shard, self.gather, type(d).from_buffer_copy(d), parity, fold_signal=True)
                                       for parity in (0, 1)) for d in self.descs]
                return
            except RuntimeError as exc:
                ctx.peer_ok = False
                self.gather = None
                if ctx.rank == 0:
                    print(f"[bench] {exc}; using NCCL all_gather_into_tensor", file=sys.stderr)
        # fallback: local [M, width] block, one NCCL all-gather (row-major only for M = 1)
        torch = ctx.torch
        self.local_out = torch.zeros((self.m, ctx.shard.width), dtype=torch.uint8, device=ctx.dev)
        self.keep = []
        self.descs = [self._desc(w, sw, self.a, self.local_out, ldo=ctx.shard.width) for (w, sw) in self.weights]
        self.nccl_gathered = torch.zeros((ctx.world, self.m, ctx.shard.width), dtype=torch.uint8, device=ctx.dev)

    # ---- one step ----
    def step(self):
        i = self.counter % self.n_sets
        self.counter += 1
        if self.gather is not None:
            self._forward_peer(self.ctx.shard, self.gather, self.descs[i], self._call_desc, self.stream, self.prepared[i], fold_signal=True)
            return
        rc = self.call(C.byref(self.descs[i]), self.stream)
        if rc != 0:
            raise RuntimeError(f"linear call failed: {rc}")
        if self.nccl_gathered is not None:
            self.ctx.dist.all_gather_into_tensor(self.nccl_gathered.view(self.ctx.world * self.m, -1), self.local_out)

    def result(self):
        """The [M, N] (world > 1) or [M, n_local] output of the last step, as a device tensor."""
        torch = self.ctx.torch
        if self.gather is not None:
            self.gather.wait(self.stream)  # the other ranks' columns of the last step
            torch.cuda.synchronize()
            return self.gather.view(torch, self.gather.epoch & 1)
        torch.cuda.synchronize()
        if self.nccl_gathered is not None:
            return self.nccl_gathered.transpose(0, 1).reshape(self.m, -1)[:, :N]
        return self.local_out

    # ---- CUDA graph of one rotation (every weight set, both buffer parities) ----
    def _capture(self, graph_steps=None):
        ctx, torch, gather = self.ctx, self.ctx.torch, self.gather
        rotation = self.n_sets * (2 if self.n_sets % 2 else 1)  # an even number of steps: the buffer parity repeats
        # A timed block of a known, even length that visits every weight set is recorded whole, its closing wait for the
        # other ranks included: the block is then one graph launch, with no step issued from the host behind it.
        self.graph_is_block = bool(graph_steps) and graph_steps % 2 == 0 and graph_steps >= self.n_sets
        if self.graph_is_block:
            rotation = graph_steps
        for _ in range(rotation):
            self.step()
        torch.cuda.synchronize()
        ctx.barrier()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        epoch_before, counter_before = gather.epoch, self.counter
        captured = True
        try:
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    self.stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                    for _ in range(rotation):
                        self.step()
                    if self.graph_is_block:
                        gather.wait(self.stream)
        except Exception as exc:  # capture is an optimisation of the issue rate, never a requirement
            captured = False
            print(f"[bench] rank {ctx.rank}: CUDA-graph capture failed ({type(exc).__name__}: {exc}); issuing steps one by one", file=sys.stderr)
        self.stream = ctx.stream
        # the capture ran the host-side counters forward without running a step: put them back
        gather.epoch, self.counter = epoch_before, counter_before
        verdict = torch.tensor([1 if captured else 0], device=ctx.dev)
        ctx.dist.all_reduce(verdict, op=ctx.dist.ReduceOp.MIN)  # all ranks replay, or none does
        if int(verdict.item()) == 1:
            self.graph, self.rotation, self.graph_parity = graph, rotation, epoch_before & 1

    def run_steps(self, steps):
        """Issues exactly `steps` steps on the stream (graph replays of whole rotations, the rest one by one).  With the
        signalling folded into the kernels a step's wait for the other ranks rides in the next step's kernel; the wait
        of the last step is issued here, so that the timed block ends with every rank's columns in place."""
        if self.graph is not None and self.graph_is_block:
            if steps == self.rotation and (self.gather.epoch & 1) == self.graph_parity:
                self.graph.replay()
                self.gather.epoch += self.rotation
                self.counter += self.rotation
                return
            for _ in range(steps):
                self.step()
        else:
            self._run_steps(steps)
        if self.gather is not None:
            self.gather.wait(self.stream)

    def _run_steps(self, steps):
        if self.graph is None:
            for _ in range(steps):
                self.step()
            return
        if (self.gather.epoch & 1) != self.graph_parity:
            raise RuntimeError("buffer parity differs from the captured one")
        calls, rest = divmod(steps, self.rotation)
        for _ in range(calls):
            self.graph.replay()
            self.gather.epoch += self.rotation
            self.counter += self.rotation
        for _ in range(rest):
            self.step()

    def align(self):
        """Brings the step parity back to the one the graph was captured with."""
        if self.graph is not None and (self.gather.epoch & 1) != self.graph_parity:
            self.step()

    def time_blocks(self, steps, warmup, blocks):
        """W warm-up steps, then `blocks` blocks of exactly `steps` steps, each between two CUDA events with a barrier
        + synchronize on both sides; returns the per-block milliseconds, max over ranks."""
        ctx, torch = self.ctx, self.ctx.torch
        self.align()
        for _ in range(warmup + (warmup & 1)):
            self.step()
        out = []
        for _ in range(blocks):
            self.align()
            ms = event_time_ms(torch, lambda: self.run_steps(steps), 1, 0, ctx.barrier if ctx.dist else None)
            out.append(ctx.max_over_ranks(ms))
        return out

    def launches_per_step(self):
        lib = self.ctx.B.lib()
        lib.fth_b200_reset_launch_count()
        self.step()
        n = lib.fth_b200_launch_count()
        self.variant = self.ctx.B.last_variant()  # the kernel family of the step's last launch
        self.ctx.torch.cuda.synchronize()
        return int(n)

    def close(self):
        if self.gather is not None:
            self.ctx.torch.cuda.synchronize()
            self.ctx.barrier()
            self.graph = None
            self.gather.close()
            self.gather = None


def oracle_row_check(ctx, case):
    """N = 1: the timed kernel's output row for weight set 0 against the CPU oracle (full row, M = 1)."""
    import oracle as O
    from tests import util
    torch = ctx.torch
    case.counter = 0
    case.step()
    got = case.result().cpu().numpy()
    w, sw = case.weights[0]
    a = case.a.cpu().numpy()
    w_host = w.cpu().numpy()
    want = O.fp8_linear(O.OP_MATMUL, O.E4M3, a, case.sa, w_host, sw, case.so)

    def bound():
        aa = np.abs(O.fp8_decode(O.E4M3, a).astype(np.float64)) * case.sa
        ww = np.abs(O.fp8_decode(O.E4M3, w_host).astype(np.float64)) * sw
        return (aa @ ww) * 2.0 ** -20
    rep = util.fp8_parity_report(got, want, O.E4M3, bound, case.so)
    rep["oracle"] = "CPU restatement of the reference Common kernel (oracle/feather_oracle.c), full output row of the timed kernel"
    rep["ok"] = bool(rep["failed"] == 0 and rep["class_ok"])
    del torch
    return rep


def gather_check(ctx):
    """N > 1: with one seeded weight shared by all ranks, the gathered [M, N] result on every rank against that rank's
    own single-GPU result on the full weight.  Returns the number of differing bytes summed over ranks and cases."""
    torch, B = ctx.torch, ctx.B
    total, cases = 0, []
    w_full, sw = synth(torch, (K, N), 0.02, SEED + 7, ctx.dev)  # same seed on every rank: the same weight
    w_i8 = w_full.view(torch.int8)
    for kind, m in (("fp8_e4m3", 1), ("fp8_e4m3", 256), ("int8", 16)):
        w_src = w_i8 if kind == "int8" else w_full
        part = w_src[:, ctx.n0:ctx.n1].contiguous()
        sharded = LinearCase(ctx, kind, m, weights=[(part, sw), (part, sw)], use_graph=False)
        single_ctx = Ctx.__new__(Ctx)
        single_ctx.__dict__.update(ctx.__dict__)
        single_ctx.world, single_ctx.dist, single_ctx.n0, single_ctx.n1, single_ctx.n_local = 1, None, 0, N, N
        single = LinearCase(single_ctx, kind, m, weights=[(w_src, sw)])
        if kind == "int8":  # the single-GPU run sees all N channel scales, the shard its slice of the same vector
            assert torch.equal(single.scales[ctx.n0:ctx.n1], sharded.scales)
        single.step()
        want = single.result().clone()
        bad = 0
        for _ in range(2):  # both buffer parities
            sharded.step()
            got = sharded.result()
            bad += int((got != want).sum().item())
        sharded.close()
        cases.append(f"{kind} M={m}")
        total += bad
        del sharded, single, part
    del w_full
    return ctx.sum_over_ranks(total), cases


def sweep(ctx, peaks, quick):
    """FP8 and INT8 at M = 1, 16, 256, 4096 over this rank's columns; at N > 1 the step includes the gather."""
    torch, B = ctx.torch, ctx.B
    out = {}
    shared = {}
    # Memory-bound cases first: the dense ones run the chip into its power cap, and a GEMV timed right behind one
    # (INT8 M = 1 behind FP8 M = 4096) read 13 % slow.  A dense case timed right behind another dense case reads up to
    # 25 % slow for the same reason (same SM clock, same kernel: measured in both orders), so each dense case starts
    # after a one-second pause: these are burst figures, against the burst peak.
    for m in (1, 16, 256, 4096):
        for kind in ("fp8_e4m3", "int8"):
            if quick and m in (16, 256):
                continue
            key = kind
            steps = 200 if m <= 256 else 20
            case = LinearCase(ctx, kind, m, weights=shared.get(key), graph_steps=steps)
            shared[key] = case.weights
            if m > 256:
                torch.cuda.synchronize()
                time.sleep(1.0)
            clocks = ClockSampler(ctx.local_rank)
            clocks.start()
            blocks = case.time_blocks(steps, 4, 3)
            clocks.stop_flag = True
            clocks.join()
            ms = float(np.median(blocks)) / steps
            n_local = ctx.n_local
            gbs = algorithmic_bytes(m, n_local, kind == "int8") / (ms * 1e-3) / 1e9
            tfl = 2.0 * m * K * n_local / (ms * 1e-3) / 1e12
            rec = {"us": round(ms * 1e3, 2), "GB/s_per_gpu": round(gbs, 1), "TFLOP/s_per_gpu": round(tfl, 2),
                   "hbm_frac": round(gbs / peaks["hbm_gbs"], 3), "tensor_frac": round(tfl / (2.0 * peaks["bf16_tflops"]), 3),
                   "kernel": B.last_variant() if ctx.world == 1 else "tcgen05, gather signalling folded in"}
            seen = clocks.summary()
            if seen.get("sm_mhz"):  # the clock the case ran at, and the time scaled to 1 GHz (compares runs at different clocks)
                rec["sm_mhz"] = seen["sm_mhz"]
                rec["us_x_ghz"] = round(ms * 1e3 * seen["sm_mhz"] / 1e3, 2)
                rec["clock_reasons"] = seen["reasons"]
            if m > 256:
                rec["note"] = "burst figure: one second of idle before the timed blocks"
            if ctx.world > 1:
                rec["whole_job_TFLOP/s"] = round(tfl * ctx.world, 1)
                rec["whole_job_weight_GB/s"] = round(K * N / (ms * 1e-3) / 1e9, 1)
                rec["nvlink_bytes_out_per_rank_per_step"] = m * n_local * (ctx.world - 1)
                rec["nvlink_GB/s_out_per_rank"] = round(m * n_local * (ctx.world - 1) / (ms * 1e-3) / 1e9, 1)
                if case.gather is None:
                    rec["gather"] = "NCCL all-gather"
                elif case.gather.multicast and m > 128:
                    rec["gather"] = "one multicast store per output tile (NVLS) + flag wait"
                else:
                    rec["gather"] = "peer stores + flag wait"
            out[f"{kind}_m{m}"] = rec
            case.close()
            del case
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
                           "kernel": B.last_variant(), "what": "the 168 projections alone, each on its own input"}
        del keep, graph
    # the whole step on the device: projections and the operators between them (QwenRmsNorm, Add, SiLU * Mul), chained
    from infer_b200.decoder_step import DecoderStep
    names = ["q", "k", "v", "o", "gate", "up", "down"]
    layer_weights = []
    for _ in range(layers):
        layer = {}
        for name, (k, n) in zip(names, shapes):
            layer[name] = torch.randint(0, 120, (k, n), dtype=torch.uint8, device=dev)
            layer[name + "_scale"] = 2.0 ** -20
        for g in ("g1", "g2"):
            layer[g] = (torch.randn(hidden, device=dev) * 0.1).to(torch.bfloat16).view(torch.int16)
        layer_weights.append(layer)
    wbytes = layers * sum(k * n for k, n in shapes)
    for m in (1, 16):
        for fused in (True, False):
            step = DecoderStep(torch, layer_weights, m, hidden, inter, 2.0 ** -9, 2.0 ** -9, fp8_dtype=B.E5M2, fused=fused)
            step.x.copy_(torch.randn((m, hidden), device=dev).to(torch.bfloat16).view(torch.int16))
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                step.run(C.c_void_p(side.cuda_stream))
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    step.run(C.c_void_p(torch.cuda.current_stream().cuda_stream))
            ms = event_time_ms(torch, graph.replay, 20, 3) / 20
            result[f"whole_step_m{m}_{'fused' if fused else 'node_by_node'}"] = {
                "us": round(ms * 1e3, 1), "launches": step.launches, "weight_GB/s": round(wbytes / (ms * 1e-3) / 1e9, 1),
                "hbm_frac_of_weights": round(wbytes / (ms * 1e-3) / 1e9 / measured_peaks()["hbm_gbs"], 3),
                "what": "24 layers, every node on the device: " + ("6 launches per layer (fth_b200_fp8_linear_fused)" if fused else "12 launches per layer")}
            del graph, step
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


def reference_x86_other_configs():
    """The reference's x86 kernels for configs 2, 3, 4 and 5-INT8 on this box's host cores: best of a few compute()
    calls after Prepare(), through the unmodified reference library.  Thread counts are the reference's own: FP8 linear
    at most 4 OpenMP threads (src/kernel/x86/linear_fp8.cc:45-70), INT8 linear one thread (scalar loops,
    src/kernel/x86/int8.cc:461-682), INT8 conv all OpenMP threads (src/kernel/x86/int8.cc:684-2346)."""
    import oracle as O
    from tests import util
    if not O.have_ref():
        return {"unavailable": "the reference library is not present on this box"}
    out = {"host_cpus": os.cpu_count()}
    try:
        # config 2: INT8 MatMul M=128 K=1024 N=1024
        case = util.make_int8_linear(128, 1024, 1024, seed=2)
        kern = O.int8_linear(O.OP_MATMUL, case["a"], case["sa"], 0, case["w"], case["ws"], None, case["so"], 0, impl="ref", device=O.X86, return_kernel=True)
        kern.prepare()
        out["config2_int8_m128_k1024_n1024"] = {"ms": round(kern.time_compute(2) * 1e3, 2), "threads": 1}
        # config 3: INT8 conv + the INT8 ReLU node behind it
        case = util.make_int8_conv(1, 64, 160, 160, 64, 3, 3, seed=3)
        kern = O.int8_conv2d(case["x"], case["sx"], 0, case["w"], case["ws"], None, case["bias"], case["so"], 0, impl="ref", device=O.X86,
                             return_kernel=True)
        kern.prepare()
        flags = open("/proc/cpuinfo").read()
        out["config3_conv_64x160x160"] = {"ms": round(kern.time_compute(5) * 1e3, 2), "threads": os.cpu_count(), "avx_vnni": " avx_vnni" in flags,
                                          "note": "conv node only; the ReLU node behind it is a 1.6 MB table lookup"}
        # config 4: the three projection shapes at M = 1 (FP8 E5M2, packed BF16 GEMV), times their count per decode step
        total = 0.0
        per_shape = {}
        for (k, n, count) in ((1024, 1024, 4 * 24), (1024, 3584, 2 * 24), (3584, 1024, 24)):
            c = util.make_fp8_linear(O.E5M2, 1, k, n, seed=k + n, pow2=True)
            kern = O.fp8_linear(O.OP_MATMUL, O.E5M2, c["a"], c["sa"], c["w"], c["sw"], c["so"], impl="ref", device=O.X86, return_kernel=True)
            kern.prepare()
            t = kern.time_compute(20)
            per_shape[f"{k}x{n}"] = round(t * 1e6, 1)
            total += t * count
        out["config4_decode_step_m1"] = {"ms": round(total * 1e3, 2), "threads": min(4, os.cpu_count() or 1), "per_projection_us": per_shape,
                                         "note": "168 MatMul nodes only (per-shape time x count, weights of one shape stay cached); Cast / RMSNorm / Add nodes not included"}
        # config 5 INT8, M = 1: a 2048-column slice of the weight, scaled to N = 28672 (the kernel is a scalar loop over
        # outputs; its time is proportional to the number of columns)
        cols = 2048
        w, ws = util.make_int8_weight(K, cols, seed=5)
        a = np.random.default_rng(5).integers(-127, 128, (1, K), dtype=np.int8)
        kern = O.int8_linear(O.OP_MATMUL, a, 0.02, 0, w, ws, None, util.int8_out_scale(K, ws), 0, impl="ref", device=O.X86, return_kernel=True)
        kern.prepare()
        t = kern.time_compute(2)
        out["config5_int8_m1"] = {"ms": round(t * N / cols * 1e3, 1), "threads": 1, "extrapolated": f"measured {round(t * 1e3, 2)} ms on {cols} of {N} columns"}
    except Exception as exc:  # reported, never required
        out["error"] = f"{type(exc).__name__}: {exc}"
    return out


def run_gpu_arm(args):
    import torch
    import infer_b200 as B

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    dev = torch.device("cuda", local_rank)
    B.lib()  # fails loudly if the CUDA library is missing
    peaks = measured_peaks()
    ctx = Ctx(torch, B, dist, world, rank, dev)
    failures = []

    # ---- N > 1: prove the gathered bytes before timing anything ----
    gather_mismatch, gather_cases = None, None
    if world > 1:
        gather_mismatch, gather_cases = gather_check(ctx)
        if gather_mismatch != 0:
            failures.append(f"gathered result differs from the single-GPU result in {gather_mismatch} bytes")

    main = LinearCase(ctx, "fp8_e4m3", 1, graph_steps=args.steps)
    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- timed region: blocks of exactly K steps, device-timed, max over ranks; the median block is reported ----
    per_step_launches = main.launches_per_step()
    block_ms = main.time_blocks(args.steps, args.warmup, BLOCKS)
    total_ms = float(np.median(block_ms))
    variant = main.variant
    status_timed = B.device_status()
    ms_per_step = total_ms / args.steps
    bytes_step = algorithmic_bytes(1, N)
    value = bytes_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: pinned host activation in, host result out, every step ----
    a_host = torch.empty((1, K), dtype=torch.uint8).pin_memory()
    a_host.copy_(main.a.cpu())
    width = ctx.shard.width
    out_host = torch.empty((1, width), dtype=torch.uint8).pin_memory()
    full_host = torch.empty((1, N), dtype=torch.uint8).pin_memory()
    plans = []
    if world == 1:
        for i in range(2):
            w, sw = main.weights[i]
            hd = B.fp8_linear_desc(dtype=B.E4M3, op=B.OP_MATMUL, m=1, k=K, n=N, a=None, w=None, out=None, a_scale=main.sa,
                                   w_scale=sw, out_scale=main.so, ldo=width)
            w_host = w.cpu()
            hd.w = w_host.data_ptr()
            plans.append(B.Plan(hd))
            del w_host
    pc = [0]
    e2e_case = None
    if world > 1:
        e2e_case = LinearCase(ctx, "fp8_e4m3", 1, weights=main.weights, use_graph=False)
        a_stage = e2e_case.a

    def e2e_body(stream):
        # N > 1: pinned-host activation in, sharded kernels with peer stores, the gathered row back to the host (both rows
        # are a few KB: copied by the SMs on the stream, fth_b200_small_copy)
        B.small_copy(a_stage, a_host, K, stream)
        e2e_case.step()
        if e2e_case.gather is not None:
            e2e_case.gather.wait(stream)
            B.small_copy(full_host, e2e_case.gather.buffer(e2e_case.gather.rank, e2e_case.gather.epoch & 1), N, stream)
        else:
            full_host.copy_(e2e_case.nccl_gathered.view(1, -1)[:, :N], non_blocking=True)

    # The four launches of an end-to-end step are the same every time the same weight set and buffer parity come round, so
    # each (set, parity) step is recorded once and replayed with one graph launch, as fth_b200_plan_run does on one GPU.
    # A rank whose capture fails issues the calls one by one.
    e2e_graphs, e2e_pos = [], [0]
    if world > 1 and e2e_case.gather is not None:
        rotation = e2e_case.n_sets * (2 if e2e_case.n_sets % 2 else 1)
        for _ in range(rotation):
            e2e_body(ctx.stream)
        torch.cuda.synchronize()
        ctx.barrier()
        side = torch.cuda.Stream()
        epoch_before, counter_before = e2e_case.gather.epoch, e2e_case.counter
        try:
            with torch.cuda.stream(side):
                for _ in range(rotation):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        e2e_case.stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                        e2e_body(e2e_case.stream)
                    e2e_graphs.append(g)
        except Exception as exc:
            e2e_graphs = []
            print(f"[bench] rank {rank}: capture of the end-to-end step failed ({type(exc).__name__}: {exc}); issuing the calls one by one", file=sys.stderr)
        e2e_case.stream = ctx.stream
        e2e_case.gather.epoch, e2e_case.counter = epoch_before, counter_before
        torch.cuda.synchronize()

    def e2e_step():
        if world == 1:
            plans[pc[0] & 1].run(a_host, out_host, ctx.stream)
            pc[0] += 1
            return
        if e2e_graphs:
            e2e_graphs[e2e_pos[0] % len(e2e_graphs)].replay()
            e2e_pos[0] += 1
            e2e_case.gather.epoch += 1
            e2e_case.counter += 1
        else:
            e2e_body(ctx.stream)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(args.steps, 500)
    e2e_blocks = [ctx.max_over_ranks(event_time_ms(torch, e2e_step, e2e_steps, max(args.warmup, 3) if b == 0 else 0, ctx.barrier if dist else None))
                  for b in range(3)]
    e2e_ms = float(np.median(e2e_blocks)) / e2e_steps
    e2e_value = bytes_step / (e2e_ms * 1e-3) / 1e9
    status_e2e = B.device_status()
    # the host row of the last end-to-end step against the device-resident path on the same weight set
    if world == 1:
        main.counter = (pc[0] - 1) & 1
        main.step()
        e2e_mismatch = int((main.result().cpu()[:, :N] != out_host[:, :N]).sum().item())
    elif e2e_case.gather is not None:
        e2e_mismatch = int((e2e_case.result().cpu()[:, :N] != full_host).sum().item())
    else:
        e2e_mismatch = None
    if e2e_mismatch:
        failures.append(f"end-to-end host result differs from the device-resident result in {e2e_mismatch} bytes")
    e2e_mismatch = None if e2e_mismatch is None else int(ctx.max_over_ranks(float(e2e_mismatch)))
    for p in plans:
        p.close()
    e2e_graphs_used = bool(e2e_graphs)
    e2e_graphs = []
    if e2e_case is not None:
        e2e_case.close()
        e2e_case = None

    # ---- N = 1: the timed kernel's output against the CPU oracle ----
    parity = None
    if world == 1:
        parity = oracle_row_check(ctx, main)
        if not parity["ok"]:
            failures.append(f"output of the timed kernel differs from the oracle: {parity}")
    gather_kind = None
    if world > 1:
        gather_kind = "outputs stored to all ranks over NVLink from the kernels' epilogues, step flags published by the kernels' last thread block" if main.gather is not None else "NCCL all-gather"
    n_sets, graph_used = main.n_sets, main.graph is not None
    main.close()
    del main

    extra = {}
    if not args.quick or world > 1:
        extra = sweep(ctx, peaks, quick=args.quick)
        if rank == 0 and world == 1:
            extra["config4_decode_step"] = config4_decode_step(torch, B, dev, ctx.fp8_call, ctx.stream)
            extra["config3_conv"] = config3_conv(torch, B, dev, ctx.stream)
        extra["peaks"] = {"hbm_gbs": peaks["hbm_gbs"], "fp8_int8_dense_tflops": 2.0 * peaks["bf16_tflops"],
                          "note": "8-bit dense peak taken as twice the measured bf16 burst figure", "source": peaks["source"]}
    status_extra = B.device_status()
    device_status = ctx.max_over_ranks(float(max(abs(status_timed), abs(status_e2e), abs(status_extra))))
    if device_status != 0:
        failures.append(f"device status word non-zero on some rank: {int(device_status)}")
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    cpu_baseline = None
    if rank == 0 and world == 1:
        cpu_baseline = cpu_baseline_measurement(torch)
        if not args.quick:
            extra["reference_x86"] = reference_x86_other_configs()

    if rank == 0:
        achieved = value if world == 1 else value / world
        # one launch: the cluster kernel (up to about two waves of CTAs: 8 per 128-column tile) or, with more tiles, the
        # persistent kernel in its folded form (a CTA runs all K chunks of a tile and adds them from tensor memory)
        tiles_local = (ctx.n_local + 127) // 128
        step_kernel = ("tcgen05 GEMV + split-K reduce kernel" if per_step_launches != 1 else
                       "single-launch tcgen05 cluster kernel" if tiles_local < 98 else
                       "persistent tcgen05 weight-streaming kernel, one launch (the K chunks of a tile are added from tensor memory)")
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "blocks": BLOCKS, "block_ms": [round(b, 4) for b in block_ms],
            "config": bench_config(world, {
                "sharding": (f"N column-sharded over {world} GPUs, {gather_kind}" + (", steps replayed from a CUDA graph" if graph_used else "")) if world > 1 else "one GPU",
                "l2": f"inputs larger than L2: {n_sets} weight sets of {K * ctx.n_local / 1e6:.0f} MB rotated", "kernel": variant}),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
                         "peak_source": peaks["source"],
                         "note": "per GPU; step = " + (step_kernel) +
                                 (", gather signalling inside the kernel (one fth_b200_gather_wait per timed block)" if world > 1 else "") + "; median of the timed blocks"},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": K, "d2h_bytes_per_step": width if world == 1 else N,
                    "ms_per_step": round(e2e_ms, 5), "mismatch_bytes": e2e_mismatch,
                    "api": "fth_b200_plan_run (pinned host activation in, host result out; its two launches replayed from a graph)" if world == 1 else
                           "pinned host activation in, fth_b200_fp8_linear with peer stores and folded step signalling + fth_b200_gather_wait, gathered row out" +
                           (" (the four launches of a step replayed from a CUDA graph per weight set and buffer parity)" if e2e_graphs_used else "")},
            "gpu_launches": int(per_step_launches * args.steps),
            "device_status": int(device_status),
            "parity": parity,
            "gather_mismatch_bytes": gather_mismatch,
            "gather_checked": gather_cases,
            "clocks": sampler.summary(),
            "cpu_baseline": cpu_baseline,
            "extra": extra,
        }
        if failures:
            line["failures"] = failures
        print(json.dumps(line))
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if failures:
        print("[bench] FAILED: " + "; ".join(failures), file=sys.stderr)
        return 1
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--quick", action="store_true", help="shorter sweep: M = 1 and 4096 only, no x86 timings of the other configs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
