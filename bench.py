#!/usr/bin/env python
"""Benchmark of the dense GEMM hot path on N B200s of one node.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--sub-configs all|none] [--impl reference]
                    [--tile-n 256|512] [--tuning "NAME=VALUE;..."] [--ksplit-exchange fused|reduce|nccl]

One step = one pass of the hot path over the workload: one GEMM launch per GPU (plus, for the
K-split workload, the reduce-scatter of the fp32 partials and the sum + bf16 cast).  Rank 0
prints ONE JSON line.  `value` is whole-job TFLOP/s with operands resident in HBM; `e2e` is the
same metric through the C-ABI call that takes HOST buffers (host->device copies of the operands
and the device->host copy of C inside the timed region).  `roofline` bounds the kernel by the
measured cuBLAS bf16 throughput of this pool (MEASURED_PEAKS.json) scaled by the nominal ratio of
the dtype's tensor rate to bf16's; `cpu_baseline` times the CPU oracle (the reference has no CPU
GEMM of its own) on a bounded sample of the same workload.

Workloads (BASELINE.json configs):
  bf16_8192_bias   configs[1]  headline.  At N > 1 the N-split of C = A . B^T over the output
                               columns, 8192 columns per GPU, no collective: weak scaling.
  bf16_512         configs[0]  plumbing check.
  fp8_block        configs[2]  8192 x 14336 x 4096, N-split of the fixed problem: strong scaling.
  nvfp4            configs[3]  16384 x 28672 x 8192, N-split of the fixed problem: strong scaling.
  bf16_ksplit      configs[4]  8192 x 8192 x 131072, K-split + reduce-scatter (fused or NCCL) of the fp32
                               partials + bf16 cast: strong scaling; compute and communication
                               reported separately.
The default run measures the headline workload and then, in the same process and at the same N,
fp8_block, nvfp4 and bf16_ksplit (with all three exchanges at N > 1); their records go into the line's
`configs` object.  The bf16 workloads run the CTA-pair kernel with the 512-column tile (--tile-n 256
selects the narrower one).  Operand sources are drawn on the GPU from a seeded Philox generator (the host
generator needs minutes for 10^9 values) and quantised by the library's own GPU quantisers.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL_PEAK_TFLOPS = {"bf16": 2250.0, "f8e4m3": 4500.0, "nvfp4": 9000.0}
FALLBACK_PEAK_TFLOPS = 1590.0     # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent

WORKLOADS = {
    "bf16_8192_bias": dict(kind="bf16", dtype="bf16", m=8192, n=8192, k=8192, seed=1, dist="normal", scale=0.05, bias=True,
                           out="bf16", shard="n_weak", tile="256x256x64 per CTA pair"),
    "bf16_512": dict(kind="bf16", dtype="bf16", m=512, n=512, k=512, seed=0, dist="uniform", scale=1.0, bias=False,
                     out="bf16", shard="n_weak", tile="256x256x64 per CTA pair"),
    "fp8_block": dict(kind="fp8", dtype="f8e4m3", m=8192, n=14336, k=4096, seed=2, dist="normal", scale=1.0, bias=False,
                      out="bf16", shard="n_strong", tile="256x256x128 per CTA pair"),
    "nvfp4": dict(kind="nvfp4", dtype="nvfp4", m=16384, n=28672, k=8192, seed=3, dist="normal", scale=1.0, bias=False,
                  out="bf16", shard="n_strong", tile="256x256x256 per CTA pair"),
    "bf16_ksplit": dict(kind="ksplit", dtype="bf16", m=8192, n=8192, k=131072, seed=4, dist="uniform", scale=0.5,
                        bias=False, out="bf16", shard="k_strong", tile="256x256x64 per CTA pair"),
}
SUB_CONFIGS = ["fp8_block", "nvfp4", "bf16_ksplit"]
BF16_TILE_N = 512       # columns of the CTA-pair tile of the bf16 workloads (the kernels also take 256)
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, from the ncu
# captures summarised under profiles/; None where no capture exists.
TRAFFIC_BYTES = {"bf16_8192_bias": 9.694e8, "fp8_block": 3.291e8, "nvfp4": 1.5667e9}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.001):
        super().__init__(daemon=True)
        self.index, self.period, self.samples, self.reasons, self.max_mhz = index, period_s, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_min_mhz": s[0], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "period_ms": self.period * 1e3}


# --------------------------------------------------------------------------- CPU side (oracle)
def cpu_gemm_sample(w, budget_s=12.0, threads=None):
    """Times the CPU oracle (fp32 sgemm over fp32 copies of the operands, all host cores) on a slab of rows and
    a K range of the workload sized to about `budget_s` seconds.  Returns (record, seconds per pass)."""
    import torch
    from oracle import gemm_oracle as O
    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    n, k = w["n"], min(w["k"], 16384)                   # the K-split workload: one GPU's K slice at most
    probe_rows = min(w["m"], 256)
    a = O.round_to_bf16(O.normal((probe_rows, k), w["seed"], w["scale"]))
    b = O.round_to_bf16(O.normal((n, k), w["seed"] + 1000, w["scale"]))
    O.gemm_f32(a, b)                                   # warm the thread pool
    t0 = time.perf_counter(); O.gemm_f32(a, b); dt = time.perf_counter() - t0
    rate = 2.0 * probe_rows * n * k / max(dt, 1e-9)
    rows = int(min(w["m"], max(probe_rows, budget_s * rate / (2.0 * n * k))))
    rows = max(128, (rows // 128) * 128) if w["m"] >= 128 else w["m"]
    a = O.round_to_bf16(O.normal((rows, k), w["seed"], w["scale"]))
    one = 2.0 * rows * n * k / rate
    reps = int(max(1, min(30, budget_s / max(one, 1e-9)))) if rows == w["m"] else 1
    t0 = time.perf_counter()
    for _ in range(reps):
        c = O.gemm_f32(a, b)
    dt = time.perf_counter() - t0
    del c
    return {"value": 2.0 * rows * n * k * reps / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"rows 0..{rows - 1} of A against all of B ({rows}x{n}x{k}, fp32 values of the "
                      f"{w['dtype']} operands), fp32 sgemm x{reps}, {dt:.2f} s"}, dt / reps


def run_reference(args, w, rank):
    """--impl reference: the reference has no CPU (or working GPU) GEMM; its arithmetic is the oracle's,
    timed here on the host cores with all threads, a bounded slab per step."""
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        res, dt = cpu_gemm_sample(w, budget_s=args.cpu_budget)
        if i >= args.warmup:
            vals.append((res, dt))
    best = max(vals, key=lambda v: v[0]["value"])[0]
    v = sum(r["value"] for r, _ in vals) / len(vals)
    line = {"impl": "reference", "metric": "gemm_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(dt for _, dt in vals) / len(vals),
            "higher_is_better": True, "scaling": scaling_of(w), "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "config": workload_config(args.workload, w, args.gpus, tile_n=args.tile_n),
            "cpu_baseline": dict(best, value=v),
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def scaling_of(w):
    return "weak" if w["shard"] == "n_weak" else "strong"


def workload_config(name, w, gpus, exchange="fused", tile_n=0):
    m, n, k = w["m"], w["n"], w["k"]
    if w["shard"] == "n_weak":
        sharding = "single GPU" if gpus == 1 else f"N-split over {gpus} GPUs ({n} columns each), no collective"
        shape = {"m": m, "n_per_gpu": n, "n_total": n * gpus, "k": k}
    elif w["shard"] == "n_strong":
        sharding = "single GPU" if gpus == 1 else f"N-split of the fixed problem over {gpus} GPUs, no collective"
        shape = {"m": m, "n_per_gpu": n // gpus, "n_total": n, "k": k}
    else:
        sharding = ("single GPU: fp32 partials of K slices of 32768 + sum and bf16 cast" if gpus == 1 else
                    f"K-split over {gpus} GPUs, reduce-scatter of the fp32 partials "
                    + ("fused into the GEMM's epilogue: tiles added into the owner's buffer over NVLink (TMA reduce)" if exchange == "reduce"
                       else "fused into the GEMM's stores over NVLink peer memory, summed by the owner" if exchange == "fused"
                       else "by NCCL") + ", bf16 cast")
        shape = {"m": m, "n_total": n, "k_per_gpu": k // gpus, "k": k}
    tile = w["tile"] if w["kind"] not in ("bf16", "ksplit") else f"256x{tile_n or BF16_TILE_N}x64 per CTA pair"
    return dict({"workload": name, "tile": tile, "sharding": sharding,
                 "epilogue": "alpha=1" + (" + bf16 bias[n]" if w["bias"] else "") + f" -> {w['out']}",
                 "l2": "operands and output per GPU exceed the 126 MB L2"}, **shape)


# --------------------------------------------------------------------------- GPU workloads
class Workload:
    """Builds device + pinned host operands for this rank's shard; step() launches the hot path once."""

    def __init__(self, name, w, rank, world, dev, exchange="fused", tuning="", tile_n=0):
        self.exchange = exchange
        self.tile_n = tile_n or BF16_TILE_N   # bf16 workloads: columns of the CTA-pair tile
        self.tuning = tuning          # the spec's tuning string ("NAME=VALUE;..."), for A/B runs from the command line
        import numpy as np
        import torch
        from oracle import gemm_oracle as O
        from tesserae_b200 import api
        self.np, self.torch, self.O, self.api = np, torch, O, api
        self.name, self.w, self.rank, self.world, self.dev = name, w, rank, world, dev
        self.m, self.k = w["m"], w["k"]
        self.n = w["n"] if w["shard"] in ("n_weak", "k_strong") else w["n"] // world
        if w["shard"] == "k_strong":
            self.k = w["k"] // world
        self.stream = torch.cuda.current_stream().cuda_stream
        self.launches_per_step = 1
        self.e2e_api = "tesserae_gemm_run_host"
        getattr(self, "_setup_" + w["kind"])()

    def _draw(self, shape, seed):
        """Seeded fp32 source on this GPU (Philox: the same values on every rank for a given seed)."""
        t, w = self.torch, self.w
        g = t.Generator(device=self.dev).manual_seed(seed)
        if w["dist"] == "normal":
            return t.randn(shape, generator=g, dtype=t.float32, device=self.dev) * w["scale"]
        return (t.rand(shape, generator=g, dtype=t.float32, device=self.dev) * 2 - 1) * w["scale"]

    def _pin(self, x):
        return x.cpu().pin_memory()

    def _setup_bf16(self):
        t, w, api = self.torch, self.w, self.api
        self.a = self._draw((self.m, self.k), w["seed"]).to(t.bfloat16)
        self.b = self._draw((self.n, self.k), w["seed"] + 1000 + self.rank).to(t.bfloat16)
        self.bias = (t.randn(self.n, generator=t.Generator(device=self.dev).manual_seed(w["seed"] + 2000 + self.rank),
                             device=self.dev) * 0.1).to(t.bfloat16) if w["bias"] else None
        self.a_host, self.b_host = self._pin(self.a), self._pin(self.b)
        self.bias_host = self._pin(self.bias) if w["bias"] else None
        self.c_host = t.empty((self.m, self.n), dtype=t.bfloat16).pin_memory()
        self.c = t.empty((self.m, self.n), dtype=t.bfloat16, device=self.dev)
        tile_n = self.tile_n
        self.plan = api.GemmPlan(api.KernelSpec(name=f"gemm_bf16_cg2_bf16_b{int(w['bias'])}" + ("" if tile_n == 256 else f"_n{tile_n}"),
                                                elem=api.BF16, tile=(128, tile_n, 64), cta_group=2, out_elem=api.BF16,
                                                has_bias=int(w["bias"]), tuning=self.tuning))
        self.step = lambda: self.plan.run(self.a, self.b, self.c, self.bias, 1.0, self.m, self.n, self.k, stream=self.stream)
        self.e2e_step = lambda: self.plan.run_host(self.a_host, self.b_host, self.c_host, self.bias_host, 1.0,
                                                   self.m, self.n, self.k)
        self.h2d = self.a_host.numel() * 2 + self.b_host.numel() * 2 + (self.n * 2 if w["bias"] else 0)
        self.d2h = self.c_host.numel() * 2

    def _setup_fp8(self):
        t, api, w = self.torch, self.api, self.w
        n0 = self.rank * self.n
        src = self._draw((self.m, self.k), w["seed"])
        self.a = t.empty((self.m, self.k), dtype=t.uint8, device=self.dev)
        self.sa = t.empty((self.m, self.k // 128), dtype=t.float32, device=self.dev)
        api.quantize_fp8_rows(src, self.a, self.sa, self.m, self.k, stream=self.stream)
        src = self._draw((w["n"], self.k), w["seed"] + 1000)[n0:n0 + self.n].contiguous()   # the shard's rows of the one B
        self.b = t.empty((self.n, self.k), dtype=t.uint8, device=self.dev)
        self.sb = t.empty(((self.n + 127) // 128, self.k // 128), dtype=t.float32, device=self.dev)
        api.quantize_fp8_blocks(src, self.b, self.sb, self.n, self.k, stream=self.stream)
        del src
        self.ga = self.gb = 1.0
        self.c = t.empty((self.m, self.n), dtype=t.bfloat16, device=self.dev)
        self.plan = api.GemmPlan(api.KernelSpec(name="gemm_fp8blk_cg2_n256", elem=api.F8E4M3, tile=(128, 256, 128),
                                                cta_group=2, out_elem=api.BF16, scale_mode=api.SCALE_FP8_BLOCK,
                                                tuning=self.tuning))
        self._finish_scaled()
        # Stream-K tail: when this rank's tile count leaves a nearly empty last wave the plan asks for a workspace and
        # the device step goes through the workspace entry point.
        self.tail_bytes = self.plan.tail_workspace_bytes(self.m, self.n, self.k)
        if self.tail_bytes:
            self.tail_ws = t.zeros(self.tail_bytes // 4, dtype=t.float32, device=self.dev)
            self.launches_per_step = 2
            self.step = lambda: self.plan.run_scaled_ws(self.a, self.b, self.c, self.sa, self.sb, self.tail_ws, self.tail_bytes,
                                                        None, 1.0, self.m, self.n, self.k, stream=self.stream)

    def _setup_nvfp4(self):
        t, api, w = self.torch, self.api, self.w
        n0 = self.rank * self.n
        ws4 = t.zeros(4, dtype=t.uint8, device=self.dev)

        def quant(rows, seed):
            src = self._draw((rows, self.k), seed)
            q = t.empty((rows, self.k // 2), dtype=t.uint8, device=self.dev)
            sf = t.zeros((api.nvfp4_scale_bytes(rows, self.k),), dtype=t.uint8, device=self.dev)
            g = api.quantize_nvfp4(src, q, sf, ws4, rows, self.k, stream=self.stream)
            return q, sf, g
        self.a, self.sa, self.ga = quant(self.m, w["seed"])
        qb, sfb, self.gb = quant(w["n"], w["seed"] + 1000)         # one per-tensor scale for the whole B, not per shard
        per_row_block = (self.k // 64) * 512                       # scale bytes of one 128-row block
        self.b = qb[n0:n0 + self.n].contiguous()
        self.sb = sfb[(n0 // 128) * per_row_block:((n0 + self.n + 127) // 128) * per_row_block].contiguous()
        del qb, sfb
        self.c = t.empty((self.m, self.n), dtype=t.bfloat16, device=self.dev)
        self.plan = api.GemmPlan(api.KernelSpec(name="gemm_nvfp4_cg2_n256", elem=api.F4E2M1, tile=(128, 256, 256),
                                                cta_group=2, out_elem=api.BF16, scale_mode=api.SCALE_NVFP4,
                                                tuning=self.tuning))
        self._finish_scaled()

    def _finish_scaled(self):
        """Device step through tesserae_gemm_run_scaled; end-to-end step through tesserae_gemm_run_scaled_host with
        pinned host copies of the quantised operands and scale tables (they go up, C comes back, inside the call)."""
        t = self.torch
        self.step = lambda: self.plan.run_scaled(self.a, self.b, self.c, self.sa, self.sb, None, 1.0, self.m, self.n,
                                                 self.k, stream=self.stream, global_a=self.ga, global_b=self.gb)
        self.h_in = [self._pin(x) for x in (self.a, self.b, self.sa, self.sb)]
        self.c_host = t.empty((self.m, self.n), dtype=t.bfloat16).pin_memory()
        self.h2d = sum(x.numel() * x.element_size() for x in self.h_in)
        self.d2h = self.c_host.numel() * 2
        self.e2e_api = "tesserae_gemm_run_scaled_host"
        self.e2e_step = lambda: self.plan.run_scaled_host(self.h_in[0], self.h_in[1], self.c_host, self.h_in[2], self.h_in[3],
                                                          None, 1.0, self.m, self.n, self.k, global_a=self.ga, global_b=self.gb)

    def _setup_ksplit(self):
        t, api, w = self.torch, self.api, self.w
        import torch.distributed as dist
        # K slice of this rank of the one seeded A and B: contiguous M x K/G and N x K/G buffers
        k0 = self.rank * self.k
        self.a = self._draw((self.m, w["k"]), w["seed"])[:, k0:k0 + self.k].to(t.bfloat16).contiguous()
        self.b = self._draw((self.n, w["k"]), w["seed"] + 1000)[:, k0:k0 + self.k].to(t.bfloat16).contiguous()
        self.a_host, self.b_host = self._pin(self.a), self._pin(self.b)
        self.partial = t.empty((self.m, self.n), dtype=t.float32, device=self.dev)       # scratch: fp32 partial C
        rows = self.m // self.world
        self.mine = t.empty((rows, self.n), dtype=t.float32, device=self.dev) if self.world > 1 else self.partial
        self.c = t.empty((rows, self.n), dtype=t.bfloat16, device=self.dev)
        self.c_host = t.empty((rows, self.n), dtype=t.bfloat16).pin_memory()
        fused = self.world > 1 and self.exchange == "fused"
        reduce_ = self.world > 1 and self.exchange == "reduce"
        tile_n = self.tile_n
        self.plan = api.GemmPlan(api.KernelSpec(name=("gemm_bf16_cg2_f32_scatter" if fused else
                                                      "gemm_bf16_cg2_f32_scatter_add" if reduce_ else "gemm_bf16_cg2_f32_b0")
                                                + ("" if tile_n == 256 else f"_n{tile_n}"),
                                                elem=api.BF16, tile=(128, tile_n, 64), cta_group=2, out_elem=api.F32,
                                                scatter=1 if fused else 2 if reduce_ else 0))
        nbytes = self.partial.numel() * 4
        self.launches_per_step = 2
        if fused:
            # Exchange fused into the GEMM: every tile's TMA store lands in its owner's staging slot
            # stag[buffer][source rank] over NVLink while the tensor cores run on; one barrier, then each
            # owner sums its `world` slots and casts.  Two buffers, so step i+1's stores cannot reach a slot
            # that a slower peer is still summing in step i.
            import torch.distributed._symmetric_memory as symm
            self.partial = None
            stag = symm.empty((2, self.world, rows, self.n), dtype=t.float32, device=self.dev)
            hdl = symm.rendezvous(stag, dist.group.WORLD.group_name)
            slot = rows * self.n * 4
            self._symm, self._it = (stag, hdl), 0

            def step(ev=None):
                buf = self._it & 1
                self._it += 1
                dst = [hdl.buffer_ptrs[g] + (buf * self.world + self.rank) * slot for g in range(self.world)]
                if ev:
                    ev[0].record()
                self.plan.ksplit_scatter(self.a, self.b, dst, rows, self.m, self.n, self.k, stream=self.stream, start_owner=self.rank)
                if ev:
                    ev[1].record()
                hdl.barrier(channel=0)
                if ev:
                    ev[3].record()
                api.reduce_cast_bf16(stag[buf], self.world, rows * self.n, self.c, rows * self.n, stream=self.stream)
                if ev:
                    ev[2].record()
            self.step = step
            self._finish_ksplit()
            return

        if reduce_:
            # Exchange and sum fused into the GEMM: every tile is ADDED (TMA reduce, fp32 add in the owner's memory
            # system) into the owner's one M/G x N buffer; one barrier; the owner casts.  No staging per source, no
            # sum pass.  Two buffers: the one a step has cast is cleared right away and is written again only two
            # steps later, after every rank has passed the barrier of the step in between.
            import torch.distributed._symmetric_memory as symm
            self.partial = None
            acc = symm.empty((2, rows, self.n), dtype=t.float32, device=self.dev)
            hdl = symm.rendezvous(acc, dist.group.WORLD.group_name)
            acc.zero_()
            t.cuda.synchronize()
            hdl.barrier(channel=0)
            self._symm, self._it = (acc, hdl), 0
            half = rows * self.n * 4

            def step(ev=None):
                buf = self._it & 1
                self._it += 1
                dst = [hdl.buffer_ptrs[g] + buf * half for g in range(self.world)]
                if ev:
                    ev[0].record()
                self.plan.ksplit_scatter(self.a, self.b, dst, rows, self.m, self.n, self.k, stream=self.stream, start_owner=self.rank)
                if ev:
                    ev[1].record()
                hdl.barrier(channel=0)
                if ev:
                    ev[3].record()
                api.cast_clear_bf16(acc[buf], self.c, rows * self.n, stream=self.stream)
                if ev:
                    ev[2].record()
            self.launches_per_step = 2
            self.step = step
            self._finish_ksplit()
            return

        # One GPU holds the whole K: it is still multiplied in slices of at most 32768, each into its own fp32
        # partial, and the partials are summed by the cast pass.  The tensor core's own fp32 accumulation over
        # 131072 terms drifts (measured 1.3e-2 of the floored magnitude against 4e-3 with four slices).
        slices = max(1, self.k // 32768) if self.world == 1 else 1
        if slices > 1:
            self.partial = t.empty((slices, self.m, self.n), dtype=t.float32, device=self.dev)
            self.mine = self.partial
            nbytes = self.partial.numel() * 4

        def step(ev=None):
            if ev:
                ev[0].record()
            self.plan.ksplit_partials(self.a, self.b, self.partial, nbytes, self.m, self.n, self.k, slices, stream=self.stream)
            if ev:
                ev[1].record()
            if self.world > 1:
                dist.reduce_scatter_tensor(self.mine, self.partial, op=dist.ReduceOp.SUM)
            if ev:
                ev[3].record()
            api.reduce_cast_bf16(self.mine, slices, self.m * self.n if slices > 1 else 0, self.c, self.c.numel(),
                                 stream=self.stream)
            if ev:
                ev[2].record()
        self.launches_per_step = slices + 1
        self.step = step
        self._finish_ksplit()

    def _finish_ksplit(self):
        t = self.torch

        def e2e():
            self.a.copy_(self.a_host, non_blocking=True)
            self.b.copy_(self.b_host, non_blocking=True)
            self.step()
            self.c_host.copy_(self.c, non_blocking=True)
            t.cuda.current_stream().synchronize()
        self.e2e_step = e2e
        self.e2e_api = "harness copies around the device-pointer K-split entry points (no host-buffer K-split call exists)"
        self.h2d = self.a_host.numel() * 2 + self.b_host.numel() * 2
        self.d2h = self.c_host.numel() * 2

    def _check_ksplit(self):
        """Sampled entries of every owner's rows: each rank's fp64 partial over its own K slice, summed over the
        ranks, against the owner's bf16 output."""
        import torch.distributed as dist
        np, O, t = self.np, self.O, self.torch
        rows_per = self.m // self.world
        local = [0, rows_per // 2, rows_per - 1]
        rows = [g * rows_per + r for g in range(self.world) for r in local]
        cols = list(range(0, self.n, 61))
        part = O.gemm_f64_entries(self.a[rows].float().cpu().numpy(), self.b[cols].float().cpu().numpy(),
                                  list(range(len(rows))), list(range(len(cols))), 1.0, None)
        tot = t.from_numpy(np.ascontiguousarray(part)).to(self.dev)
        if self.world > 1:
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        want = tot.cpu().numpy()[3 * self.rank:3 * self.rank + 3]
        got = self.c[local][:, cols].float().cpu().numpy()
        rms = float(np.sqrt(np.mean(want ** 2)))
        return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), rms / 128)))

    def _sampled_operands(self, rows, cols):
        """fp32 values (oracle arithmetic) of rows `rows` of A and rows `cols` of B, and the sampled bias."""
        np, O, t, w = self.np, self.O, self.torch, self.w
        idx = lambda v: t.as_tensor(v, device=self.dev)
        if w["kind"] == "bf16":
            bias = self.bias[idx(cols)].float().cpu().numpy() if self.bias is not None else None
            return self.a[idx(rows)].float().cpu().numpy(), self.b[idx(cols)].float().cpu().numpy(), bias
        if w["kind"] == "fp8":
            a = O.dequantize_fp8_rows(self.a[idx(rows)].cpu().numpy(), self.sa[idx(rows)].cpu().numpy())
            qb = O.e4m3_bits_to_f32(self.b[idx(cols)].cpu().numpy())
            sb = self.sb[idx([c // 128 for c in cols])].cpu().numpy()
            b = (qb.reshape(len(cols), self.k // 128, 128) * sb[:, :, None]).reshape(len(cols), self.k).astype(np.float32)
            return a, b, None
        kg = self.k // 64

        def nv(q, sf, g, rr):
            rr = np.asarray(rr)
            codes = O.unpack_e2m1(q[idx(rr)].cpu().numpy())
            blocks = sf.view(-1, kg, 512)[idx(rr // 128)].cpu().numpy()
            off = ((rr % 128) % 32) * 16 + ((rr % 128) // 32) * 4
            s_bits = np.stack([blocks[i, :, off[i]:off[i] + 4].reshape(-1) for i in range(len(rr))])
            return O.dequantize_nvfp4(codes, s_bits, g)
        return nv(self.a, self.sa, self.ga, rows), nv(self.b, self.sb, self.gb, cols), None

    def flops_total(self):
        w = self.w
        if w["shard"] == "n_weak":
            return 2.0 * w["m"] * w["n"] * w["k"] * self.world
        return 2.0 * w["m"] * w["n"] * w["k"]

    def check(self):
        """Sampled entries of this rank's output against the oracle in fp64 (untimed).  The operands are read back
        from the device as the bytes the kernel saw and turned into values by the oracle's own (de)quantisers."""
        if self.w["kind"] == "ksplit":
            return self._check_ksplit()
        np, O = self.np, self.O
        rows = [0, self.m // 2, self.m - 1]
        cols = list(range(0, self.n, 61))
        a, b, bias = self._sampled_operands(rows, cols)
        want = O.gemm_f64_entries(a, b, list(range(len(rows))), list(range(len(cols))), 1.0, bias)
        got = self.c[rows][:, cols].float().cpu().numpy()
        rms = float(np.sqrt(np.mean(want ** 2)))
        return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), rms / 128)))

    def close(self):
        try:
            self.plan.close()
        except Exception:
            pass


def roofline_peak(w, elapsed_ms):
    peaks = measured_peaks()
    ratio = NOMINAL_PEAK_TFLOPS[w["dtype"]] / NOMINAL_PEAK_TFLOPS["bf16"]
    if peaks:
        sustained = elapsed_ms >= 100.0       # back-to-back launches for 0.1 s or more run under the power cap
        base = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        note = (f"measured: cuBLAS bf16 8192^3 {'sustained' if sustained else 'burst'} figure of this pool "
                f"({base} TFLOP/s)" + (f" x {ratio:g} (nominal {w['dtype']}/bf16 tensor rate)" if ratio != 1 else ""))
        return base * ratio, note
    return FALLBACK_PEAK_TFLOPS * ratio, "fallback: no MEASURED_PEAKS.json"


def measure(name, w, rank, local_rank, world, dev, args, exchange="fused", extras=False):
    """Builds the workload, runs warm-up + the timed steps + burst + (K-split) split + end-to-end legs and the
    oracle check, reduces over the ranks (max) and returns the record (on every rank) plus the live workload."""
    import torch
    import torch.distributed as dist
    wl = Workload(name, w, rank, world, dev, exchange=exchange, tuning=args.tuning if name == args.workload else "",
                  tile_n=args.tile_n)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wl.step()
    sync_all()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # K-split: every timed step also records (start, GEMM done, exchange + cast done), so that the compute and the
    # exchange shares come from the same steps, under the same clocks, as the step time itself
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)] if w["kind"] == "ksplit" else None
    e0.record()
    for i in range(args.steps):
        if marks:
            wl.step(marks[i])
        else:
            wl.step()
    e1.record()
    sync_all()
    clocks = sampler.stop()
    elapsed_ms = e0.elapsed_time(e1)
    status = wl.plan.status()

    # ---- burst figure (the regime MEASURED_PEAKS calls "burst": a kernel timed alone, not under the sustained
    # power cap): after an idle gap, two untimed steps bring the clocks up and the third is timed; best of 10.
    burst_ms = []
    for _ in range(10):
        time.sleep(0.02)
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wl.step(); wl.step()
        b0.record(); wl.step(); b1.record()
        torch.cuda.synchronize()
        burst_ms.append(b0.elapsed_time(b1))
    sync_all()

    # ---- K-split: compute and communication separately, means over the timed steps
    split = None
    if marks:
        split = [sum(m[0].elapsed_time(m[1]) for m in marks) / len(marks), sum(m[1].elapsed_time(m[2]) for m in marks) / len(marks),
                 sum(m[1].elapsed_time(m[3]) for m in marks) / len(marks), sum(m[3].elapsed_time(m[2]) for m in marks) / len(marks)]

    # ---- end to end from pinned host buffers
    wl.e2e_step()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        wl.e2e_step()
    torch.cuda.synchronize()
    e2e_ms = 1e3 * (time.perf_counter() - t0)
    wl.step()                                     # the check reads the device-resident output of a plain step
    torch.cuda.synchronize()
    max_rel = wl.check()

    sp = split or [0.0, 0.0, 0.0, 0.0]
    vals = [elapsed_ms, e2e_ms, float(status), max_rel, min(burst_ms)] + sp + [-sp[0], -sp[2]]
    tt = torch.tensor(vals, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, status, max_rel, burst, gemm_ms, comm_ms, wait_ms, cast_ms, neg_gemm_min, neg_wait_min = tt.tolist()

    flops_step = wl.flops_total()
    ms_per_step = elapsed_ms / args.steps
    value = flops_step / (ms_per_step * 1e-3) / 1e12
    peak, peak_note = roofline_peak(w, elapsed_ms)
    kernel_ms = gemm_ms if split else ms_per_step
    kernel_tflops = flops_step / world / (kernel_ms * 1e-3) / 1e12
    nominal = NOMINAL_PEAK_TFLOPS[w["dtype"]]
    rec = {
        "value": value, "unit": "TFLOP/s", "ms_per_step": ms_per_step, "steps": args.steps, "warmup": args.warmup,
        "scaling": scaling_of(w), "dtype": w["dtype"], "config": workload_config(name, w, world, exchange, tile_n=args.tile_n),
        "pct_of_nominal_dense_peak": 100.0 * value / world / nominal,
        "burst": {"value": flops_step / (burst * 1e-3) / 1e12, "unit": "TFLOP/s",
                  "note": "best of 10 single steps, each after an idle gap and two untimed steps",
                  "pct_of_nominal_dense_peak": 100.0 * flops_step / world / (burst * 1e-3) / 1e12 / nominal},
        "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peak, "unit": "TFLOP/s",
                     "frac": kernel_tflops / peak, "traffic": TRAFFIC_BYTES.get(name),
                     "peak_source": peak_note, "kernel": wl.plan.spec.name,
                     "algorithmic_flops_per_launch": flops_step / world},
        "e2e": {"value": flops_step / (e2e_ms / args.e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "steps": args.e2e_steps,
                "ms_per_step": e2e_ms / args.e2e_steps, "api": wl.e2e_api,
                "per_rank_copy_gbs": (wl.h2d + wl.d2h) / (e2e_ms / args.e2e_steps * 1e-3) / 1e9},
        "gpu_launches": args.steps * wl.launches_per_step,
        "clocks": clocks,
        "kernel_status": int(status), "max_rel_err_vs_oracle_sample": max_rel,
        "stream_k_tail_workspace_bytes": int(getattr(wl, "tail_bytes", 0)),
    }
    if split:
        rec["ksplit"] = {"exchange": exchange if world > 1 else "none", "gemm_ms": gemm_ms,
                         "reduce_scatter_plus_cast_ms": comm_ms,
                         "exposed_after_gemm_ms": ms_per_step - gemm_ms,
                         # the part after the GEMM, split at the end of the barrier / collective; max and min over the
                         # ranks: a rank whose GEMM ends early spends the difference waiting in the barrier
                         "gemm_ms_min_rank": -neg_gemm_min, "barrier_or_collective_ms": wait_ms,
                         "barrier_or_collective_ms_min_rank": -neg_wait_min, "sum_cast_ms": cast_ms}
    return rec, wl, sync_all


def pcie_probe(wl, world, dev):
    """Achieved host->device and device->host GB/s of this rank's link with all ranks copying at once (what bounds
    the end-to-end leg): one plain copy of A up and of C back, CUDA events; min / max over the ranks."""
    import torch
    import torch.distributed as dist
    src, dst = (wl.a_host if hasattr(wl, "a_host") else wl.h_in[1]), wl.c_host     # (scaled workloads: the B operand)
    d_in = torch.empty_like(src, device=dev)
    d_out = torch.empty_like(dst, device=dev)
    out = []
    for h, d, up in ((src, d_in, True), (dst, d_out, False)):
        for _ in range(2):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world > 1:
                dist.barrier()
            ev0.record()
            (d.copy_(h, non_blocking=True) if up else h.copy_(d, non_blocking=True))
            ev1.record()
            torch.cuda.synchronize()
        out.append(h.numel() * h.element_size() / (ev0.elapsed_time(ev1) * 1e-3) / 1e9)
    t = torch.tensor([out[0], out[1], -out[0], -out[1]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mx0, mx1, mn0, mn1 = t.tolist()
    return {"h2d_gbs_per_rank": {"min": -mn0, "max": mx0}, "d2h_gbs_per_rank": {"min": -mn1, "max": mx1},
            "note": "all ranks copy at the same time; a per-rank figure that falls as N grows means the ranks share a "
                    "host-side limit (root complex / host DRAM), not their own PCIe link"}


def sustained_leg(fn, local_rank, seconds, flops_per_call):
    """Back-to-back calls for about `seconds`, NVML sampled every 2 ms: TFLOP/s, median SM MHz and the product
    time x clock (SM cycles per call), which separates idle cycles from a lower clock."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record(); torch.cuda.synchronize()
    n = max(20, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
    sampler = ClockSampler(local_rank, period_s=0.002)
    sampler.start()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / n
    rec = {"value": flops_per_call / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "calls": n, "seconds": ms * n * 1e-3,
           "ms_per_call": ms, "clocks": clocks}
    if clocks.get("sm_mhz"):
        rec["sm_cycles_per_call"] = ms * 1e-3 * clocks["sm_mhz"] * 1e6
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="bf16_8192_bias", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="tesserae_b200", choices=["tesserae_b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work per cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sub-configs", default=None, choices=["all", "none"],
                    help="also measure fp8_block, nvfp4 and bf16_ksplit in the same process (default: all for the "
                         "headline workload, none otherwise)")
    ap.add_argument("--sustained-seconds", type=float, default=1.0)
    ap.add_argument("--no-cublas-leg", action="store_true",
                    help="skip the same-process cuBLAS comparison and the one-second sustained legs (short runs under a profiler)")
    ap.add_argument("--tile-n", type=int, default=0, choices=[0, 256, 512],
                    help="bf16 workloads: columns of the CTA-pair tile (default 512: measured 4-5 %% ahead of 256 on the "
                         "headline and 16 %% on the K-split, where the step runs under the power cap)")
    ap.add_argument("--tuning", default="", help="tuning string of the main workload's kernel spec, e.g. GROUP_M=4 or TAIL_SPLITS=1")
    ap.add_argument("--ksplit-exchange", default="fused", choices=["reduce", "fused", "nccl"],
                    help="K-split at 2+ GPUs: tiles added into the owner's buffer by the GEMM's own stores (reduce), stored "
                         "to per-source slots and summed by the owner (fused), or NCCL reduce-scatter of plain partials")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(args.warmup, 3)
    if args.sub_configs is None:
        args.sub_configs = "all" if args.workload == "bf16_8192_bias" else "none"

    if args.impl == "reference":
        run_reference(args, w, rank)
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU: tesserae_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    rec, wl, sync_all = measure(args.workload, w, rank, local_rank, world, dev, args, exchange=args.ksplit_exchange)
    line = {"metric": "gemm_tflops", "value": rec["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": rec["scaling"],
            "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic (seeded Philox draws on the GPU; FP8 / NVFP4 operands made by the library's GPU quantisers)"}
    line.update({k: v for k, v in rec.items() if k not in ("value", "unit", "ms_per_step", "steps", "warmup", "scaling", "dtype")})

    # ---- where the end-to-end leg's time goes: achieved copy rates per rank with all ranks copying
    if w["kind"] != "ksplit":
        line["e2e"]["copy_probe"] = pcie_probe(wl, world, dev)

    # ---- the headline kernel against cuBLAS in the same process, both regimes, with the clock seen
    if w["kind"] == "bf16" and w["m"] >= 4096 and not args.no_cublas_leg:
        flops_one = 2.0 * wl.m * wl.n * wl.k
        bt = wl.b.t()
        cub = lambda: torch.matmul(wl.a, bt)
        burst = []
        for _ in range(10):
            time.sleep(0.02)
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            cub(); cub()
            b0.record(); cub(); b1.record()
            torch.cuda.synchronize()
            burst.append(b0.elapsed_time(b1))
        sync_all()
        ours_sus = sustained_leg(wl.step, local_rank, args.sustained_seconds, flops_one)
        sync_all()
        cub_sus = sustained_leg(cub, local_rank, args.sustained_seconds, flops_one)
        sync_all()
        line["sustained"] = ours_sus
        line["cublas_same_box"] = {"burst": flops_one / (min(burst) * 1e-3) / 1e12, "sustained": cub_sus["value"],
                                   "unit": "TFLOP/s per GPU", "sustained_detail": cub_sus,
                                   "note": "torch.matmul(A, B^T) bf16 on this rank's operands, no bias, same regimes as "
                                           "`burst` and `sustained` of this line"}
        line["vs_cublas_same_box"] = {"burst": (line["burst"]["value"] / world) / line["cublas_same_box"]["burst"],
                                      "sustained": ours_sus["value"] / cub_sus["value"]}
    wl.close()
    del wl
    torch.cuda.empty_cache()

    # ---- the other BASELINE configs, same process, same N
    if args.sub_configs == "all":
        subs = {}
        for name in SUB_CONFIGS:
            if name == args.workload:
                continue
            sw = WORKLOADS[name]
            try:
                srec, swl, _ = measure(name, sw, rank, local_rank, world, dev, args, exchange="fused")
                if sw["kind"] == "ksplit" and world > 1:
                    keep = ("value", "ms_per_step", "ksplit", "max_rel_err_vs_oracle_sample", "kernel_status",
                            "pct_of_nominal_dense_peak")
                    outs = {"fused": swl.c.clone()}
                    for other in ("reduce", "nccl"):
                        swl.close(); del swl
                        torch.cuda.empty_cache()
                        orec, swl, _ = measure(name, sw, rank, local_rank, world, dev, args, exchange=other)
                        outs[other] = swl.c.clone()
                        srec[other] = {k: orec[k] for k in keep}
                    flags = []
                    ref = outs["nccl"].float()
                    # one bf16 step at the largest output magnitude: a difference of that size is one rounding apart
                    step = float(torch.exp2(torch.floor(torch.log2(ref.abs().max().clamp_min(2.0 ** -100))) - 7))
                    for x in ("reduce", "fused"):
                        same = torch.equal(outs[x].view(torch.int16), outs["nccl"].view(torch.int16))
                        d = (outs[x].float() - ref).abs()
                        flags += [0.0 if same else 1.0, float(d.max()), float(d.max()) / step]
                    flags = torch.tensor(flags, dtype=torch.float64, device=dev)
                    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
                    for j, x in enumerate(("reduce", "fused")):
                        srec[f"{x}_equals_nccl"] = flags[3 * j].item() == 0.0
                        srec[f"{x}_vs_nccl_max_abs_diff"] = flags[3 * j + 1].item()
                        srec[f"{x}_vs_nccl_max_diff_in_bf16_steps_of_max_abs"] = flags[3 * j + 2].item()
                    srec["exchange_note"] = ("all three exchanges sum the same fp32 partials: `reduce` in the order the tiles "
                                             "arrive at the owner, `fused` in rank order, NCCL in its ring order; with 2 ranks "
                                             "the sums are equal to the bit, beyond that the bf16 results may differ in the "
                                             "last place")
                subs[name] = srec
                swl.close(); del swl
            except Exception as exc:                       # a sub-record must not take the headline down
                subs[name] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.empty_cache()
        line["configs"] = subs

    if rank == 0:
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_gemm_sample(w, budget_s=args.cpu_budget)[0]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
