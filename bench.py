#!/usr/bin/env python
"""Benchmark of the BitLinear hot path at the Llama-3-8B MLP shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--workload ...]

Headline workload ("llama3-8b-mlp", the second configuration of the target specification): hidden 4096,
intermediate 14336, 4096 tokens per GPU; the gate, up (4096 -> 14336) and down (14336 -> 4096) projections.
One step = for each projection: per-token int8 activation quantisation, the int8 x ternary forward,
dx = dy.W off the packed codes, and the STE gradient dW = dy^T.x.  Inputs are synthetic (seeded normal draws
of the stated shapes); weights are random latent f32 matrices ternarised by the absmean quantiser before the
timed region.

One JSON line is printed by rank 0.  `value` is tokens/s with every input resident in HBM; `e2e` is the same
metric through the host-buffer C-ABI entry point (pinned host memory, copies inside the timed region).  The
same line also carries, measured in the same process:
  hbm_kernels   (1 GPU only) the batch-1 and streaming kernels against the measured copy bandwidth, and the
                latency of the CPU-runnable 2048 x 2048 configuration;
  partitioned   the three partitioned configurations, strong scaling over the N GPUs of the run: the full QAT
                step over all linears of a Llama-3.2-1B-shaped decoder and of a Qwen3.5-9B-shaped hybrid decoder
                (8192 tokens per step split over the GPUs, quantiser inside the step, f32 dW summed over the GPUs),
                and one Llama-3-70B-shaped layer with output rows sharded.  At N > 1 every in-switch exchange is
                checked against NCCL (and against an exact integer pattern) before the timed steps; a mismatch
                ends the run with exit code 3.
`--impl reference` times the CPU restatement of the reference's own code path on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "alice-train_b200"))

WORKLOADS = {
    # name: (tokens per GPU, [(projection, out_features, in_features)])
    "llama3-8b-mlp": (4096, [("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]),
    "small": (1024, [("gate", 2048, 1024), ("down", 1024, 2048)]),
    # one Llama-3-70B-shaped decoder layer, 8192 tokens per STEP (rows of W sharded over the GPUs; rowshard_block)
    "llama3-70b-layer": (8192, [("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
                                ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672)]),
}
DECODER_WORKLOADS = ("llama32-1b-qat", "qwen35-9b-hybrid", "llama-tiny")
METRIC = "BitLinear fwd+bwd tokens/s at Llama-8B shape"
UNIT = "tokens/s"
NVLINK_ALLREDUCE_BUSBW_GBS = 725.0   # measured on this pool: 8-rank NCCL all-reduce bus bandwidth at 1 GiB
NVLINK_PEER_COPY_GBS = 770.0         # measured on this pool: peer copy per direction (nominal 900)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def dram_traffic(kernel: str, workload: str):
    """DRAM read + write bytes of one launch, from the ncu captures summarised under profiles/ (a text table:
    kernel, workload, bytes).  None when no capture of that kernel and workload has been recorded."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.txt")
    try:
        for line in open(path):
            f = line.split("#")[0].split()
            if len(f) >= 3 and f[0] == kernel and f[1] == workload:
                return float(f[2])
    except OSError:
        pass
    return None


def compact(o, digits=5):
    """Floats rounded to `digits` significant digits (the JSON line is read by people and by a log tail)."""
    if isinstance(o, float):
        return float(f"{o:.{digits}g}") if o == o and abs(o) != float("inf") else None
    if isinstance(o, dict):
        return {k: compact(v, digits) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [compact(v, digits) for v in o]
    return o


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU while a timed region runs.  Reads NVML from a thread every few
    milliseconds (the region is some tens of milliseconds long; `nvidia-smi -lms` starts too slowly to land samples in
    it) and keeps the samples taken between mark_begin() and mark_end(); falls back to an `nvidia-smi -lms 50` child
    process when NVML cannot be loaded.  Nothing is set, only read."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None
        self.thread, self.stop_flag, self.samples, self.t_begin, self.t_end, self.nvml = None, None, [], None, None, None

    def _nvml_handle(self):
        import pynvml
        import torch
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def _loop(self, nv, h):
        while not self.stop_flag.is_set():
            try:
                t = time.time()
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.samples.append((t, float(sm), pw, int(rs)))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            nv, h = self._nvml_handle()
            self.nvml = (nv, h, float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
            self.stop_flag = threading.Event()
            self.thread = threading.Thread(target=self._loop, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu), "-f", self.path],
                                         stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def stop(self) -> dict:
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            nv, _, mx = self.nvml
            inside = [x for x in self.samples if (self.t_begin is None or x[0] >= self.t_begin) and (self.t_end is None or x[0] <= self.t_end)]
            use = inside if inside else self.samples
            names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown), ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown), ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap))
            reasons = sorted({n for _, _, _, r in use for n, bit in names if r & bit})
            return {"sm_mhz": statistics.median([x[1] for x in use]) if use else None, "sm_max_mhz": mx,
                    "power_w_max": max([x[2] for x in use]) if use else None, "samples": len(use),
                    "sampled": "NVML every ~2 ms inside the timed region" if inside else "NVML, no sample fell inside the timed region",
                    "reasons": reasons}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        try:
            for line in open(self.path):
                f = [s.strip() for s in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                    pw.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "sampled": "nvidia-smi -lms 50 around the timed region",
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------- reference (CPU) arm
def cpu_step(orc, layers, tokens, seed=0, row_frac=1.0):
    """One pass of the reference's CPU code path over `tokens` tokens: for each projection the
    dense f32 products it runs on fake-quantised weights — tiled_matmul_bt (src/blas.rs:161-198)
    for the forward and matmul_bt_backward (src/llama_backward.rs:107-138) for dx and dW.
    Single-threaded, as those functions are in the reference.  `row_frac` < 1 runs the first
    ceil(out * row_frac) output rows of every projection only (the work of all three products is
    proportional to the rows), i.e. that fraction of a token's work.  Returns seconds."""
    t = 0.0
    for li, (_, out_full, inn, wq_full) in enumerate(layers):
        out = max(1, int(np.ceil(out_full * row_frac)))
        wq = wq_full if out == out_full else np.ascontiguousarray(wq_full[:out])
        g = np.random.Generator(np.random.Philox(1000 + seed + li))
        x = g.standard_normal((tokens, inn), dtype=np.float32)
        dy = (g.standard_normal((tokens, out), dtype=np.float32) * np.float32(1e-2)).astype(np.float32)
        dw = np.zeros((out, inn), np.float32)
        t0 = time.perf_counter()
        orc.matmul_bt(x, wq, tokens, out, inn, tiled=True)
        orc.lib.orc_matmul_bt_backward(dy.reshape(-1), x.reshape(-1), wq.reshape(-1),
                                       np.zeros(tokens * inn, np.float32).ctypes.data_as(C.c_void_p),
                                       dw.reshape(-1).ctypes.data_as(C.c_void_p), tokens, out, inn)
        t += time.perf_counter() - t0
    return t


def cpu_layers(orc, projs):
    layers = []
    for li, (name, out, inn) in enumerate(projs):
        g = np.random.Generator(np.random.Philox(10 + li))
        w = (g.standard_normal((out, inn), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        _, wq = orc.fq_vec(w, threads=orc.max_threads())  # rayon in the reference: all cores
        layers.append((name, out, inn, wq.reshape(out, inn)))
    return layers


def cpu_sample_plan(orc, layers, projs, tokens, budget_s, passes):
    """Fraction of every projection's output rows to run so that `passes` passes over `tokens` tokens take about
    `budget_s` seconds.  A short calibration pass (1/256 of the rows) gives a lower bound of the cost, a fixed figure of
    1.3e-8 s per weight and token (what the strided loops of matmul_bt_backward cost once the matrix no longer fits
    the caches) an upper one; one trial pass at the planned size then corrects the plan if it still overshoots."""
    weights = sum(o * i for _, o, i in projs)
    cal = 1.0 / 256.0
    secs = cpu_step(orc, layers, tokens, seed=55, row_frac=cal)
    done = sum(max(1, int(np.ceil(o * cal))) * i for _, o, i in projs) / weights
    full = max(secs / done, 1.3e-8 * weights * tokens)      # seconds for all rows, `tokens` tokens
    target = budget_s / max(passes, 1)
    frac = min(1.0, max(1.0 / 512.0, target / full))
    trial = cpu_step(orc, layers, tokens, seed=56, row_frac=frac)
    if trial > 1.3 * target:
        frac = max(1.0 / 512.0, frac * target / trial)
    return frac


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import pyoracle as orc
    tokens_full, projs = WORKLOADS[args.workload]
    layers = cpu_layers(orc, projs)
    sample = min(args.cpu_tokens, tokens_full)
    row_frac = cpu_sample_plan(orc, layers, projs, sample, 100.0, args.steps + args.warmup)
    for i in range(args.warmup):
        cpu_step(orc, layers, sample, seed=i, row_frac=row_frac)
    times = [cpu_step(orc, layers, sample, seed=100 + i, row_frac=row_frac) for i in range(args.steps)]
    total = sum(times)
    rows_done = sum(max(1, int(np.ceil(o * row_frac))) * i for _, o, i in projs) / sum(o * i for _, o, i in projs)
    value = sample * rows_done * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_gpu": tokens_full, "projections": {n: [o, i] for n, o, i in projs},
                   "parallelism": "host cores (rank 0 only)",
                   "step": "per projection: forward, dx, dW of the reference's CPU code path on fake-quantised f32 weights",
                   "note": f"each step is a bounded sample: {sample} tokens through {100 * rows_done:.2f} % of every projection's output rows, scaled linearly"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "host_cores": os.cpu_count(), "kind": "port",
                         "sample": f"{sample} of {tokens_full} tokens per step through {100 * rows_done:.2f} % of the output rows of "
                                   f"all projections (fwd tiled_matmul_bt + matmul_bt_backward), single thread as those functions are in "
                                   f"the reference; oracle built -O3 with hardware FMA; weights fake-quantised with {orc.max_threads()} threads outside the timed region"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(compact(line, 6)), flush=True)
    return 0


# ------------------------------------------------------------------------------ environment
class Env:
    """Process-wide state of a native run: rank, device, process group, library context."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        import alice_train
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a B200: the library has no CPU path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.ctx = alice_train.GpuContext.on_torch_stream(self.local)
        self.pk = peaks()

    def fence(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        t = self.torch.tensor([v], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        t = self.torch.tensor([0 if ok else 1], device=self.dev, dtype=self.torch.int32)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return int(t.item()) == 0

    def close(self):
        if self.world > 1 and not getattr(self, "_closed", False):
            self._closed = True
            self.dist.destroy_process_group()


def timed_steps(env, step, steps, warmup):
    """`warmup` untimed steps, then exactly `steps` steps between fences; CUDA events; max over ranks.  ms total."""
    torch = env.torch
    for _ in range(warmup):
        step()
    env.fence()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    env.fence()
    return env.max_over_ranks(t0.elapsed_time(t1))


# ----------------------------------------------------------------------------- headline workload
def run_main(env, args):
    torch, dist = env.torch, env.dist
    from alice_train import _ffi, bitlinear as bl

    world, rank, dev, ctx, pk = env.world, env.rank, env.dev, env.ctx, env.pk
    tokens, projs = WORKLOADS[args.workload]

    # ---- set-up (untimed): latent weights -> codes, inputs resident in HBM
    gen = torch.Generator(device=dev)
    layers = []
    for li, (name, out, inn) in enumerate(projs):
        gen.manual_seed(10 + li)  # identical weights on every rank (data parallel)
        w_lat = torch.randn((out, inn), generator=gen, device=dev, dtype=torch.float32) * 0.02
        h = bl.BitLinearWeights(out, inn, ctx).quantize_(w_lat)
        del w_lat
        gen.manual_seed(1000 + 97 * rank + li)  # each rank has its own tokens
        x = torch.randn((tokens, inn), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        dy = (torch.randn((tokens, out), generator=gen, device=dev, dtype=torch.float32) * 1e-2).to(torch.bfloat16)
        layers.append(dict(
            name=name, out=out, inn=inn, w=h, x=x, dy=dy,
            qa=bl.QuantizedActivations(torch.empty((tokens, inn), dtype=torch.int8, device=dev),
                                       torch.empty(tokens, dtype=torch.float32, device=dev),
                                       torch.empty(tokens, dtype=torch.int32, device=dev)),
            y=torch.empty((tokens, out), dtype=torch.bfloat16, device=dev),
            dx=torch.empty((tokens, inn), dtype=torch.bfloat16, device=dev),
            dW=torch.zeros((out, inn), dtype=torch.float32, device=dev)))
    ctx.sync()
    # data parallel: dW lives in symmetric memory and is summed inside NVSwitch by the library's own kernel;
    # NCCL remains the exchange where the GPUs have no multicast mapping (or on request)
    switch, exchange, exchange_check = None, "none", None
    if world > 1:
        exchange = "nccl"
        if args.dw_exchange == "switch":
            try:
                from alice_train import parallel
                switch = parallel.SwitchDwAllReducer(ctx, [(L["out"], L["inn"]) for L in layers], dev, ctas=args.exchange_ctas)
                for L, buf in zip(layers, switch.dW):
                    L["dW"] = buf
                exchange = "switch"
            except RuntimeError as e:
                if rank == 0:
                    print(f"[bench] in-switch exchange unavailable ({e}); using NCCL", file=sys.stderr)

    classes = ("act_quant", "fwd", "dx", "dw")
    ev = {c: [] for c in classes}

    def step(record: bool):
        handles = []
        for li, L in enumerate(layers):
            def timed(cls, fn):
                if record:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    fn()
                    b.record()
                    ev[cls].append((a, b, L["name"]))
                else:
                    fn()
            # dW first: its all-reduce (data parallel runs) then overlaps this projection's other kernels
            timed("dw", lambda: bl.ste_dw(ctx, L["dy"], L["x"], L["dW"], beta=0.0))
            if switch is not None:  # data parallel over tokens: the one exchange step is the sum of dW
                switch.submit(li)
            elif world > 1:
                handles.append(dist.all_reduce(L["dW"], op=dist.ReduceOp.SUM, async_op=True))
            timed("act_quant", lambda: bl.act_quant_int8(ctx, L["x"], L["qa"]))
            timed("fwd", lambda: bl.bitlinear_fwd(L["w"], L["qa"], y=L["y"]))
            timed("dx", lambda: bl.bitlinear_dx(L["w"], L["dy"], dx=L["dx"]))
        for hnd in handles:
            hnd.wait()
        if switch is not None:
            switch.wait()

    for _ in range(args.warmup):
        step(False)
    # correctness of the in-switch sum, before anything is timed: every dW buffer is summed a second time by NCCL
    # from a copy; the two must agree (bit for bit at 2 GPUs; the reductions add in different orders beyond that)
    if switch is not None:
        worst, same = 0.0, 0
        ok = True
        for li, L in enumerate(layers):
            bl.ste_dw(ctx, L["dy"], L["x"], L["dW"], beta=0.0)
            ctx.sync()
            ref = L["dW"].clone()
            dist.all_reduce(ref, op=dist.ReduceOp.SUM)
            switch.submit(li)
            switch.wait()
            ctx.sync()
            diff, scale = (L["dW"] - ref).abs().max().item(), ref.abs().max().item()
            same += int(torch.equal(L["dW"], ref))
            worst = max(worst, diff / scale if scale > 0 else 0.0)
            if diff > 1e-6 * scale or (world == 2 and diff != 0.0):
                ok = False
            del ref
        exchange_check = {"buffers": len(layers), "vs_nccl_bit_identical": same, "vs_nccl_max_rel_diff": worst}
        if not env.all_ok(ok):
            raise ExchangeMismatch(f"in-switch all-reduce of dW differs from NCCL: {exchange_check}")
    sampler = ClockSampler(env.local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    env.fence()
    launches0 = ctx.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    env.fence()
    sampler.mark_end()
    launches = ctx.launch_count() - launches0
    ms_total = env.max_over_ranks(t0.elapsed_time(t1))
    clocks = sampler.stop() if rank == 0 else None
    ctx.sync()

    # ---- per-kernel-class device times measured inside the timed region
    per = {}
    for c in classes:
        ts = [a.elapsed_time(b) for a, b, _ in ev[c]]
        per[c] = {"launches": len(ts), "ms_total": sum(ts), "ms_avg": sum(ts) / max(len(ts), 1)}
    ops_per_launch = 2.0 * tokens * sum(o * i for _, o, i in projs) / len(projs)  # average over projections
    for c in ("fwd", "dx", "dw"):
        per[c]["tops_avg"] = ops_per_launch / (per[c]["ms_avg"] * 1e-3) / 1e12 if per[c]["ms_avg"] > 0 else None
    aq_bytes = sum(tokens * i * 3 + tokens * 8 for _, _, i in projs) / len(projs)
    per["act_quant"]["gbs_avg"] = aq_bytes / (per["act_quant"]["ms_avg"] * 1e-3) / 1e9 if per["act_quant"]["ms_avg"] > 0 else None
    per["act_quant"]["frac_of_hbm"] = per["act_quant"]["gbs_avg"] / pk["hbm_gbs"] if per["act_quant"]["gbs_avg"] else None
    # tensor-pipe ceilings at the clocks this GPU holds: MMA-only kernels of the production tile shape
    probe = {}
    for kind, key in ((1, "int8_tops"), (0, "bf16_tflops")):
        ops = C.c_double(0.0)
        best = None
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            _ffi.check(_ffi.load().ab_tensor_peak_probe(ctx.handle, kind, 4000, C.byref(ops)), ctx.handle)
            b.record()
            torch.cuda.synchronize()
            t = a.elapsed_time(b)
            best = t if best is None else min(best, t)
        probe[key] = ops.value / (best * 1e-3) / 1e12
    ctx.sync()
    # Which measured cuBLAS figure is the honest denominator depends on the regime the timed region ran in: a region
    # shorter than about a second that never saw the power cap ran at burst clocks (compare bf16_tflops); a long,
    # power-capped one ran sustained (compare bf16_tflops_sustained).  Both fractions are printed, and the fraction
    # of the MMA-only probe beside them (what the tensor pipe could do with operands already in shared memory).
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    regime = "sustained" if (ms_total >= 1000.0 and capped) else "burst"
    bf16_peak = pk["bf16_tflops_sustained"] if regime == "sustained" else pk["bf16_tflops"]
    fr = {}
    for c in ("fwd", "dx", "dw"):
        a = per[c]["tops_avg"]
        mult = 2.0 if c == "fwd" else 1.0    # no int8 figure is measured on this pool: twice the bf16 rate, as the hardware's
        fr[c] = {"frac_burst": a / (mult * pk["bf16_tflops"]), "frac_sustained": a / (mult * pk["bf16_tflops_sustained"]),
                 "frac_probe": a / (probe["int8_tops"] if c == "fwd" else probe["bf16_tflops"])}
    dom = max(("fwd", "dx", "dw"), key=lambda c: per[c]["ms_total"])
    kernel_names = {"fwd": "gemm_pair_kernel<FWD / FWT> int8 x ternary (weights in tensor memory from 8192 input features)",
                    "dx": "gemm_pair_kernel<DXT> bf16 x ternary (expanded weights in tensor memory)",
                    "dw": "gemm_pair_kernel<DW> bf16 x bf16"}
    peak = (2.0 if dom == "fwd" else 1.0) * bf16_peak
    roofline = {"bound": "tensor", "kernel": kernel_names[dom], "achieved": per[dom]["tops_avg"], "peak": peak, "unit": "TFLOP/s",
                "frac": per[dom]["tops_avg"] / peak, "traffic": dram_traffic(dom, args.workload),
                "frac_burst": fr[dom]["frac_burst"], "frac_sustained": fr[dom]["frac_sustained"], "frac_probe": fr[dom]["frac_probe"],
                "regime": f"{regime} ({ms_total:.0f} ms timed, power cap {'seen' if capped else 'not seen'})",
                "peak_source": f"{pk['source']} cuBLAS bf16 {regime} {bf16_peak} TFLOP/s" + (" x 2 (int8)" if dom == "fwd" else ""),
                "algorithmic_ops_per_launch": ops_per_launch}

    value = world * tokens * args.steps / (ms_total * 1e-3)

    # ---- end to end through the host-buffer C-ABI entry point (pinned memory, copies timed)
    e2e = None
    if not args.no_e2e:
        host = []
        for L in layers:
            host.append(dict(x=L["x"].cpu().pin_memory(), dy=L["dy"].cpu().pin_memory(),
                             y=torch.empty((tokens, L["out"]), dtype=torch.bfloat16).pin_memory(),
                             dx=torch.empty((tokens, L["inn"]), dtype=torch.bfloat16).pin_memory()))
        lib = _ffi.load()
        # what one PCIe direction carries here: a 256 MiB pinned copy each way, alone
        pcie = {}
        probe_d = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        probe_h = torch.empty(256 << 20, dtype=torch.uint8).pin_memory()
        for name, (dst, src) in (("h2d_gbs", (probe_d, probe_h)), ("d2h_gbs", (probe_h, probe_d))):
            dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            pcie[name] = (256 << 20) / (a.elapsed_time(b) * 1e-3) / 1e9
        del probe_d, probe_h

        # calls only queue their work (AB_OPT_ASYNC_HOST_STEP) and the step ends with one sync, so the copies in of
        # one projection overlap the GEMMs and copies out of the one before; the projection with the largest dx
        # (down) goes first so that the step does not end on its copy out
        ctx.set_async_host_step(True)
        order = sorted(range(len(layers)), key=lambda i: -layers[i]["inn"])

        def e2e_step():
            pending = []
            for li in order:
                L, Hh = layers[li], host[li]
                _ffi.check(lib.ab_bitlinear_step_host(ctx.handle, L["w"].handle, C.c_void_p(Hh["x"].data_ptr()),
                                                      C.c_void_p(Hh["dy"].data_ptr()), tokens,
                                                      C.c_void_p(Hh["y"].data_ptr()), C.c_void_p(Hh["dx"].data_ptr()),
                                                      C.c_void_p(L["dW"].data_ptr())), ctx.handle)
                if switch is not None:      # the data-parallel sum of dW belongs to the step end to end as well
                    switch.submit(li)
                elif world > 1:
                    pending.append(dist.all_reduce(L["dW"], op=dist.ReduceOp.SUM, async_op=True))
            for hnd in pending:
                hnd.wait()
            if switch is not None:
                switch.wait()
            ctx.sync()
        e2e_steps = max(2, min(args.steps, 5))
        e2e_step()
        env.fence()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        env.fence()
        dt = env.max_over_ranks(time.perf_counter() - w0)
        h2d = sum(tokens * (i + o) * 2 for _, o, i in projs)
        per_dir = h2d * e2e_steps / dt / 1e9
        e2e = {"value": world * tokens * e2e_steps / dt, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": h2d, "steps": e2e_steps,
               "pcie": {"h2d_gbs_alone": pcie["h2d_gbs"], "d2h_gbs_alone": pcie["d2h_gbs"], "achieved_gbs_each_way": per_dir,
                        "frac_of_pinned_copy": per_dir / min(pcie["h2d_gbs"], pcie["d2h_gbs"])},
               "note": "ab_bitlinear_step_host per projection (queued, one sync per step): x, dy in and y, dx out as bf16 through pinned host memory, both directions at once; dW stays on the device"}
        ctx.set_async_host_step(False)
        del host

    # ---- CPU baseline (oracle port), rank 0 at N = 1 only, bounded sample
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import pyoracle as orc
        cl = cpu_layers(orc, projs)
        sample = min(args.cpu_tokens, tokens)
        row_frac = cpu_sample_plan(orc, cl, projs, sample, 15.0, 1)
        secs = cpu_step(orc, cl, sample, seed=7, row_frac=row_frac)
        rows_done = sum(max(1, int(np.ceil(o * row_frac))) * i for _, o, i in projs) / sum(o * i for _, o, i in projs)
        cpu_baseline = {"value": sample * rows_done / secs, "unit": UNIT, "cores": 1, "host_cores": os.cpu_count(), "kind": "port",
                        "sample": f"{sample} of {tokens} tokens through {100 * rows_done:.2f} % of every projection's output rows "
                                  f"(fwd tiled_matmul_bt + matmul_bt_backward on fake-quantised f32 weights), {secs:.1f} s, single thread "
                                  f"as those functions are in the reference, oracle built -O3 with hardware FMA"}
        del cl

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 forward (s32 accumulate), bf16 backward (f32 accumulate)", "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_gpu": tokens,
                       "projections": {n: [o, i] for n, o, i in projs},
                       "parallelism": f"dp{world}" if world > 1 else "single",
                       "step": "per projection: dW (overwrite), act-quant int8, fwd, dx" +
                               {"switch": "; each dW summed over the GPUs inside NVSwitch (multimem kernel of the library) right after its GEMM, overlapping the rest",
                                "nccl": "; NCCL all-reduce of each dW issued right after its GEMM, overlapping the rest", "none": ""}[exchange],
                       "dw_exchange": exchange,
                       "l2": "working set per step exceeds the 126 MB L2 (dW alone is 3 x 235 MB); no explicit flush"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "kernels": per, "tensor_pipe_probe": probe, "fractions": fr,
            "tops_total": 6.0 * tokens * sum(o * i for _, o, i in projs) * args.steps / (ms_total * 1e-3) / 1e12,
        }
        if exchange_check is not None:
            line["exchange_check"] = exchange_check
    for L in layers:
        L["w"].close()
    del layers, switch
    torch.cuda.empty_cache()
    return line


# ------------------------------------------------------- memory-bound kernels (batch-1 path)
def hbm_block(env, full: bool = True):
    """Batch-1 and streaming kernels against the measured HBM copy bandwidth.  Every packed weight
    matrix of the target configurations fits the 126 MB L2, so the matvec kernels rotate over
    enough distinct matrices to exceed it (cold L2); the L2-resident figure is reported beside it."""
    torch = env.torch
    import alice_train
    from alice_train import _ffi, bitlinear as bl

    dev = env.dev
    # everything runs on one explicit stream so that the timed launch sequences can be captured into CUDA graphs:
    # these kernels take 10-50 us, less than the Python + ctypes cost of issuing one, and a replayed graph times the
    # device, not the host
    stream = torch.cuda.Stream(device=dev)
    prev = torch.cuda.current_stream(dev)
    torch.cuda.set_stream(stream)
    try:
        ctx = alice_train.GpuContext.on_torch_stream(env.local)
        lib = _ffi.load()
        pk = env.pk
        out, inn = 28672, 8192  # the largest single matrix of the target configurations (70B-shape gate projection)
        nmat = 8  # 8 x 56 MiB of canonical codes = 448 MiB > 3 x L2; launches long enough that the host stays ahead
        gen = torch.Generator(device=dev)
        gen.manual_seed(5)
        mats = []
        for i in range(nmat):
            w_lat = torch.randn((out, inn), generator=gen, device=dev) * 0.02
            mats.append(bl.BitLinearWeights(out, inn, ctx).quantize_(w_lat))
            del w_lat
        x = torch.randn(inn, generator=gen, device=dev)
        dy = torch.randn(out, generator=gen, device=dev)
        y = torch.empty(out, device=dev)
        dx = torch.empty(inn, device=dev)
        dW = torch.zeros((8192, 8192), device=dev)
        ctx.sync()
        vp = lambda t: C.c_void_p(t.data_ptr())

        timing = {"mode": "cuda-graph replay"}

        def timeit(fn, reps, rotate):
            for i in range(3):
                fn(mats[i % len(mats)])
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(reps):
                        fn(mats[i % nmat] if rotate else mats[0])
                graph.replay()
                torch.cuda.synchronize()
                a.record()
                graph.replay()
                b.record()
                torch.cuda.synchronize()
                return a.elapsed_time(b) / reps * 1e-3
            except Exception as e:  # capture refused: time the launch loop itself
                timing["mode"] = f"launch loop (graph capture failed: {type(e).__name__})"
                torch.cuda.synchronize()
                a.record()
                for i in range(reps):
                    fn(mats[i % nmat] if rotate else mats[0])
                b.record()
                torch.cuda.synchronize()
                return a.elapsed_time(b) / reps * 1e-3

        code_bytes = out * inn / 4
        res = {}
        cases = {
            "matvec_fwd": (lambda w: _ffi.check(lib.ab_ternary_matvec(ctx.handle, w.handle, vp(x), vp(y)), ctx.handle),
                           code_bytes + 4 * (out + inn)),
            "matvec_bwd": (lambda w: _ffi.check(lib.ab_ternary_matvec_backward(ctx.handle, w.handle, vp(dy), vp(dx)), ctx.handle),
                           code_bytes + 4 * (out + inn)),
            "bitlinear_backward_prenorm": (lambda w: _ffi.check(lib.ab_bitlinear_backward(ctx.handle, w.handle, vp(x), vp(dy), 1, 1e-6, vp(dx), None), ctx.handle),
                                           code_bytes + 4 * (2 * out + 2 * inn)),
        }
        for name, (fn, nbytes) in cases.items():
            cold = timeit(fn, 6 * nmat, True)
            warm = timeit(fn, 6 * nmat, False)
            res[name] = {"us": cold * 1e6, "gbs": nbytes / cold / 1e9, "frac": nbytes / cold / 1e9 / pk["hbm_gbs"],
                         "l2_us": warm * 1e6}
        if full:
            # the same three entry points with AB_OPT_EXACT_MATVEC: f32 adds on the CUDA cores, as the reference's loops do
            ctx.set_exact_matvec(True)
            for name, (fn, nbytes) in cases.items():
                cold = timeit(fn, 2 * nmat, True)
                res[name + "_f32"] = {"us": cold * 1e6, "gbs": nbytes / cold / 1e9, "frac": nbytes / cold / 1e9 / pk["hbm_gbs"]}
            ctx.set_exact_matvec(False)
        t = timeit(lambda w: _ffi.check(lib.ab_ste_weight_grad(ctx.handle, vp(x), 8192, vp(dy), 8192, vp(dW)), ctx.handle), 20, False)
        nb = 8.0 * 8192 * 8192 + 4 * (8192 + 8192)
        res["ste_weight_grad"] = {"us": t * 1e6, "gbs": nb / t / 1e9, "frac": nb / t / 1e9 / pk["hbm_gbs"]}
        for m in mats[1:]:
            m.close()
        del mats[1:]
        # kernel (1) at the Llama-3-8B gate shape (235 MB of latent weights, above L2)
        w_lat = torch.randn((14336, 4096), generator=gen, device=dev) * 0.02
        hq = bl.BitLinearWeights(14336, 4096, ctx)
        t = timeit(lambda w: hq.quantize_(w_lat), 20, False)
        nb = 4.25 * 14336 * 4096
        res["fq_absmean_pack"] = {"us": t * 1e6, "gbs": nb / t / 1e9, "frac": nb / t / 1e9 / pk["hbm_gbs"]}
        xa = torch.randn((4096, 14336), generator=gen, device=dev).to(torch.bfloat16)
        qa = bl.act_quant_int8(ctx, xa)
        t = timeit(lambda w: bl.act_quant_int8(ctx, xa, qa), 20, False)
        nb = 4096 * 14336 * 3 + 8 * 4096
        res["act_quant_int8"] = {"us": t * 1e6, "gbs": nb / t / 1e9, "frac": nb / t / 1e9 / pk["hbm_gbs"]}
        # the steps either side of the linears, fused with the activation quantiser, and the optimizer fused with kernel (1)
        if full:
            nw = 14336 * 4096
            flat, grad = w_lat.view(-1), torch.randn(nw, generator=gen, device=dev) * 1e-3
            t = timeit(lambda w: bl.sgd_step_fq(ctx, flat, grad, 1e-4, 0.0, hq), 10, False)
            res["sgd_step_fq"] = {"us": t * 1e6, "gbs": (12.0 + 0.25) * nw / t / 1e9, "frac": (12.0 + 0.25) * nw / t / 1e9 / pk["hbm_gbs"],
                                  "note": "w, g read + w written + codes; the separate quantiser call of the next step is saved"}
            am, av = torch.zeros(nw, device=dev), torch.zeros(nw, device=dev)
            t = timeit(lambda w: bl.adamw_step_fq(ctx, flat, grad, am, av, 1e-4, 3, weights=hq), 10, False)
            res["adamw_step_fq"] = {"us": t * 1e6, "gbs": (28.0 + 0.25) * nw / t / 1e9, "frac": (28.0 + 0.25) * nw / t / 1e9 / pk["hbm_gbs"]}
            del grad, am, av
            xn = torch.randn((4096, 4096), generator=gen, device=dev).to(torch.bfloat16)
            wn = torch.ones(4096, device=dev)
            _, qn = bl.rmsnorm_act_quant(ctx, xn, wn, 1e-5)
            t = timeit(lambda w: bl.rmsnorm_act_quant(ctx, xn, wn, 1e-5, None, qn), 20, False)
            nb = 4096 * 4096 * 3 + 12 * 4096
            res["rmsnorm_act_quant"] = {"us": t * 1e6, "gbs": nb / t / 1e9, "frac": nb / t / 1e9 / pk["hbm_gbs"]}
            gate = torch.randn((4096, 14336), generator=gen, device=dev).to(torch.bfloat16)
            _, qs = bl.swiglu_act_quant(ctx, gate, xa)
            t = timeit(lambda w: bl.swiglu_act_quant(ctx, gate, xa, None, qs), 20, False)
            nb = 4096 * 14336 * 5 + 12 * 4096
            res["swiglu_act_quant"] = {"us": t * 1e6, "gbs": nb / t / 1e9, "frac": nb / t / 1e9 / pk["hbm_gbs"]}
            del xn, gate
            # the forward of one Llama-3-8B MLP block on 4096 tokens, RMSNorm in front: fused (the norm and SwiGLU hand int8
            # activations straight to the GEMMs) against the same chain with the activations written as bf16 and quantised
            # by separate act-quant launches
            hid, inter, tok = 4096, 14336, 4096
            xin = torch.randn((tok, hid), generator=gen, device=dev).to(torch.bfloat16)
            nw_ = torch.ones(hid, device=dev)
            wg, wu, wd = (bl.BitLinearWeights(o, i, ctx).quantize_(torch.randn((o, i), generator=gen, device=dev) * 0.02)
                          for o, i in ((inter, hid), (inter, hid), (hid, inter)))
            g_out = torch.empty((tok, inter), dtype=torch.bfloat16, device=dev)
            u_out = torch.empty((tok, inter), dtype=torch.bfloat16, device=dev)
            y_out = torch.empty((tok, hid), dtype=torch.bfloat16, device=dev)
            xn_bf = torch.empty((tok, hid), dtype=torch.bfloat16, device=dev)
            mid_bf = torch.empty((tok, inter), dtype=torch.bfloat16, device=dev)
            _, q_in = bl.rmsnorm_act_quant(ctx, xin, nw_, 1e-5)
            _, q_mid = bl.swiglu_act_quant(ctx, g_out, u_out)

            def fused(_w):
                bl.rmsnorm_act_quant(ctx, xin, nw_, 1e-5, None, q_in)
                bl.bitlinear_fwd(wg, q_in, g_out)
                bl.bitlinear_fwd(wu, q_in, u_out)
                bl.swiglu_act_quant(ctx, g_out, u_out, None, q_mid)
                bl.bitlinear_fwd(wd, q_mid, y_out)

            def unfused(_w):
                bl.rmsnorm_act_quant(ctx, xin, nw_, 1e-5, xn_bf, None, quantize=False)
                bl.act_quant_int8(ctx, xn_bf, q_in)
                bl.bitlinear_fwd(wg, q_in, g_out)
                bl.bitlinear_fwd(wu, q_in, u_out)
                bl.swiglu_act_quant(ctx, g_out, u_out, mid_bf, None, quantize=False)
                bl.act_quant_int8(ctx, mid_bf, q_mid)
                bl.bitlinear_fwd(wd, q_mid, y_out)

            tf, tu = timeit(fused, 6, False), timeit(unfused, 6, False)
            res["mlp_forward_chain"] = {"tokens": tok, "fused_us": tf * 1e6, "unfused_us": tu * 1e6, "tokens_per_s_fused": tok / tf,
                                        "note": "rmsnorm -> gate, up -> swiglu -> down; fused = norm and SwiGLU emit the int8 activations themselves"}
            for hnd in (wg, wu, wd):
                hnd.close()
            del xin, g_out, u_out, y_out, xn_bf, mid_bf
        # the CPU-runnable configuration: one 2048 x 2048 layer, batch 1 (1 MiB of codes: latency, not bandwidth)
        g1 = torch.randn((2048, 2048), generator=gen, device=dev) * 0.02
        h1 = bl.BitLinearWeights(2048, 2048, ctx).quantize_(g1)
        x1, dy1 = torch.randn(2048, generator=gen, device=dev), torch.randn(2048, generator=gen, device=dev)
        dx1, dW1 = torch.empty(2048, device=dev), torch.zeros((2048, 2048), device=dev)
        c1 = {
            "matvec_bwd_us": timeit(lambda w: _ffi.check(lib.ab_ternary_matvec_backward(ctx.handle, h1.handle, vp(dy1), vp(dx1)), ctx.handle), 40, False) * 1e6,
            "bitlinear_backward_prenorm_us": timeit(lambda w: _ffi.check(lib.ab_bitlinear_backward(ctx.handle, h1.handle, vp(x1), vp(dy1), 1, 1e-6, vp(dx1), None), ctx.handle), 40, False) * 1e6,
            "ste_weight_grad_us": timeit(lambda w: _ffi.check(lib.ab_ste_weight_grad(ctx.handle, vp(x1), 2048, vp(dy1), 2048, vp(dW1)), ctx.handle), 40, False) * 1e6,
        }
        ctx.sync()
        hq.close(); h1.close(); mats[0].close()
        return {"matrix": [out, inn], "rotation_mib": nmat * code_bytes / 2**20, "timing": timing["mode"], "peak_gbs": pk["hbm_gbs"],
                "peak_source": pk["source"] + " copy bandwidth", "kernels": res, "single_layer_2048": c1,
                "note": "us = cold (rotation over distinct matrices), l2_us = one matrix re-used; frac = algorithmic bytes / time / peak; fq scored on 4.25 B/weight"}
    finally:
        torch.cuda.set_stream(prev)
        torch.cuda.empty_cache()


# --------------------------------------------- full QAT step over all linears of a decoder (data parallel)
def decoder_block(env, name, args, steps, warmup):
    """configs[2] / configs[3] of the target specification: tokens of one step split over the GPUs (strong scaling),
    kernel (1) on every linear inside the step, f32 dW of every linear summed over the GPUs."""
    torch = env.torch
    from alice_train import decoder_step as ds
    tokens_step, layers, std, guard = ds.MODELS[name]()
    world = env.world
    assert tokens_step % world == 0
    tokens = tokens_step // world
    exchange = "none" if world == 1 else args.dw_exchange
    ctas = args.partitioned_ctas
    try:
        plan = ds.DataParallelQatStep(env.ctx, layers, tokens, env.dev, weight_std=std, guard=guard, exchange=exchange, ctas=ctas)
    except RuntimeError as e:
        if exchange != "switch":
            raise
        if env.rank == 0:
            print(f"[bench] {name}: in-switch exchange unavailable ({e}); using NCCL", file=sys.stderr)
        exchange = "nccl"
        plan = ds.DataParallelQatStep(env.ctx, layers, tokens, env.dev, weight_std=std, guard=guard, exchange=exchange, ctas=ctas)
    out = {"tokens_per_step": tokens_step, "tokens_per_gpu": tokens, "linears": len(plan.linears), "params": plan.params,
           "scaling": "strong", "exchange": plan.exchange}
    check = None
    if plan.exchange == "switch":
        plan.step()
        env.ctx.sync()
        ok = True
        try:
            check = plan.check_exchange(max_linears=args.check_linears)
        except RuntimeError as e:
            ok, check = False, {"error": str(e)}
        if not env.all_ok(ok):
            raise ExchangeMismatch(f"{name}: {check}")
        plan.resync_epochs()
    launches0 = env.ctx.launch_count()
    ms = timed_steps(env, plan.step, steps, warmup) / steps
    out["gpu_launches_per_step"] = int((env.ctx.launch_count() - launches0) / (steps + warmup))
    out["ms_per_step"] = ms
    out["tokens_per_s"] = tokens_step / (ms * 1e-3)
    out["tflops_total"] = 6.0 * tokens_step * plan.params / (ms * 1e-3) / 1e12
    out["tflops_per_gpu"] = out["tflops_total"] / world
    if world > 1:
        nbytes = 4.0 * plan.params
        out["allreduce_bytes"] = nbytes
        # what the step costs without the exchange (same kernels, dW left unsummed): the difference is the exposed part
        if plan.exchange == "switch":
            saved = [(s.dw_multicast, s.flags_local, s.flags_multicast) for s in plan._steps]
            for s in plan._steps:
                s.dw_multicast = None
            ms0 = timed_steps(env, plan.step, max(2, steps // 2), 1) / max(2, steps // 2)
            for s, (a, b, c) in zip(plan._steps, saved):
                s.dw_multicast, s.flags_local, s.flags_multicast = a, b, c
            out["ms_per_step_without_exchange"] = ms0
        bus = 2.0 * (world - 1) / world * nbytes / (ms * 1e-3) / 1e9
        out["busbw_gbs_over_whole_step"] = bus
        out["busbw_frac_of_measured_nccl_1gib"] = bus / NVLINK_ALLREDUCE_BUSBW_GBS
        out["exchange_check"] = check
    plan.close()
    del plan
    torch.cuda.empty_cache()
    return out


# ------------------------------------------- one Llama-3-70B-shaped layer, output rows sharded
ROWSHARD_TOKENS, ROWSHARD_LINEARS = WORKLOADS["llama3-70b-layer"]


def rowshard_block(env, args, steps, warmup):
    """The seven ternary linears of one Llama-3-70B decoder layer (hidden 8192, intermediate 28672, 8 KV heads x 128),
    8192 tokens per step, W ~ N(0, 0.015^2).  Every GPU holds out/N rows of each latent and packed matrix (strong
    scaling: the step's work is fixed).  One step: the two-call quantiser over all seven linears with ONE all-reduce of
    their seven f64 sums of |w| between the calls; then per linear act-quant (replicated), forward of the local rows
    followed by an all-gather of y, the dx partial product followed by a reduce-scatter over tokens, and the local rows
    of dW (no exchange).  The two big exchanges are issued asynchronously and waited for at the end of the step."""
    torch, dist = env.torch, env.dist
    from alice_train import _ffi, bitlinear as bl, parallel

    world, rank, dev, ctx, pk = env.world, env.rank, env.dev, env.ctx, env.pk
    tokens = ROWSHARD_TOKENS
    assert tokens % world == 0
    gen = torch.Generator(device=dev)
    layers = []
    for li, (name, out, inn) in enumerate(ROWSHARD_LINEARS):
        r0, r1 = parallel.row_shard(out, world, rank, align=128)
        rows = r1 - r0
        gen.manual_seed(7000 + 131 * li + rank)     # this GPU's rows of the latent matrix
        w_lat = torch.randn((rows, inn), generator=gen, device=dev, dtype=torch.float32) * 0.015
        gen.manual_seed(8000 + li)                  # x and dy are the same on every GPU (replicated activations)
        x = torch.randn((tokens, inn), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        dy = (torch.randn((tokens, out), generator=gen, device=dev, dtype=torch.float32) * 1e-2).to(torch.bfloat16)
        layers.append(dict(
            name=name, out=out, inn=inn, rows=rows, w=bl.BitLinearWeights(rows, inn, ctx), w_lat=w_lat, x=x,
            dy=dy[:, r0:r1].contiguous(),
            qa=bl.QuantizedActivations(torch.empty((tokens, inn), dtype=torch.int8, device=dev),
                                       torch.empty(tokens, dtype=torch.float32, device=dev),
                                       torch.empty(tokens, dtype=torch.int32, device=dev)),
            y=torch.empty((tokens, rows), dtype=torch.bfloat16, device=dev),
            y_all=torch.empty((world, tokens, rows), dtype=torch.bfloat16, device=dev) if world > 1 else None,
            dx=torch.empty((tokens, inn), dtype=torch.bfloat16, device=dev),
            dx_mine=torch.empty((tokens // world, inn), dtype=torch.bfloat16, device=dev) if world > 1 else None,
            dW=torch.zeros((rows, inn), dtype=torch.float32, device=dev)))
        del dy
    # the two big exchanges: the library's in-switch kernels on symmetric-memory buffers (forward shards are written
    # straight into the gathered layout, dx partials into the buffer the switch reduces), NCCL otherwise
    exchange = "none"
    if world > 1:
        exchange = "nccl"
        if args.dw_exchange == "switch":
            try:
                bufs = []
                for L in layers:
                    L["ybuf"] = parallel.SwitchBuffer(ctx, world * tokens * L["rows"] * 2, dev)
                    L["dxbuf"] = parallel.SwitchBuffer(ctx, tokens * L["inn"] * 2, dev)
                    bufs += [L["ybuf"], L["dxbuf"]]
                    L["y_all"] = L["ybuf"].view(torch.bfloat16, (world, tokens, L["rows"]))
                    L["y"] = L["y_all"][rank]
                    L["dx"] = L["dxbuf"].view(torch.bfloat16, (tokens, L["inn"]))
                parallel.SwitchBuffer.ready(bufs, dev)
                exchange = "switch"
            except RuntimeError as e:
                if rank == 0:
                    print(f"[bench] in-switch exchange unavailable ({e}); using NCCL", file=sys.stderr)
    ctx.sync()
    classes = ("fq", "act_quant", "fwd", "dx", "dw")
    ev = {c: [] for c in classes}
    sums = torch.zeros(len(layers), dtype=torch.float64, device=dev)

    def step(record: bool):
        handles = []

        def timed(cls, fn):
            if record:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                ev[cls].append((a, b))
            else:
                fn()

        def quantise():   # all seven sums of |w| travel in ONE 56-byte all-reduce, ahead of the step's big exchanges
            for i, L in enumerate(layers):
                L["w"].shard_abs_sum(L["w_lat"], sums[i:i + 1])
            parallel.global_abs_sum(sums)
            for i, L in enumerate(layers):
                L["w"].quantize_shard_(L["w_lat"], sums[i:i + 1], L["out"] * L["inn"])
        timed("fq", quantise)
        for L in layers:
            timed("act_quant", lambda: bl.act_quant_int8(ctx, L["x"], L["qa"]))
            timed("fwd", lambda: bl.bitlinear_fwd(L["w"], L["qa"], y=L["y"]))
            if exchange == "switch":
                L["ybuf"].start(_ffi.AB_XCHG_ALLGATHER, ctas=args.exchange_ctas)
            elif world > 1:
                handles.append(dist.all_gather_into_tensor(L["y_all"], L["y"], async_op=True))
            timed("dx", lambda: bl.bitlinear_dx(L["w"], L["dy"], dx=L["dx"]))
            if exchange == "switch":
                L["dxbuf"].start(_ffi.AB_XCHG_REDUCESCATTER_BF16, out_local=L["dx_mine"], ctas=args.exchange_ctas)
            elif world > 1:
                handles.append(dist.reduce_scatter_tensor(L["dx_mine"], L["dx"], op=dist.ReduceOp.SUM, async_op=True))
            timed("dw", lambda: bl.ste_dw(ctx, L["dy"], L["x"], L["dW"], beta=0.0))
        for hnd in handles:
            hnd.wait()
        if exchange == "switch":
            _ffi.check(_ffi.load().ab_dp_allreduce_wait(ctx.handle), ctx.handle)

    for _ in range(warmup):
        step(False)
    # both in-switch exchanges against NCCL on copies of the same inputs, before anything is timed.  The all-gather must
    # be bit-identical.  The reduce-scatter adds the GPUs' bf16 partials in f32 inside the switch and truncates the sum
    # to bf16, so it is held against NCCL's f32 reduce-scatter of the same partials: within one bf16 unit in the last
    # place of the exact sum (2^-7 relative) at any number of GPUs.  (NCCL's own bf16 reduce-scatter rounds after every
    # ring step and drifts further from the f32 sum than that where partials cancel.)
    check = None
    if exchange == "switch":
        ctx.sync()
        ok, ag_same, rs_worst = True, 0, 0.0
        for L in layers:
            mine = L["y"].clone()
            ref_all = torch.empty_like(L["y_all"])
            dist.all_gather_into_tensor(ref_all, mine)
            ag_same += int(torch.equal(ref_all, L["y_all"]))
            ok &= torch.equal(ref_all, L["y_all"])
            bl.bitlinear_dx(L["w"], L["dy"], dx=L["dx"])
            ctx.sync()
            part = L["dx"].float()
            ref_rs = torch.empty(L["dx_mine"].shape, dtype=torch.float32, device=part.device)
            dist.reduce_scatter_tensor(ref_rs, part, op=dist.ReduceOp.SUM)
            L["dxbuf"].start(_ffi.AB_XCHG_REDUCESCATTER_BF16, out_local=L["dx_mine"], ctas=args.exchange_ctas)
            _ffi.check(_ffi.load().ab_dp_allreduce_wait(ctx.handle), ctx.handle)
            ctx.sync()
            a = L["dx_mine"].float()
            tol = ref_rs.abs() * (2.0 ** -7) + 1e-6 * float(ref_rs.abs().max().item()) + 1e-30
            worst = float(((a - ref_rs).abs() / tol).max().item())
            rs_worst = max(rs_worst, worst)
            ok &= worst <= 1.0
            del mine, ref_all, part, ref_rs
        check = {"allgather_bit_identical": ag_same, "of": len(layers), "reduce_scatter_worst_over_one_bf16_ulp_of_f32_sum": rs_worst}
        if not env.all_ok(bool(ok)):
            raise ExchangeMismatch(f"llama3-70b-layer: in-switch exchange differs from its reference: {check}")
    env.fence()
    launches0 = ctx.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step(True)
    t1.record()
    env.fence()
    launches = ctx.launch_count() - launches0
    ms_total = env.max_over_ranks(t0.elapsed_time(t1))
    per = {}
    for c in classes:
        ts = [a.elapsed_time(b) for a, b in ev[c]]
        per[c] = {"ms_per_step": sum(ts) / steps}
    ops_rank = 2.0 * tokens * sum(L["rows"] * L["inn"] for L in layers)       # per GEMM class, this GPU, one step
    for c in ("fwd", "dx", "dw"):
        per[c]["tops"] = ops_rank / (per[c]["ms_per_step"] * 1e-3) / 1e12
    fq_bytes = 4.25 * sum(L["rows"] * L["inn"] for L in layers)
    per["fq"]["gbs"] = fq_bytes / (per["fq"]["ms_per_step"] * 1e-3) / 1e9
    gather_bytes = sum(tokens * L["out"] * 2 for L in layers) if world > 1 else 0
    rs_bytes = sum(tokens * L["inn"] * 2 for L in layers) if world > 1 else 0
    ms = ms_total / steps
    out = {"tokens_per_step": tokens, "scaling": "strong", "exchange": exchange, "ms_per_step": ms,
           "tokens_per_s": tokens / (ms * 1e-3), "gpu_launches_per_step": int(launches / steps),
           "tflops_total": 6.0 * tokens * sum(o * i for _, o, i in ROWSHARD_LINEARS) / (ms * 1e-3) / 1e12,
           "kernels_ms": {c: per[c]["ms_per_step"] for c in classes},
           "tops": {c: per[c]["tops"] for c in ("fwd", "dx", "dw")}, "fq_gbs": per["fq"]["gbs"]}
    if world > 1:
        moved = (world - 1) / world * (gather_bytes + rs_bytes)      # bytes that arrive at (and leave) each GPU per step
        out["exchange_bytes_per_gpu"] = moved
        out["busbw_gbs_over_whole_step"] = moved / (ms * 1e-3) / 1e9
        out["busbw_frac_of_measured_peer_copy"] = out["busbw_gbs_over_whole_step"] / NVLINK_PEER_COPY_GBS
        out["exchange_check"] = check
    for L in layers:
        L["w"].close()
    del layers
    torch.cuda.empty_cache()
    return out


def decode_block(env, layers=None, replays=20):
    """Packed decode over a .alice file (src/inference.rs:1211-1490): a Qwen3.5-9B-shaped model (src/qwen35.rs:67-102) is
    written by the library's exporter from latent weights drawn on the device, re-opened by the streaming reader, and one
    token's linear chain (248 ternary matvecs at m = 1 for 32 layers) is replayed from a CUDA graph.  The embedding table is
    cut to 4096 rows (it is not on the measured chain).  Bytes per token = the packed codes of every projection."""
    torch = env.torch
    import alice_train
    from alice_train import bitlinear as bl, export as ex
    dev = env.dev
    stream = torch.cuda.Stream(device=dev)
    prev = torch.cuda.current_stream(dev)
    torch.cuda.set_stream(stream)
    tmp = tempfile.NamedTemporaryFile(suffix=".alice", delete=False)
    try:
        ctx = alice_train.GpuContext.on_torch_stream(env.local)
        cfg = ex.Qwen35Config.qwen35_9b()
        cfg.vocab_size = 4096
        if layers:
            cfg.num_hidden_layers = layers
            cfg.layer_types = cfg.layer_types[:layers]
        gen = torch.Generator(device=dev)
        gen.manual_seed(21)

        def layer_tensors():
            for i in range(cfg.num_hidden_layers):
                t = {}
                for name, out, inn in cfg.projection_shapes(i):
                    t[name] = (out, inn)
                for name, count in cfg.fp32_shapes(i):
                    t[name] = np.ones(count, np.float32)
                yield t

        def quantizer(shape):
            out, inn = shape
            w_lat = torch.randn((out, inn), generator=gen, device=dev) * 0.02
            h = bl.BitLinearWeights(out, inn, ctx).quantize_(w_lat)
            ctx.sync()
            res = (h.gamma, h.to_packed())
            h.close()
            return res

        t0 = time.time()
        emb = np.zeros((cfg.vocab_size, cfg.hidden_size), np.float32)
        stats = ex.export_alice_model(tmp, cfg, layer_tensors(), emb, np.ones(cfg.hidden_size, np.float32), None, 0, 0.0, ctx, quantizer)
        tmp.flush()
        t_write = time.time() - t0
        t0 = time.time()
        model = alice_train.StreamingAliceModel.from_file(tmp.name, ctx, load_embeddings=False)
        ctx.sync()
        t_open = time.time() - t0
        h0 = torch.randn(cfg.hidden_size, generator=gen, device=dev)
        h = h0.clone()
        for _ in range(2):
            h.copy_(h0)
            model.decode_linears(h)
        torch.cuda.synchronize()
        finite = bool(torch.isfinite(h).all().item())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            model.decode_linears(h)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        sec = a.elapsed_time(b) * 1e-3 / replays
        linears = sum(len(L["w"]) for L in model.layers)
        nbytes = model.packed_bytes
        # CPU: the reference's own loop (ternary_matmul_bt at m = 1, single thread) over one DeltaNet layer's projections
        cpu = None
        try:
            from oracle import pyoracle as orc   # the CPU baseline leg: the only use of the oracle here
            lay = model.layers[0]["w"]
            r = np.random.default_rng(3)
            t_cpu, cpu_bytes = 0.0, 0
            for name, w in lay.items():
                o, n = w.out_features(), w.in_features()
                packed = w.to_packed()
                x = r.standard_normal(n).astype(np.float32)
                t1 = time.perf_counter()
                orc.ternary_matmul_bt(x, packed, w.scale, np.zeros(o, np.float32), 1, o, n)
                t_cpu += time.perf_counter() - t1
                cpu_bytes += packed.size
            cpu = {"tokens_per_s": 1.0 / (t_cpu * nbytes / cpu_bytes), "cores": 1, "kind": "port",
                   "sample": f"ternary_matmul_bt at m = 1 over the 8 projections of layer 0 ({t_cpu:.2f} s), scaled to {linears} projections by bytes"}
        except Exception as e:  # noqa: BLE001
            cpu = {"error": f"{type(e).__name__}: {e}"[:200]}
        model.close()
        return {"model": "qwen35-9b shapes", "layers": cfg.num_hidden_layers, "linears": linears, "file_bytes": stats.total_bytes,
                "packed_bytes_per_token": nbytes, "write_s": t_write, "open_s": t_open, "ms_per_token": sec * 1e3,
                "tokens_per_s": 1.0 / sec, "gbs": nbytes / sec * 1e-9, "frac_of_hbm": nbytes / sec * 1e-9 / env.pk["hbm_gbs"],
                "peak_gbs": env.pk["hbm_gbs"], "peak_source": f"{env.pk['source']} copy bandwidth", "timing": "cuda-graph replay of one token",
                "finite": finite, "cpu_baseline": cpu}
    finally:
        torch.cuda.set_stream(prev)
        tmp.close()
        try:
            os.unlink(tmp.name)
        except OSError:
            pass


def lm_head_block(env, steps=5, warmup=2, model="llama32-1b", tokens=8192):
    """The unquantised output head over the whole vocabulary (src/bin/train_qat_70b.rs:1024-1101): logits = h W^T,
    softmax cross-entropy with its gradient, d_hidden = d_logits W, dW += d_logits^T h; 8192 tokens.  Per-kernel CUDA events."""
    torch = env.torch
    import alice_train
    from alice_train import lm_head as lh
    vocab, hidden = {"llama32-1b": (128256, 2048), "qwen35-9b": (248320, 4096)}[model]
    m = tokens
    dev = env.dev
    ctx = env.ctx
    gen = torch.Generator(device=dev)
    gen.manual_seed(31)
    w = (torch.randn((vocab, hidden), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    h = torch.randn((m, hidden), generator=gen, device=dev).to(torch.bfloat16)
    tg = torch.randint(0, vocab, (m,), generator=gen, device=dev, dtype=torch.int32)
    head = lh.LmHead(ctx, w)
    logits = torch.empty((m, vocab), dtype=torch.float32, device=dev)
    loss = torch.empty(m, dtype=torch.float32, device=dev)
    d = torch.empty((m, vocab), dtype=torch.bfloat16, device=dev)
    d_hidden = torch.empty((m, hidden), dtype=torch.float32, device=dev)
    dW = torch.zeros((vocab, hidden), dtype=torch.float32, device=dev)
    names = ("logits", "cross_entropy", "d_hidden", "dw")
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(steps)]
    for it in range(warmup + steps):
        e = ev[it - warmup] if it >= warmup else None
        if e: e[0].record()
        head.logits(h, logits)
        if e: e[1].record()
        lh.cross_entropy(ctx, logits, tg, 1.0 / m, loss, d)
        if e: e[2].record()
        head.backward(d, h, d_hidden, None, want_dw=False)
        if e: e[3].record()
        head.backward(d, h, None, dW, dw_beta=1.0, want_dhidden=False)
        if e: e[4].record()
    torch.cuda.synchronize()
    ms = {n: sum(e[i].elapsed_time(e[i + 1]) for e in ev) / steps for i, n in enumerate(names)}
    flops = 2.0 * m * vocab * hidden
    ce_bytes = m * vocab * (4 + 2) + 8 * m
    total = sum(ms.values())
    pk = env.pk
    out = {"model": model, "tokens": m, "vocab": vocab, "hidden": hidden, "ms": ms, "ms_total": total, "tokens_per_s": m / (total * 1e-3),
           "tflops": {n: flops / (ms[n] * 1e-3) * 1e-12 for n in ("logits", "d_hidden", "dw")},
           "frac_of_bf16_burst": {n: flops / (ms[n] * 1e-3) * 1e-12 / pk["bf16_tflops"] for n in ("logits", "d_hidden", "dw")},
           "cross_entropy_gbs": ce_bytes / (ms["cross_entropy"] * 1e-3) * 1e-9,
           "cross_entropy_frac_of_hbm": ce_bytes / (ms["cross_entropy"] * 1e-3) * 1e-9 / pk["hbm_gbs"],
           "loss_mean": float(loss.mean().item()), "ln_vocab": float(np.log(vocab)),
           "note": "cross-entropy scored on 6 B per logit (f32 logits read once, bf16 gradient written once); its kernels read the logits twice"}
    del head, logits, d, dW, w
    torch.cuda.empty_cache()
    return out


class ExchangeMismatch(RuntimeError):
    """An in-switch exchange did not reproduce its reference: the run's numbers would describe a wrong result."""


def guarded(env, fn, *a, **k):
    """An optional block must not cost the headline line: errors are recorded in its place."""
    try:
        return fn(*a, **k)
    except SystemExit:
        raise
    except Exception as e:  # noqa: BLE001
        import traceback
        if env.rank == 0:
            traceback.print_exc()
        try:
            env.torch.cuda.empty_cache()
        except Exception:  # noqa: BLE001
            pass
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def partitioned_summary(p):
    """The few numbers per partitioned workload that must survive a truncated log (repeated inside `config`)."""
    s = {}
    for name, b in p.items():
        if not isinstance(b, dict) or "error" in b:
            s[name] = "error"
            continue
        s[name] = {"tok_s": b.get("tokens_per_s"), "ms": b.get("ms_per_step")}
    return s


def run_native(args):
    env = Env()
    line = None
    try:
        if args.workload in DECODER_WORKLOADS:
            blk = decoder_block(env, args.workload, args, args.steps, args.warmup)
            if env.rank == 0:
                line = {"metric": f"QAT step tokens/s over all ternary linears ({args.workload})", "value": blk["tokens_per_s"], "unit": UNIT,
                        "n_gpus": env.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": blk["ms_per_step"],
                        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                        "dtype": "int8 forward (s32 accumulate), bf16 backward (f32 accumulate)", "data": "synthetic",
                        "config": {"workload": args.workload, "parallelism": f"dp{env.world}"}, "block": blk}
        elif args.workload == "llama3-70b-layer":
            blk = rowshard_block(env, args, args.steps, args.warmup)
            if env.rank == 0:
                line = {"metric": "BitLinear fwd+bwd tokens/s, one Llama-3-70B-shaped layer, output rows sharded", "value": blk["tokens_per_s"],
                        "unit": UNIT, "n_gpus": env.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": blk["ms_per_step"],
                        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                        "dtype": "int8 forward (s32 accumulate), bf16 backward (f32 accumulate)", "data": "synthetic",
                        "config": {"workload": args.workload, "parallelism": f"rows/{env.world}"}, "block": blk}
        elif args.workload == "hbm-kernels":
            blk = hbm_block(env)
            if env.rank == 0:
                dom = blk["kernels"]["matvec_bwd"]
                line = {"metric": "batch-1 ternary kernels, achieved HBM GB/s", "value": dom["gbs"], "unit": "GB/s", "n_gpus": 1,
                        "higher_is_better": True, "data": "synthetic", "dtype": "f32 x 2-bit codes", "config": {"workload": "hbm-kernels"},
                        "roofline": {"bound": "hbm", "kernel": "matvec kernel (dx = W^T dy, integer path)", "achieved": dom["gbs"],
                                     "peak": blk["peak_gbs"], "unit": "GB/s", "frac": dom["frac"], "traffic": dram_traffic("matvec", "hbm-kernels"),
                                     "peak_source": blk["peak_source"]}, "block": blk}
        elif args.workload == "lm-head":
            models = ("llama32-1b", "qwen35-9b") if args.head_tokens == 8192 else ("llama32-1b",)
            blks = {mname: lm_head_block(env, model=mname, tokens=args.head_tokens) for mname in models}
            if env.rank == 0:
                b0 = blks["llama32-1b"]
                dom = max(("logits", "d_hidden", "dw"), key=lambda n: b0["ms"][n])
                line = {"metric": "output head (logits + cross-entropy + backward) tokens/s, vocabulary 128256 x hidden 2048", "value": b0["tokens_per_s"],
                        "unit": UNIT, "n_gpus": 1, "higher_is_better": True, "data": "synthetic", "dtype": "bf16 (f32 accumulate)",
                        "config": {"workload": "lm-head"},
                        "roofline": {"bound": "tensor", "kernel": f"gemm_pair_kernel bf16 x bf16 ({dom})", "achieved": b0["tflops"][dom],
                                     "peak": env.pk["bf16_tflops"], "unit": "TFLOP/s", "frac": b0["frac_of_bf16_burst"][dom], "traffic": None,
                                     "peak_source": f"{env.pk['source']} cuBLAS bf16 burst"}, "blocks": blks}
        elif args.workload == "alice-decode":
            blk = decode_block(env)
            if env.rank == 0:
                line = {"metric": "packed decode tokens/s over all ternary linears of a .alice model (m = 1)", "value": blk["tokens_per_s"],
                        "unit": UNIT, "n_gpus": 1, "higher_is_better": True, "data": "synthetic", "dtype": "f32 x 2-bit codes",
                        "config": {"workload": "alice-decode", "model": blk["model"]},
                        "roofline": {"bound": "hbm", "kernel": "matvec_tma_kernel over the file's projections", "achieved": blk["gbs"],
                                     "peak": blk["peak_gbs"], "unit": "GB/s", "frac": blk["frac_of_hbm"], "traffic": None,
                                     "peak_source": blk["peak_source"]}, "cpu_baseline": blk.pop("cpu_baseline"), "block": blk}
        else:
            line = run_main(env, args)
            extras = args.workload == "llama3-8b-mlp" and not args.no_extras
            if extras and env.world == 1:
                blk = guarded(env, hbm_block, env, False)
                if line is not None:
                    line["hbm_kernels"] = blk
            if extras:
                part = {}
                ps, pw = args.partitioned_steps, 2
                for name in ("llama32-1b-qat", "qwen35-9b-hybrid"):
                    part[name] = guarded(env, decoder_block, env, name, args, ps, pw)
                part["llama3-70b-layer"] = guarded(env, rowshard_block, env, args, ps, pw)
                if line is not None:
                    line["config"]["partitioned"] = partitioned_summary(part)
                    line["partitioned"] = part      # last key: survives a log that keeps only its tail
        if env.rank == 0 and line is not None:
            print(json.dumps(compact(line)), flush=True)
    except ExchangeMismatch as e:     # of the workload that was asked for (inside the default line's extras it is recorded instead)
        if env.rank == 0:
            print(f"[bench] {e}", file=sys.stderr)
        return 3
    finally:
        env.close()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="llama3-8b-mlp", choices=sorted(WORKLOADS) + ["hbm-kernels", "alice-decode", "lm-head"] + list(DECODER_WORKLOADS))
    ap.add_argument("--cpu-tokens", type=int, default=64, help="tokens per CPU-baseline sample")
    ap.add_argument("--dw-exchange", default="switch", choices=["switch", "nccl"],
                    help="sum of dW / all-gather / reduce-scatter: the library's in-switch kernels (default) or NCCL")
    ap.add_argument("--exchange-ctas", type=int, default=0, help="CTAs of the in-switch exchange kernel (0 = library default)")
    ap.add_argument("--partitioned-ctas", type=int, default=0, help="the same for the decoder workloads, whose exchange is much larger per unit of compute (0 = 32 at 2 GPUs, 16 at 4, 8 at 8: measured)")
    ap.add_argument("--partitioned-steps", type=int, default=5, help="timed steps of each partitioned workload inside the default run")
    ap.add_argument("--check-linears", type=int, default=12, help="dW buffers per decoder workload whose in-switch sum is checked against NCCL (0 = all)")
    ap.add_argument("--head-tokens", type=int, default=8192, help="tokens of the lm-head workload (a small value gives a case a profiler can capture)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no hbm_kernels / partitioned blocks)")
    args = ap.parse_args()
    if args.partitioned_ctas == 0:
        ws = int(os.environ.get("WORLD_SIZE", "1"))
        args.partitioned_ctas = 32 if ws <= 2 else (16 if ws <= 4 else 8)
    if args.impl == "reference":
        return run_reference(args)
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())
