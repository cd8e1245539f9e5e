#!/usr/bin/env python
"""Benchmark of the BitLinear hot path at the Llama-3-8B MLP shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload ("llama3-8b-mlp", the second configuration of the target specification): hidden 4096,
intermediate 14336, 4096 tokens per GPU; the gate, up (4096 -> 14336) and down (14336 -> 4096)
projections.  One step = for each projection: per-token int8 activation quantisation, the
int8 x ternary forward, dx = dy.W off the packed codes, and the STE gradient dW = dy^T.x.
Inputs are synthetic (seeded normal draws of the stated shapes); weights are random latent f32
matrices ternarised by the absmean quantiser before the timed region.

One JSON line is printed by rank 0.  `value` is tokens/s with every input resident in HBM;
`e2e` is the same metric through the host-buffer C-ABI entry point (pinned host memory, copies
inside the timed region).  `--impl reference` times the CPU restatement of the reference's own
code path on the host cores instead (see oracle/).
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
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "alice-train_b200"))

WORKLOADS = {
    # name: (tokens per GPU, [(projection, out_features, in_features)])
    "llama3-8b-mlp": (4096, [("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]),
    "small": (1024, [("gate", 2048, 1024), ("down", 1024, 2048)]),
    # one Llama-3-70B-shaped decoder layer, 8192 tokens per STEP (rows of W sharded over the GPUs; run_rowshard)
    "llama3-70b-layer": (8192, [("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
                                ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672)]),
}
METRIC = "BitLinear fwd+bwd tokens/s at Llama-8B shape"
UNIT = "tokens/s"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu), "-f", self.path],
                                         stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [s.strip() for s in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        # the busiest half of the samples is the timed region (the sampler also sees set-up)
        sm_sorted = sorted(sm)
        return {"sm_mhz": statistics.median(sm_sorted) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import pyoracle as orc
    tokens_full, projs = WORKLOADS[args.workload]
    layers = cpu_layers(orc, projs)
    sample = args.cpu_tokens
    # ~2e-8 s per weight and token on one core: keep warm-up + timed steps near two minutes whatever K is by
    # running a fraction of every projection's output rows per step (never less than 1/64)
    est = 2e-8 * sum(o * i for _, o, i in projs) * sample * (args.steps + args.warmup)
    row_frac = 1.0 if est <= 120.0 else max(1.0 / 64.0, 120.0 / est)
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
                   "note": "CPU restatement of the reference's f32 path; each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": "port",
                         "sample": f"{sample} of {tokens_full} tokens per step through {100 * rows_done:.1f} % of the output rows of "
                                   f"all projections (fwd tiled_matmul_bt + matmul_bt_backward), single thread as in the reference; "
                                   f"weights fake-quantised with {orc.max_threads()} threads outside the timed region"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------- native arm
def run_native(args):
    import torch
    import torch.distributed as dist

    import alice_train
    from alice_train import _ffi, bitlinear as bl

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a B200: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = alice_train.GpuContext.on_torch_stream(local)
    tokens, projs = WORKLOADS[args.workload]
    pk = peaks()

    # ---- set-up (untimed): latent weights -> codes, inputs resident in HBM
    gen = torch.Generator(device=dev)
    layers = []
    for li, (name, out, inn) in enumerate(projs):
        gen.manual_seed(10 + li)  # identical weights on every rank (data parallel)
        w_lat = torch.randn((out, inn), generator=gen, device=dev, dtype=torch.float32) * 0.02
        h = bl.BitLinearWeights(out, inn, ctx).quantize_(w_lat)
        gen.manual_seed(1000 + 97 * rank + li)  # each rank has its own tokens
        x = torch.randn((tokens, inn), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        dy = (torch.randn((tokens, out), generator=gen, device=dev, dtype=torch.float32) * 1e-2).to(torch.bfloat16)
        layers.append(dict(
            name=name, out=out, inn=inn, w=h, w_lat=w_lat, x=x, dy=dy,
            qa=bl.QuantizedActivations(torch.empty((tokens, inn), dtype=torch.int8, device=dev),
                                       torch.empty(tokens, dtype=torch.float32, device=dev),
                                       torch.empty(tokens, dtype=torch.int32, device=dev)),
            y=torch.empty((tokens, out), dtype=torch.bfloat16, device=dev),
            dx=torch.empty((tokens, inn), dtype=torch.bfloat16, device=dev),
            dW=torch.zeros((out, inn), dtype=torch.float32, device=dev)))
    ctx.sync()
    # data parallel: dW lives in symmetric memory and is summed inside NVSwitch by the library's own kernel;
    # NCCL remains the exchange where the GPUs have no multicast mapping (or on request)
    switch, exchange = None, "none"
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

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    fence()
    launches0 = ctx.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    fence()
    launches = ctx.launch_count() - launches0
    ms = torch.tensor([t0.elapsed_time(t1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
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
    dom = max(("fwd", "dx", "dw"), key=lambda c: per[c]["ms_total"])
    # denominators: the measured cuBLAS bf16 figure for the bf16 kernels; the peaks file has no int8
    # entry, so the int8 kernel is set against the MMA-only probe measured just above
    peak_bf16 = pk["bf16_tflops_sustained"]
    peak = probe["int8_tops"] if dom == "fwd" else peak_bf16
    roofline = {"bound": "tensor", "kernel": {"fwd": "gemm_pair_kernel<FWD> int8 x ternary", "dx": "gemm_pair_kernel<DX> bf16 x ternary",
                                              "dw": "gemm_pair_kernel<DW> bf16 x bf16"}[dom],
                "achieved": per[dom]["tops_avg"], "peak": peak, "unit": "TFLOP/s",
                "frac": per[dom]["tops_avg"] / peak if per[dom]["tops_avg"] else None,
                # DRAM read + write bytes of one launch from the ncu capture summarised in
                # profiles/gemm_pair_kernel_llama8b_mlp.md (gate projection; llama3-8b-mlp workload only)
                "traffic": ({"fwd": 95.0e6, "dx": 158.3e6, "dw": 363.3e6}[dom] if args.workload == "llama3-8b-mlp" else None),
                "peak_source": ("int8 MMA-only probe (ab_tensor_peak_probe) in this run" if dom == "fwd"
                                else f"{pk['source']} bf16 sustained {peak_bf16} TFLOP/s"),
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
        fence()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        fence()
        dt = torch.tensor([time.perf_counter() - w0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        h2d = sum(tokens * (i + o) * 2 for _, o, i in projs)
        e2e = {"value": world * tokens * e2e_steps / float(dt.item()), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": h2d, "steps": e2e_steps,
               "note": "ab_bitlinear_step_host per projection (queued, one sync per step): x, dy in and y, dx out as bf16 through pinned host memory; dW stays on the device"}
        ctx.set_async_host_step(False)

    # ---- CPU baseline (oracle port), rank 0 at N = 1 only, bounded sample
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import pyoracle as orc
        cl = cpu_layers(orc, projs)
        cpu_step(orc, cl, 1)
        secs = cpu_step(orc, cl, args.cpu_tokens, seed=7)
        cpu_baseline = {"value": args.cpu_tokens / secs, "unit": UNIT, "cores": 1, "kind": "port",
                        "sample": f"{args.cpu_tokens} of {tokens} tokens through all projections (fwd tiled_matmul_bt + "
                                  f"matmul_bt_backward on fake-quantised f32 weights), single thread as in the reference"}

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
            "clocks": clocks, "kernels": per, "tensor_pipe_probe": probe,
            "fractions": {"fwd_of_int8_probe": per["fwd"]["tops_avg"] / probe["int8_tops"],
                          "dx_of_bf16_measured": per["dx"]["tops_avg"] / peak_bf16,
                          "dw_of_bf16_measured": per["dw"]["tops_avg"] / peak_bf16},
            "tops_total": 6.0 * tokens * sum(o * i for _, o, i in projs) * args.steps / (ms_total * 1e-3) / 1e12,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------- memory-bound kernels (batch-1 path)
def run_hbm(args):
    """Batch-1 and streaming kernels against the measured HBM copy bandwidth.  Every packed weight
    matrix of the target configurations fits the 126 MB L2, so the matvec kernels rotate over
    enough distinct matrices to exceed it (cold L2); the L2-resident figure is reported beside it."""
    import torch

    import alice_train
    from alice_train import _ffi, bitlinear as bl

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    # everything runs on one explicit stream so that the timed launch sequences can be captured into CUDA graphs:
    # these kernels take 10-50 us, less than the Python + ctypes cost of issuing one, and a replayed graph times the
    # device, not the host
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    ctx = alice_train.GpuContext.on_torch_stream(0)
    lib = _ffi.load()
    pk = peaks()
    out, inn = 28672, 8192  # the largest single matrix of the target configurations (70B-shape gate projection)
    nmat = 8  # 8 x 56 MiB of canonical codes = 448 MiB > 3 x L2; launches long enough that the host stays ahead
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    mats = []
    for i in range(nmat):
        w_lat = torch.randn((out, inn), generator=gen, device=dev) * 0.02
        mats.append(bl.BitLinearWeights(out, inn, ctx).quantize_(w_lat))
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
            fn(mats[i % nmat])
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
        "ternary_matvec (fwd)": (lambda w: _ffi.check(lib.ab_ternary_matvec(ctx.handle, w.handle, vp(x), vp(y)), ctx.handle),
                                 code_bytes + 4 * (out + inn)),
        "ternary_matvec_backward": (lambda w: _ffi.check(lib.ab_ternary_matvec_backward(ctx.handle, w.handle, vp(dy), vp(dx)), ctx.handle),
                                    code_bytes + 4 * (out + inn)),
        "bitlinear_backward pre_norm": (lambda w: _ffi.check(lib.ab_bitlinear_backward(ctx.handle, w.handle, vp(x), vp(dy), 1, 1e-6, vp(dx), None), ctx.handle),
                                        code_bytes + 4 * (2 * out + 2 * inn)),
    }
    for name, (fn, nbytes) in cases.items():
        cold = timeit(fn, 6 * nmat, True)
        warm = timeit(fn, 6 * nmat, False)
        res[name] = {"bytes": nbytes, "cold_us": cold * 1e6, "cold_gbs": nbytes / cold / 1e9,
                     "cold_frac_of_hbm": nbytes / cold / 1e9 / pk["hbm_gbs"], "l2_resident_us": warm * 1e6,
                     "l2_resident_gbs": nbytes / warm / 1e9}
    # the same three entry points with AB_OPT_EXACT_MATVEC: f32 adds on the CUDA cores, as the reference's loops do
    ctx.set_exact_matvec(True)
    for name, (fn, nbytes) in cases.items():
        cold = timeit(fn, 6 * nmat, True)
        res[name + " [f32 adds]"] = {"bytes": nbytes, "cold_us": cold * 1e6, "cold_gbs": nbytes / cold / 1e9,
                                     "cold_frac_of_hbm": nbytes / cold / 1e9 / pk["hbm_gbs"]}
    ctx.set_exact_matvec(False)
    t = timeit(lambda w: _ffi.check(lib.ab_ste_weight_grad(ctx.handle, vp(x), 8192, vp(dy), 8192, vp(dW)), ctx.handle), 20, False)
    nb = 8.0 * 8192 * 8192 + 4 * (8192 + 8192)
    res["ste_weight_grad"] = {"bytes": nb, "cold_us": t * 1e6, "cold_gbs": nb / t / 1e9, "cold_frac_of_hbm": nb / t / 1e9 / pk["hbm_gbs"]}
    # kernel (1) at the Llama-3-8B gate shape (235 MB of latent weights, above L2)
    w_lat = torch.randn((14336, 4096), generator=gen, device=dev) * 0.02
    hq = bl.BitLinearWeights(14336, 4096, ctx)
    t = timeit(lambda w: hq.quantize_(w_lat), 20, False)
    nb = 4.25 * 14336 * 4096
    res["fq_absmean_pack"] = {"bytes": nb, "cold_us": t * 1e6, "cold_gbs": nb / t / 1e9, "cold_frac_of_hbm": nb / t / 1e9 / pk["hbm_gbs"],
                              "note": "scored on 4.25 B/weight; the kernels read the tensor twice and also write the two GEMM operand copies"}
    xa = torch.randn((4096, 14336), generator=gen, device=dev).to(torch.bfloat16)
    qa = bl.act_quant_int8(ctx, xa)
    t = timeit(lambda w: bl.act_quant_int8(ctx, xa, qa), 20, False)
    nb = 4096 * 14336 * 3 + 8 * 4096
    res["act_quant_int8"] = {"bytes": nb, "cold_us": t * 1e6, "cold_gbs": nb / t / 1e9, "cold_frac_of_hbm": nb / t / 1e9 / pk["hbm_gbs"]}
    ctx.sync()
    dom = res["ternary_matvec_backward"]
    line = {"metric": "batch-1 ternary kernels, achieved HBM GB/s", "value": dom["cold_gbs"], "unit": "GB/s", "n_gpus": 1,
            "higher_is_better": True, "data": "synthetic", "dtype": "f32 x 2-bit codes",
            "config": {"workload": "hbm-kernels", "matrix": [out, inn], "rotation": f"{nmat} distinct packed matrices ({nmat * code_bytes / 2**20:.0f} MiB of codes) so every launch reads cold lines"},
            "roofline": {"bound": "hbm", "kernel": "matvec_mma_kernel (dx = W^T dy, integer path)", "achieved": dom["cold_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": dom["cold_frac_of_hbm"], "traffic": None, "peak_source": pk["source"] + " copy bandwidth"},
            "timing": timing["mode"], "kernels": res}
    print(json.dumps(line), flush=True)
    return 0

# ------------------------------------------- one Llama-3-70B-shaped layer, output rows sharded
ROWSHARD_TOKENS, ROWSHARD_LINEARS = WORKLOADS["llama3-70b-layer"]


def run_rowshard(args):
    """--workload llama3-70b-layer: the seven ternary linears of one Llama-3-70B decoder layer (hidden 8192,
    intermediate 28672, 8 KV heads x 128), 8192 tokens per step, W ~ N(0, 0.015^2).  Every GPU holds out/N rows of
    each latent and packed matrix (strong scaling: the step's work is fixed).  One step: the two-call quantiser over
    all seven linears with ONE all-reduce of their seven f64 sums of |w| between the calls; then per linear act-quant
    (replicated), forward of the local rows followed by an all-gather of y, the dx partial product followed by a
    reduce-scatter over tokens, and the local rows of dW (no exchange).  The two big exchanges are issued
    asynchronously and waited for at the end of the step."""
    import torch
    import torch.distributed as dist

    import alice_train
    from alice_train import _ffi, bitlinear as bl, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a B200: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = alice_train.GpuContext.on_torch_stream(local)
    tokens = ROWSHARD_TOKENS
    assert tokens % world == 0
    pk = peaks()
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

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    fence()
    launches0 = ctx.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    fence()
    launches = ctx.launch_count() - launches0
    ms = torch.tensor([t0.elapsed_time(t1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    clocks = sampler.stop() if rank == 0 else None
    per = {}
    for c in classes:
        ts = [a.elapsed_time(b) for a, b in ev[c]]
        per[c] = {"launches": len(ts), "ms_per_step": sum(ts) / args.steps}
    ops_rank = 2.0 * tokens * sum(L["rows"] * L["inn"] for L in layers)       # per GEMM class, this GPU, one step
    for c in ("fwd", "dx", "dw"):
        per[c]["tops"] = ops_rank / (per[c]["ms_per_step"] * 1e-3) / 1e12
    fq_bytes = 4.25 * sum(L["rows"] * L["inn"] for L in layers)
    per["fq"]["gbs"] = fq_bytes / (per["fq"]["ms_per_step"] * 1e-3) / 1e9
    dom = max(("fwd", "dx", "dw"), key=lambda c: per[c]["ms_per_step"])
    peak_bf16 = pk["bf16_tflops_sustained"]
    gather_bytes = sum(tokens * L["out"] * 2 for L in layers) if world > 1 else 0
    rs_bytes = sum(tokens * L["inn"] * 2 for L in layers) if world > 1 else 0
    if rank == 0:
        line = {
            "metric": "BitLinear fwd+bwd tokens/s, one Llama-3-70B-shaped layer, output rows sharded", "value": tokens * args.steps / (ms_total * 1e-3),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 forward (s32 accumulate), bf16 backward (f32 accumulate)", "data": "synthetic",
            "config": {"workload": "llama3-70b-layer", "tokens_per_step": tokens, "linears": {n: [o, i] for n, o, i in ROWSHARD_LINEARS},
                       "parallelism": f"rows/{world}" if world > 1 else "single",
                       "step": "quantise the local rows of all linears (one all-reduce of the 7 sums of |w|); then per linear: act-quant, fwd -> all-gather y (bf16), "
                               "dx partial -> reduce-scatter over tokens (bf16), dW rows (local)",
                       "exchange": exchange,
                       "exchange_bytes_per_step": {"all_gather_y_total": gather_bytes, "reduce_scatter_dx_input_per_gpu": rs_bytes},
                       "l2": "latent shards, dW and activations exceed the 126 MB L2 at every N; no explicit flush"},
            "roofline": {"bound": "tensor", "kernel": f"gemm_pair_kernel<{dom.upper()}>", "achieved": per[dom]["tops"], "peak": peak_bf16,
                         "unit": "TFLOP/s", "frac": per[dom]["tops"] / peak_bf16, "traffic": None,
                         "peak_source": f"{pk['source']} bf16 sustained"},
            "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "clocks": clocks, "kernels": per,
            "tops_total": 6.0 * tokens * sum(o * i for _, o, i in ROWSHARD_LINEARS) * args.steps / (ms_total * 1e-3) / 1e12,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="llama3-8b-mlp", choices=sorted(WORKLOADS) + ["hbm-kernels"])
    ap.add_argument("--cpu-tokens", type=int, default=4, help="tokens per CPU-baseline sample")
    ap.add_argument("--dw-exchange", default="switch", choices=["switch", "nccl"],
                    help="data-parallel sum of dW: the library's in-switch kernel (default) or NCCL")
    ap.add_argument("--exchange-ctas", type=int, default=0, help="CTAs of the in-switch exchange kernel (0 = library default)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps * args.cpu_tokens > 24:  # ~3.5 s of CPU per token: one token per step is enough when K is large
            args.cpu_tokens = max(1, 24 // args.steps)
        return run_reference(args)
    if args.workload == "hbm-kernels":
        return run_hbm(args)
    if args.workload == "llama3-70b-layer":
        return run_rowshard(args)
    return run_native(args)


if __name__ == "__main__":
    sys.exit(main())
