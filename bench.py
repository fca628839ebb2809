#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path (Hadamard + int4 quantise + int4 GEMM + dequant).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one pass over the linears of one decoder layer for one batch of
token rows: per linear, kernel (a) (fused [Hadamard ->] absmax -> int4 pack) and
kernel (b) (int4 GEMM with the dequant epilogue).  The default workload is
the LLaMA-2-7B layer at prefill size (M = 2048 tokens): QKV 4096->12288, o_proj
4096->4096, gate/up 4096->22016 (quantiser only) and down_proj 11008->4096 with
the online Hadamard had_172 (x) Walsh_64.  Activations and weights are seeded
synthetic tensors with the benchmark's value distributions (quarot_b200/synth.py).

N > 1 (launched with torch.distributed.run, one rank per GPU): token rows are
sharded, weights replicated, no collective on the data path; every rank processes
M rows per step (weak scaling) and the reported value is the whole-job aggregate.

One JSON line is printed by rank 0.  Beside the headline it carries `other_configs`:
short device-timed runs of the remaining benchmark configurations (single linear,
decode at M = 1/8/32/64, the 70B layer; for N > 1 the 70B layer with its rows split
over the ranks and the 70B MLP with its output channels split over the ranks) and,
for N > 1, a `parity` block that compares the multi-GPU results with the single-GPU
result on a small shape.  --impl reference times the CPU restatement of the upstream
torch path (oracle/) on the host cores for the same metric and config; that arm does
not import the product package.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# (name, K, N, online Hadamard on K?) per linear of one decoder layer -- the same tables as quarot_b200/synth.py
# (tests/test_package_cpu.py keeps them equal); repeated here so that the reference arm needs no product import.
LAYERS = {
    "LLAMA2_7B": (("qkv", 4096, 12288, False), ("o_proj", 4096, 4096, False),
                  ("gate_up", 4096, 22016, False), ("down", 11008, 4096, True)),
    "LLAMA2_70B": (("qkv", 8192, 10240, False), ("o_proj", 8192, 8192, False),
                   ("gate_up", 8192, 57344, False), ("down", 28672, 8192, True)),
    "LLAMA2_70B_MLP": (("gate_up", 8192, 57344, False), ("down", 28672, 8192, True)),
    "LLAMA2_7B_MLP": (("gate_up", 4096, 22016, False), ("down", 11008, 4096, True)),
    "CONFIG0": (("cfg0", 4096, 4096, True),),
}
WORKLOADS = {
    # name: (layer table name, default tokens per GPU)
    "llama2_7b_prefill": ("LLAMA2_7B", 2048),
    "config0": ("CONFIG0", 2048),
    "llama2_7b_decode": ("LLAMA2_7B", 32),
    "llama2_70b_prefill": ("LLAMA2_70B", 4096),
    # the two 70B MLP linears with their output channels split over the ranks and an
    # all-gather of the fp16 result; every rank sees all token rows (use --tokens to sweep M)
    "llama2_70b_mlp_colsplit": ("LLAMA2_70B_MLP", 4096),
    # the MLP block around the path (first of the rows that come after it): quantise -> gate/up -> SiLU product ->
    # Hadamard + quantise -> down, with the product as separate elementwise kernels or inside the GEMM epilogue
    "llama2_7b_mlp_swiglu": ("LLAMA2_7B_MLP", 2048),
    "llama2_70b_mlp_swiglu": ("LLAMA2_70B_MLP", 4096),
    # the step in front of the path: RMSNorm + Quantizer of the hidden state (fused kernel vs the two modules)
    "llama2_7b_rmsnorm_quant": ("LLAMA2_7B", 2048),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_INT8_TOPS = 4500.0
DECODE_MAX_M = 128      # workloads with at most this many token rows are reported against the HBM roofline

# DRAM traffic of the dominant kernel's launches of one step, from ncu captures (dram__bytes_read.sum +
# dram__bytes_write.sum of one launch per linear; the captures are summarised under profiles/).
# Key: (workload, tokens per GPU).  7B prefill: qkv 29.46 + 6.26 MB, o_proj 12.66 + 0, gate/up 49.46 + 44.87,
# down 33.90 + 0.34 -- below the algorithmic bytes because most of the fp16 output is still in L2 when a launch ends.
NCU_TRAFFIC_BYTES = {("llama2_7b_prefill", 2048): 176.95e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def layer_ops(layers, M):
    return sum(2.0 * M * N * K for (_, K, N, _) in layers)


def bytes_quant(M, K):
    return 2.0 * M * K + M * K / 2.0 + 2.0 * M


def bytes_gemm(M, K, N):
    return M * K / 2.0 + N * K / 2.0 + 2.0 * M + 2.0 * N + 2.0 * M * N


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def window(self, t0, t1):
        """Median SM MHz of the samples taken between two perf_counter stamps."""
        vals = []
        for (t, line) in self.lines:
            if t0 <= t <= t1:
                try:
                    vals.append(float(line.split(",")[0]))
                except ValueError:
                    pass
        return statistics.median(vals) if vals else None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for (_, line) in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ reference (CPU) arm
def _cpu_activations(O, M, K, seed):
    """Outlier-Gaussian fp16 activations: the generator of quarot_b200/synth.py, restated for the CPU arm."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    idx = torch.randperm(K, generator=g)[: min(8, K)]
    x[:, idx] *= 50.0
    return x.to(torch.float16)


def _cpu_weights(O, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    scales = (torch.rand(N, 1, generator=g) * 0.015 + 0.005).to(torch.float16)
    return O.pack_i4(codes), scales


def cpu_reference_run(layers, M_full, steps, warmup, budget_s=20.0, rows=None):
    """Times the CPU restatement of the upstream torch path on a bounded sample of token rows.

    Weights are unpacked to int32 once, outside the timed region (as the fake-quant
    reference keeps them); per step and per linear: Hadamard (fp32 butterflies, cast
    to fp16), per-token scale, quantise, pack, unpack, int32 matmul, fp32 dequant.
    Imports only oracle/, never the product package.
    """
    from oracle import quarot_oracle as O
    cores = torch.get_num_threads()
    if rows is None:
        # pick the sample so that one step costs about budget_s / (steps + warmup)
        a = torch.randint(-8, 8, (16, 4096), dtype=torch.int32)
        b = torch.randint(-8, 8, (1024, 4096), dtype=torch.int32)
        t0 = time.perf_counter()
        _ = a @ b.T
        rate = 2.0 * 16 * 1024 * 4096 / max(time.perf_counter() - t0, 1e-6)   # int ops / s
        per_token_ops = layer_ops(layers, 1)
        target = budget_s / max(steps + warmup, 1)
        rows = int(max(1, min(64, M_full, rate * target / per_token_ops)))
    ms = rows
    data = []
    for (name, K, N, had) in layers:
        x = _cpu_activations(O, ms, K, seed=1234)
        w, sw = _cpu_weights(O, N, K, seed=4321)
        data.append((x, O.unpack_i4(w), sw, had))

    def step():
        outs = []
        for (x, wu, sw, had) in data:
            y = O.hadamard(x.float()).to(torch.float16) if had else x
            s = O.quantizer_scales(y)
            p = O.pack_i4(O.sym_quant_codes(y, s))
            acc = O.unpack_i4(p) @ wu.T
            outs.append(O.sym_dequant_fp32(acc, s, sw).to(torch.float16))
        return outs

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    tops = layer_ops(layers, ms) / dt / 1e12
    return {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port",
            "sample": "%d of %d token rows per step, %d steps; weights pre-unpacked to int32 outside the "
                      "timed region; ms_per_step is scaled linearly to %d rows" % (ms, M_full, steps, M_full),
            "ms_per_step_full": dt * 1e3 * (M_full / ms), "ms_per_step_sample": dt * 1e3, "tokens_per_s": ms / dt}


# ------------------------------------------------------------------ device arm
def build_device_workload(layers, M, dev, nsets):
    from quarot_b200 import synth
    from quarot_b200.functional import hadamard as FH
    work = []
    for li, (name, K, N, had) in enumerate(layers):
        khad = FH.get_hadK(K)[1] if had else 0
        table = FH.device_table(khad, dev) if khad > 1 else None
        xs = [synth.activations_device(M, K, seed=1234 + 17 * s + li, device=dev) for s in range(nsets)]
        ws = [synth.weights_device(N, K, seed=4321 + 13 * s + li, device=dev) for s in range(nsets)]
        work.append({
            "name": name, "K": K, "N": N, "khad": khad, "table": table, "x": xs,
            "w": [w for (w, _) in ws], "sw": [s.view(-1).contiguous() for (_, s) in ws],
            "q": torch.empty((M, K // 2), dtype=torch.uint8, device=dev),
            "s": torch.empty((M,), dtype=torch.float16, device=dev),
            "out": torch.empty((M, N), dtype=torch.float16, device=dev),
        })
    return work


def fused_quant_rows():
    """Largest M for which Sequential(Quantizer, Linear4bit) runs as ONE launch (quantiser inside the GEMV)."""
    from quarot_b200.nn import fused
    return fused.QuantLinear4bit.FUSED_MAX_ROWS


def device_step(qb, work, set_idx, part="all"):
    """One step.  part = "all" | "quant" (kernel (a) launches only) | "gemm" (kernel (b) launches only; the packed
    activations of the last full step are reused).  Returns the number of kernels launched."""
    launches = 0
    M = work[0]["x"][0].shape[0]
    fuse = M <= fused_quant_rows()
    for L in work:
        if L["khad"] == 0 and fuse:
            # a few token rows, no transform: the quantiser runs inside the weight-streaming kernel (one launch)
            if part != "quant":
                qb.quant_linear_i4(L["x"][set_idx], L["w"][set_idx], L["sw"][set_idx], out=L["out"])
                launches += 1
            continue
        if part != "gemm":
            qb.hadamard_quant(L["x"][set_idx], L["table"], L["khad"], 1.0, out_q=L["q"], out_s=L["s"])
            launches += 1
        if part != "quant":
            qb.linear_i4(L["q"], L["s"], L["w"][set_idx], L["sw"][set_idx], out=L["out"])
            launches += 1
    return launches


def capture_graphs(dev, nsets, fn):
    """One CUDA graph per buffer set of fn(set_idx); None when capture is not possible."""
    try:
        graphs = []
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for sidx in range(nsets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    fn(sidx)
                graphs.append(g)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        return graphs
    except Exception as exc:   # capture is an optimisation of the harness, not of the kernels
        sys.stderr.write("bench.py: CUDA graph capture failed (%s); timing eager launches\n" % exc)
        torch.cuda.synchronize(dev)
        return None


def timed_steps(dev, dist, run, steps, warmup):
    """ms per step of run(i), CUDA events on the current stream, barrier + synchronize on both sides, max over ranks."""
    for i in range(warmup):
        run(i)
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        run(i)
    e1.record()
    torch.cuda.synchronize(dev)
    t1 = time.perf_counter()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, (t0, t1)


def measure_layers(qb, layers, M, dev, dist, steps, warmup, use_graph=True, breakdown=True, nsets=3):
    """Device-timed step of `layers` at M token rows: whole step, and kernel (a) / kernel (b) launches alone
    (each as its own graph replay, so the split is free of Python launch time)."""
    work = build_device_workload(layers, M, dev, nsets)
    for i in range(nsets):
        device_step(qb, work, i)
    torch.cuda.synchronize(dev)
    res = {"work": work}

    def runner(part):
        graphs = capture_graphs(dev, nsets, lambda s: device_step(qb, work, s, part)) if use_graph else None
        if graphs is not None:
            return (lambda i: graphs[i % nsets].replay()), True
        return (lambda i: device_step(qb, work, i % nsets, part)), False

    run_all, graphed = runner("all")
    res["launch_mode"] = "cuda_graph_replay" if graphed else "eager"
    res["run_all"] = run_all
    res["ms_step"], res["window"] = timed_steps(dev, dist, run_all, steps, warmup)
    res["launches_per_step"] = device_step(qb, work, 0)
    if breakdown:
        run_g, _ = runner("gemm")
        res["gemm_ms"], _ = timed_steps(dev, None, run_g, steps, warmup)
        res["gemm_launches"] = device_step(qb, work, 0, "gemm")
        res["quant_launches"] = device_step(qb, work, 0, "quant")
        if res["quant_launches"]:
            run_q, _ = runner("quant")
            res["quant_ms"], _ = timed_steps(dev, None, run_q, steps, warmup)
        else:
            res["quant_ms"] = 0.0
        device_step(qb, work, 0)      # leave q / s consistent
    torch.cuda.synchronize(dev)
    return res


def roofline_record(layers, M, res, peaks, peak_src, workload, int8_probe, region_s):
    """`roofline` of the dominant kernel, kernel (b): tensor-bound at prefill sizes, HBM-bound at decode sizes."""
    fused = M <= fused_quant_rows()
    if M <= DECODE_MAX_M:
        nbytes = sum(bytes_gemm(M, K, N) + (2.0 * M * K - M * K / 2.0 if (fused and not had) else 0.0)
                     for (_, K, N, had) in layers)
        achieved = nbytes / (res["gemm_ms"] * 1e-3) / 1e9
        rec = {"bound": "hbm", "kernel": ("gemv_i4_kernel with the quantiser inside (three linears) and gemv_mma_i4_kernel (down)" if fused else
                          "gemv_mma_i4_kernel" if M <= 32 else "gemm_i4_decode_kernel") + ", one launch per linear",
               "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
               "peak_source": "hbm_gbs of MEASURED_PEAKS.json (%s)" % peak_src,
               "algorithmic_bytes_per_step": nbytes, "kernel_ms_per_step": res["gemm_ms"],
               "frac_of_nominal_8000": achieved / 8000.0}
    else:
        ops = layer_ops(layers, M)
        achieved = ops / (res["gemm_ms"] * 1e-3) / 1e12
        burst, sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
        use_burst = region_s < 1.0
        peak = burst if use_burst else sustained
        rec = {"bound": "tensor", "kernel": "gemm_i4_2sm_kernel (one launch per linear)",
               "achieved": achieved, "peak": peak, "unit": "TOPS", "frac": achieved / peak,
               "peak_source": "2 x %s of MEASURED_PEAKS.json (%s): dense int8 runs at twice the bf16 rate on these tensor "
                              "cores and the file holds no int8 figure; the timed region lasted %.3f s, so the %s figure "
                              "applies" % ("bf16_tflops" if use_burst else "bf16_tflops_sustained", peak_src, region_s,
                                           "burst" if use_burst else "sustained"),
               "peak_burst_2x_bf16": burst, "peak_sustained_2x_bf16": sustained,
               "int8_measured_tops": int8_probe, "frac_of_int8_measured": (achieved / int8_probe) if int8_probe else None,
               "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
               "peak_exceeded": bool(achieved > peak),
               "kernel_ms_per_step": res["gemm_ms"]}
    rec["traffic"] = NCU_TRAFFIC_BYTES.get((workload, M))
    if rec["traffic"] is not None:
        rec["traffic_note"] = "ncu dram bytes read + written by the step's launches of this kernel (one capture per linear)"
        rec["algorithmic_bytes_per_step"] = float(sum(bytes_gemm(M, K, N) for (_, K, N, _) in layers))
    return rec


def int8_probe_tops(dev):
    """Dense int8 GEMM rate of the library on this GPU (torch._int_mm, 8192^3), as a cross-check of the peak."""
    try:
        a = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device=dev)
        b = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device=dev).t()
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize(dev)
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        return 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception as exc:
        sys.stderr.write("bench.py: int8 probe skipped (%r)\n" % (exc,))
        return None


def e2e_run(qb, layers, M, dev, steps, warmup, work):
    """Same step through the module API with HOST buffers: per linear, activations are copied
    from pinned host memory, pushed through Sequential([HadamardQuantizer|Quantizer], Linear4bit)
    and the fp16 result is copied back to pinned host memory.  Copies run on their own streams
    so that transfers of neighbouring linears and of neighbouring steps overlap the kernels and each other."""
    mods, hx, hout = [], [], []
    for L in work:
        lin = qb.nn.Linear4bit(L["K"], L["N"]).to(dev)
        lin.weight = L["w"][0]
        lin.weight_scales = L["sw"][0].view(-1, 1)
        front = qb.nn.HadamardQuantizer(L["K"]) if L["khad"] else qb.nn.Quantizer()
        mods.append(torch.nn.Sequential(front, lin))
        hx.append(L["x"][0].cpu().pin_memory())
        hout.append(torch.empty((M, L["N"]), dtype=torch.float16).pin_memory())
    h2d_bytes = sum(t.numel() * 2 for t in hx)
    d2h_bytes = sum(t.numel() * 2 for t in hout)
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dx = [torch.empty_like(L["x"][0]) for L in work]

    def step():
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)
        ready = []
        with torch.cuda.stream(s_in):
            for i in range(len(work)):
                dx[i].copy_(hx[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
                ready.append(ev)
        for i in range(len(work)):
            main.wait_event(ready[i])
            out = mods[i](dx[i])
            done = torch.cuda.Event()
            done.record(main)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                hout[i].copy_(out, non_blocking=True)
                out.record_stream(s_out)
        # no join here: the copy-out of this step overlaps the copy-in and the kernels of the next one (the host link
        # is full duplex); inputs are safe because the next copy-in waits for an event recorded behind this step's
        # kernels, outputs because the copy-out stream keeps its order

    def copies_only(which):
        """The step's host copies alone, one direction at a time: what the host link gives this rank."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        douts = [torch.empty((M, L["N"]), dtype=torch.float16, device=dev) for L in work] if which == "d2h" else None
        torch.cuda.synchronize(dev)
        e0.record(main)
        for _ in range(3):
            for i in range(len(work)):
                if which == "h2d":
                    dx[i].copy_(hx[i], non_blocking=True)
                else:
                    hout[i].copy_(douts[i], non_blocking=True)
        e1.record(main)
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / 3

    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for _ in range(steps):
        step()
    main.wait_stream(s_out)          # the timed region ends when the last result has reached the host
    e1.record(main)
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    h2d_ms, d2h_ms = copies_only("h2d"), copies_only("d2h")
    return ms, h2d_bytes, d2h_bytes, h2d_ms, d2h_ms


def colsplit_run(steps, warmup, layers, M, dev, world, rank, dist):
    """Column split: rank r owns N/G output channels of each linear; kernel (a) runs on all M rows on every
    rank, the local GEMM produces [M, N/G], the slabs are all-gathered and interleaved into [M, N].
    Times the local compute alone and compute + collective (CUDA events, max over ranks)."""
    import quarot_b200 as qb
    from quarot_b200 import dist as qd, synth
    from quarot_b200.functional import hadamard as FH
    mods = []
    for li, (name, K, N, had) in enumerate(layers):
        khad = FH.get_hadK(K)[1] if had else 0
        table = FH.device_table(khad, dev) if khad > 1 else None
        x = synth.activations_device(M, K, seed=1234 + li, device=dev)
        w, sw = synth.weights_device(N // world, K, seed=4321 + li + 100 * rank, device=dev)
        lin = qd.ColumnSplitLinear4bit.__new__(qd.ColumnSplitLinear4bit)
        torch.nn.Module.__init__(lin)
        lin.group, lin.world, lin.rank = None, world, rank
        lin.register_buffer("weight", w)
        lin.register_buffer("weight_scales", sw)
        lin.bias, lin.out_features, lin._compute = None, N, qb.linear_i4
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
        mods.append((name, K, N, khad, table, x, lin, out))

    # third mode: the epilogue stores straight into every rank's [M, N] matrix (symmetric memory), no all-gather
    fused = None
    if dist is not None:
        try:
            fused = []
            for (name, K, N, khad, table, x, lin, out) in mods:
                f = qd.FusedColumnSplitLinear4bit.__new__(qd.FusedColumnSplitLinear4bit)
                torch.nn.Module.__init__(f)
                f.group, f.world, f.rank = None, world, rank
                f.register_buffer("weight", lin.weight)
                f.register_buffer("weight_scales", lin.weight_scales)
                f.bias, f.out_features, f._compute = None, N, qb.linear_i4
                fused.append((f, qd.SymmetricOutput(M, N, dev)))
        except Exception as e:        # symmetric memory not available on this box: report the other two modes
            sys.stderr.write("bench.py: fused column split skipped: %r\n" % (e,))
            fused = None

    def step(collective):
        for i, (name, K, N, khad, table, x, lin, out) in enumerate(mods):
            q, s, _ = qb.hadamard_quant(x, table, khad, 1.0)
            pq = qb.PackedQuantizedTensor(q, s)
            if collective == "fused":
                fused[i][0](pq, fused[i][1])
            elif collective:
                lin(pq, gathered_out=out)
            else:
                lin.local_forward(pq)

    res = {}
    modes = [("compute_ms", False), ("compute_plus_allgather_ms", True)]
    if fused is not None:
        modes.append(("fused_peer_store_ms", "fused"))
    for label, coll in modes:
        res[label], _ = timed_steps(dev, dist, lambda i: step(coll), steps, max(warmup, 3))
    return res


def colsplit_line_parts(res, layers, M, n_gpus):
    ops = layer_ops(layers, M)           # whole job: every output channel is computed exactly once
    tops = lambda t: ops / (t * 1e-3) / 1e12
    exchanged = sum(2 * M * (N // n_gpus) * (n_gpus - 1) for (_, _, N, _) in layers)
    out = {"compute_only": {"ms_per_step": res["compute_ms"], "value": tops(res["compute_ms"]), "unit": "TOPS"},
           "nccl_allgather": {"ms_per_step": res["compute_plus_allgather_ms"],
                              "value": tops(res["compute_plus_allgather_ms"]), "unit": "TOPS"},
           "fused_peer_store": None, "exchanged_bytes_per_rank": exchanged}
    if "fused_peer_store_ms" in res:
        t = res["fused_peer_store_ms"]
        out["fused_peer_store"] = {"ms_per_step": t, "value": tops(t), "unit": "TOPS",
                                   "nvlink_out_gbs_per_rank": exchanged / (t * 1e-3) / 1e9}
    return out


def multi_gpu_parity(dev, world, rank, dist):
    """Small-shape equality checks of the multi-GPU forms against the single-GPU result (outside any timed region):
    row sharding, column split with the NCCL all-gather, column split with the epilogue storing into the peers."""
    import quarot_b200 as qb
    from quarot_b200 import dist as qd, synth
    M, K, N = 64 * world + 192, 1024, 512 * world
    x = synth.activations(M, K, seed=5).to(dev)
    w, sw = synth.weights(N, K, seed=6)
    w, sw = w.to(dev), sw.to(dev)
    q, s, _ = qb.hadamard_quant(x, None, 0, 1.0)
    single = qb.linear_i4(q, s, w, sw)
    out = {}
    lo, hi = qd.shard_rows(M, world, rank)
    ql, sl, _ = qb.hadamard_quant(x[lo:hi].contiguous(), None, 0, 1.0)
    rows = qd.gather_rows(qb.linear_i4(ql, sl, w, sw), M)
    out["row_sharded"] = bool(torch.equal(rows, single))
    pq = qb.PackedQuantizedTensor(q, s)
    col = qd.ColumnSplitLinear4bit(w, sw.view(-1, 1))
    out["column_split_nccl_allgather"] = bool(torch.equal(col(pq).view(M, N), single))
    try:
        fused = qd.FusedColumnSplitLinear4bit(w, sw.view(-1, 1))
        target = qd.SymmetricOutput(M, N, dev)
        ok = True
        for _ in range(2):
            ok = ok and bool(torch.equal(fused(pq, target), single))
        out["column_split_fused_peer_store"] = ok
    except Exception as exc:
        out["column_split_fused_peer_store"] = "skipped: %r" % (exc,)
    flags = torch.tensor([1 if v is True or isinstance(v, str) else 0 for v in out.values()], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    out["all_ranks_ok"] = bool(int(flags.min()) == 1)
    out["shape"] = {"M": M, "K": K, "N": N}
    return out


def mlp_run(args, layers, M, dev):
    """One MLP block: Quantizer -> gate/up Linear4bit -> act_fn(gate) * up -> OnlineHadamard + Quantizer -> down
    Linear4bit.  Two variants: the product as torch elementwise kernels on the [M, 2 I] GEMM output, and the
    product inside the GEMM epilogue (the projections never reach memory).  CUDA events, buffers larger than L2."""
    import quarot_b200 as qb
    from quarot_b200 import synth
    from quarot_b200.functional import hadamard as FH
    (_, K, N2, _), (_, I, Nd, _) = layers
    nsets = 3
    xs = [synth.activations_device(M, K, seed=77 + i, device=dev) for i in range(nsets)]
    wgu = [synth.weights_device(N2, K, seed=88 + i, device=dev) for i in range(nsets)]     # rows already interleaved
    wd = [synth.weights_device(Nd, I, seed=99 + i, device=dev) for i in range(nsets)]
    khad = FH.get_hadK(I)[1]
    table = FH.device_table(khad, dev) if khad > 1 else None
    both = torch.empty((M, N2), dtype=torch.float16, device=dev)
    hbuf = torch.empty((M, I), dtype=torch.float16, device=dev)
    out = torch.empty((M, Nd), dtype=torch.float16, device=dev)

    def step(i, fused):
        q, s, _ = qb.hadamard_quant(xs[i], None, 0, 1.0)
        if fused:
            h = qb.linear_i4_swiglu(q, s, wgu[i][0], wgu[i][1].view(-1), out=hbuf)
        else:
            g_u = qb.linear_i4(q, s, wgu[i][0], wgu[i][1].view(-1), out=both).view(M, -1, 2, 128)
            h = (torch.nn.functional.silu(g_u[:, :, 0, :]) * g_u[:, :, 1, :]).reshape(M, I)
        q2, s2, _ = qb.hadamard_quant(h, table, khad, 1.0)
        qb.linear_i4(q2, s2, wd[i][0], wd[i][1].view(-1), out=out)

    res = {}
    for label, fused in (("unfused_ms", False), ("fused_ms", True)):
        res[label], _ = timed_steps(dev, None, lambda i: step(i % nsets, fused), args.steps, max(args.warmup, nsets))
    return res


def norm_run(args, M, K, dev):
    """RMSNorm + Quantizer of an [M, K] hidden state: the fused kernel against the two modules (torch elementwise
    and reduction kernels for the norm, the quantise-only kernel behind it).  CUDA events, rotating inputs > L2."""
    import quarot_b200 as qb
    from quarot_b200 import synth
    from quarot_b200.nn.fused import RMSNormQuantizer
    nsets = 12
    xs = [synth.activations_device(M, K, seed=7 + i, device=dev) for i in range(nsets)]
    fused = RMSNormQuantizer(K)
    norm, quant = qb.nn.RMSNorm(K), qb.nn.Quantizer()
    res = {}
    for label, fn in (("unfused_ms", lambda x: quant(norm(x))), ("fused_ms", fused)):
        res[label], _ = timed_steps(dev, None, lambda i: fn(xs[i % nsets]), args.steps, max(args.warmup, 3))
    return res


def heads_hadamard_run(dev, steps, warmup):
    """The small online Hadamard over the heads axis in front of o_proj (a transposed view [B, S, head_dim, heads],
    n = 32 for LLaMA-2-7B): read + write of the [2048, 4096] fp16 attention output."""
    import quarot_b200 as qb
    M, heads, hd = 2048, 32, 128
    had = qb.nn.OnlineHadamard(heads)
    xs = [torch.randn(1, M, heads, hd, device=dev, dtype=torch.float16) for _ in range(12)]
    for i in range(12):
        had(xs[i].transpose(-1, -2))
    # one graph per tensor (12 x 16.8 MB, more than the L2 holds), so that the figure is the kernel's and not the
    # eager Python call's
    graphs = capture_graphs(dev, 12, lambda i: had(xs[i].transpose(-1, -2)))
    if graphs is not None:
        ms, _ = timed_steps(dev, None, lambda i: graphs[i % 12].replay(), steps, warmup)
    else:
        ms, _ = timed_steps(dev, None, lambda i: had(xs[i % 12].transpose(-1, -2)), steps, warmup)
    nbytes = 2.0 * 2 * M * heads * hd
    return {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "shape": [1, M, heads, hd],
            "launch_mode": "cuda_graph_replay" if graphs is not None else "eager"}


# --profile-case NAME: the launches one kernel summary under profiles/ was captured from.  Every case runs its kernel
# a few times on inputs larger than L2 where the kernel streams from HBM, and nothing else of the benchmark.
PROFILE_CASES = {
    # name: (kind, M, K, N or Kronecker factor)
    "gemm_qkv": ("linear", 2048, 4096, 12288),
    "gemm_o": ("linear", 2048, 4096, 4096),
    "gemm_gate_up": ("linear", 2048, 4096, 22016),
    "gemm_down": ("linear", 2048, 11008, 4096),
    "decode1_qkv": ("linear", 1, 4096, 12288),            # mma.sync weight-streaming kernel
    "decode8_qkv": ("linear", 8, 4096, 12288),
    "decode16_down": ("linear", 16, 11008, 4096),
    "decode32_gate_up": ("linear", 32, 4096, 22016),
    "decode64_qkv": ("linear", 64, 4096, 12288),          # tcgen05 decode kernel, row split
    "decode64_down": ("linear", 64, 11008, 4096),         # tcgen05 decode kernel, unit split
    "decode1_quant_qkv": ("quant_linear", 1, 4096, 12288),  # CUDA-core kernel with the quantiser inside
    "quant_4096": ("hadq", 2048, 4096, 0),
    "walsh_4096": ("hadq", 2048, 4096, 1),
    "had_172x64": ("hadq", 2048, 11008, 172),
    "had_28x1024": ("hadq", 1024, 28672, 28),
    "heads_axis": ("heads", 2048, 4096, 32),
    "kv_decode": ("kv", 16, 2048, 32),
}


def profile_case(name, dev, reps=3):
    import quarot_b200 as qb
    from quarot_b200 import synth, _lib
    from quarot_b200.functional import hadamard as FH
    kind, M, K, N = PROFILE_CASES[name]
    if kind == "linear":
        x = synth.activations_device(M, K, device=dev)
        w, sw = synth.weights_device(N, K, device=dev)
        q, sx, _ = qb.hadamard_quant(x, None, 0, 1.0)
        fn = lambda: qb.linear_i4(q, sx, w, sw.view(-1))
    elif kind == "quant_linear":
        x = synth.activations_device(M, K, device=dev)
        w, sw = synth.weights_device(N, K, device=dev)
        fn = lambda: qb.quant_linear_i4(x, w, sw.view(-1))
    elif kind == "hadq":
        x = synth.activations_device(M, K, device=dev)
        table = FH.device_table(N, dev) if N > 1 else None
        fn = lambda: qb.hadamard_quant(x, table, N, 1.0)
    elif kind == "heads":
        x = torch.randn(M, N, K // N, device=dev, dtype=torch.float16)
        had = qb.nn.OnlineHadamard(N)
        fn = lambda: had(x.transpose(-1, -2))
    else:
        cache, attend, qv = kv_decode_setup(dev, batch=M, seq=K, heads=N)
        fn = lambda: attend(qv)
    for _ in range(reps):
        fn()
    torch.cuda.synchronize(dev)
    if _lib.kernel_status() != 0:
        raise SystemExit("bench.py: kernel status %d" % _lib.kernel_status())
    print(json.dumps({"profile_case": name, "launch_groups": reps}))


def kv_decode_setup(dev, batch, seq, heads, page=16):
    """A paged 4-bit KV cache of `batch` sequences of `seq` tokens (one layer, head_dim 128, keys Hadamard-
    transformed), and the attention callable for one new token per sequence."""
    from quarot_b200.transformers import MultiLayerPagedKVCache4Bit
    g = torch.Generator().manual_seed(7)
    cache = MultiLayerPagedKVCache4Bit(batch, page, seq + 8, dev, 1, heads, 128, hadamard_dtype=torch.float16)
    k = (torch.randn(batch, seq, heads, 128, generator=g) * 2.0).half().to(dev)
    v = (torch.randn(batch, seq, heads, 128, generator=g) * 2.0).half().to(dev)
    cache.update(k, v, 0, {})
    k1 = (torch.randn(batch, 1, heads, 128, generator=g) * 2.0).half().to(dev)
    v1 = (torch.randn(batch, 1, heads, 128, generator=g) * 2.0).half().to(dev)
    attend = cache.update(k1, v1, 0, {})
    qv = (torch.randn(batch, 1, heads, 128, generator=g) * 1.5).half().to(dev)
    return cache, attend, qv


def kv_decode_run(dev, steps, warmup, batch=16, seq=2048, heads=32):
    """Decode attention over the paged 4-bit cache (the row after the linears): one new token per sequence against
    `seq` cached tokens; algorithmic bytes = packed K and V codes plus their (scale, zero) pairs, read once."""
    cache, attend, qv = kv_decode_setup(dev, batch, seq, heads)
    for _ in range(max(warmup, 3)):
        attend(qv)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        attend(qv)
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    tokens = batch * (seq + 1)
    nbytes = tokens * heads * 2 * (64 + 4)
    return {"ms_per_step": ms, "batch": batch, "cached_tokens": seq + 1, "heads": heads, "page_size": 16,
            "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / (ms * 1e-3) / 1e9,
            "note": "eager launches; the %.1f MB of pages exceed the 126 MB L2" % (nbytes / 1e6)}


def other_configs(qb, dev, dist, world, rank, peaks, peak_src, headline_workload, int8_probe):
    """Short device-timed runs of the benchmark configurations that are not the headline."""
    out = {}
    steps, warmup = 10, 3

    def one(name, table, M, st=steps):
        layers = LAYERS[table]
        r = measure_layers(qb, layers, M, dev, None, st, warmup)
        ops = layer_ops(layers, M)
        rec = {"tokens": M, "ms_per_step": r["ms_step"], "value": ops / (r["ms_step"] * 1e-3) / 1e12, "unit": "TOPS",
               "tokens_per_s": M / (r["ms_step"] * 1e-3), "kernel_b_ms": r["gemm_ms"], "kernel_a_ms": r["quant_ms"],
               "launches_per_step": r["launches_per_step"], "launch_mode": r["launch_mode"],
               "roofline": roofline_record(layers, M, r, peaks, peak_src, name, int8_probe, st * r["ms_step"] * 1e-3)}
        if M > DECODE_MAX_M and r["quant_ms"]:
            qbytes = sum(bytes_quant(M, K) for (_, K, _, _) in layers)
            rec["kernel_a_gbs"] = qbytes / (r["quant_ms"] * 1e-3) / 1e9
        del r
        torch.cuda.empty_cache()
        return rec

    if headline_workload != "config0":
        out["config0"] = one("config0", "CONFIG0", 2048, 20)
    if headline_workload != "llama2_7b_prefill":
        out["llama2_7b_prefill"] = one("llama2_7b_prefill", "LLAMA2_7B", 2048)
    for m in (1, 8, 32, 64):
        out["llama2_7b_decode_m%d" % m] = one("llama2_7b_decode", "LLAMA2_7B", m, 30)
    if headline_workload != "llama2_70b_prefill":
        out["llama2_70b_prefill"] = one("llama2_70b_prefill", "LLAMA2_70B", 4096, 5)
    try:
        out["heads_axis_hadamard_n32"] = heads_hadamard_run(dev, 30, 5)
    except Exception as exc:
        out["heads_axis_hadamard_n32"] = {"skipped": repr(exc)}
    try:
        out["kv_cache_decode_attention"] = kv_decode_run(dev, 30, 5)
    except Exception as exc:
        out["kv_cache_decode_attention"] = {"skipped": repr(exc)}
    if world > 1:
        # strong scaling of the 70B layer: the 4096 token rows are split over the ranks
        layers = LAYERS["LLAMA2_70B"]
        m_loc = 4096 // world
        r = measure_layers(qb, layers, m_loc, dev, dist, 5, warmup, breakdown=False)
        ops = layer_ops(layers, 4096)
        out["llama2_70b_prefill_rows_split"] = {
            "tokens_total": 4096, "tokens_per_gpu": m_loc, "ms_per_step": r["ms_step"], "scaling": "strong",
            "value": ops / (r["ms_step"] * 1e-3) / 1e12, "unit": "TOPS", "tokens_per_s": 4096 / (r["ms_step"] * 1e-3)}
        del r
        torch.cuda.empty_cache()
        layers = LAYERS["LLAMA2_70B_MLP"]
        for m in (256, 4096):
            res = colsplit_run(5, 3, layers, m, dev, world, rank, dist)
            rec = colsplit_line_parts(res, layers, m, world)
            rec["tokens"] = m
            out["llama2_70b_mlp_colsplit_m%d" % m] = rec
            torch.cuda.empty_cache()
    return out


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries below (the collective library's version banner, for one) write to file descriptor 1; the contract is
    ONE JSON line on stdout.  Everything but that line goes to stderr from here on."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    text = json.dumps(line) + "\n"
    if _RESULT_FD is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text.encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama2_7b_prefill", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="token rows per GPU (default: the workload's)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip other_configs, the sustained run and the parity block")
    ap.add_argument("--profile-case", default="", choices=[""] + sorted(PROFILE_CASES),
                    help="run one kernel case a few times and exit (the command the ncu summaries under profiles/ name)")
    args = ap.parse_args()
    keep_stdout_for_the_result()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3

    table_name, default_m = WORKLOADS[args.workload]
    layers = LAYERS[table_name]
    M = args.tokens or default_m
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n_gpus = max(args.gpus, world)
    metric = "linear4bit_fused_tops"
    config = {"workload": args.workload, "tokens_per_gpu": M,
              "linears": ["%s %d->%d%s" % (n, K, N, " +hadamard" if h else "") for (n, K, N, h) in layers],
              "sharding": "token rows sharded over ranks, weights replicated, no collective" if n_gpus > 1 else "single GPU",
              "l2": "activations and weights rotate over 3 buffer sets per step (>1 GB, L2 is 126 MB)"}

    # ------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return 0
        r = cpu_reference_run(layers, M, args.steps, max(args.warmup, 1))
        line = {"impl": "reference", "metric": metric, "value": r["value"], "unit": "TOPS", "n_gpus": n_gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step_full"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int4 codes, int32 accumulate (torch CPU int32 matmul)", "data": "synthetic",
                "config": config, "tokens_per_s": r["tokens_per_s"],
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        if not args.no_others:
            # the single-linear configuration (M 2048, K 4096, N 4096) timed in full, one step, no extrapolation
            c0 = cpu_reference_run(LAYERS["CONFIG0"], 2048, 1, 0, rows=2048)
            line["config0_in_full"] = {"ms_per_step": c0["ms_per_step_sample"], "value": c0["value"], "unit": "TOPS",
                                       "tokens": 2048, "cores": c0["cores"]}
        emit(line)
        return 0

    # ------------------------------------------------------------ our arm (GPU)
    import quarot_b200 as qb
    from quarot_b200 import _lib
    for kv in filter(None, os.environ.get("QR_TUNE", "").split(",")):   # kernel-selection knobs: QR_TUNE=gemm_2sm=0,pdl=1
        k, v = kv.split("=")
        if k == "fused_max_rows":
            qb.nn.fused.QuantLinear4bit.FUSED_MAX_ROWS = int(v)
        else:
            _lib.set_tuning(k, int(v))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if args.profile_case:
        profile_case(args.profile_case, dev)
        return 0
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    if args.workload == "llama2_7b_rmsnorm_quant":
        K = layers[0][1]
        res = norm_run(args, M, K, dev)
        nbytes = bytes_quant(M, K)
        line = {"metric": "rmsnorm_quant_gbs", "value": nbytes / (res["fused_ms"] * 1e-3) / 1e9, "unit": "GB/s",
                "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["fused_ms"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 in, fp32 norm, int4 out",
                "data": "synthetic", "config": {"workload": args.workload, "tokens_per_gpu": M, "hidden": K,
                                                "l2": "inputs rotate over 12 buffers (201 MB)"},
                "modules_unfused": {"ms_per_step": res["unfused_ms"]}, "gpu_launches": args.steps}
        emit(line)
        return 0

    if args.workload.endswith("_mlp_swiglu"):
        if world > 1:
            raise SystemExit("bench.py: the MLP-block workload is a single-GPU measurement")
        res = mlp_run(args, layers, M, dev)
        ops = layer_ops(layers, M)
        ms = res["fused_ms"]
        line = {"metric": metric, "value": ops / (ms * 1e-3) / 1e12, "unit": "TOPS", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int4 codes widened to int8, int32 accumulate, fp16 out", "data": "synthetic",
                "config": dict(config, block="Quantizer -> gate/up GEMM with SiLU product in the epilogue -> "
                                             "Hadamard+Quantizer -> down GEMM (eager launches)"),
                "product_as_separate_kernels": {"ms_per_step": res["unfused_ms"],
                                                "value": ops / (res["unfused_ms"] * 1e-3) / 1e12, "unit": "TOPS"},
                "tokens_per_s": M / (ms * 1e-3), "gpu_launches": 4 * args.steps}
        emit(line)
        return 0

    if args.workload == "llama2_70b_mlp_colsplit":
        res = colsplit_run(args.steps, args.warmup, layers, M, dev, world, rank, dist)
        parts = colsplit_line_parts(res, layers, M, n_gpus)
        # headline: the epilogue that stores into the peers' matrices where it ran (N > 1 with symmetric memory),
        # else compute + NCCL all-gather; the other variants are reported beside it
        ms = res.get("fused_peer_store_ms", res["compute_plus_allgather_ms"])
        ops = layer_ops(layers, M)
        line = {"metric": metric, "value": ops / (ms * 1e-3) / 1e12, "unit": "TOPS", "n_gpus": n_gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None,
                "dtype": "int4 codes widened to int8, int32 accumulate, fp16 out", "data": "synthetic",
                "config": dict(config, sharding="output channels split over ranks, every rank quantises all token rows; "
                                                "result assembled on every rank by " +
                                                ("tiled stores of the GEMM epilogue into the peers' matrices (NVLink)"
                                                 if "fused_peer_store_ms" in res else "an NCCL all-gather of the fp16 slabs")),
                "tokens_per_s": M / (ms * 1e-3), "gpu_launches": 2 * len(layers) * args.steps}
        line.update(parts)
        if dist is not None and not args.no_others:
            line["parity"] = multi_gpu_parity(dev, world, rank, dist)
        if rank == 0:
            emit(line)
        if dist is not None:
            dist.destroy_process_group()
        return 0

    peaks, peak_src = load_peaks()
    int8_probe = int8_probe_tops(dev)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    res = measure_layers(qb, layers, M, dev, dist, args.steps, args.warmup, use_graph=not args.no_graph)
    ms_step = res["ms_step"]
    work = res["work"]

    # the same graphs replayed for about three seconds: what the kernels sustain once clocks and power settle; the
    # median SM clock sampled meanwhile lets the clock dependence be read (time x MHz) without touching any setting
    sustained = None
    if not args.no_others:
        n_sus = max(args.steps, int(3000.0 / max(ms_step, 1e-3)))
        sus_ms, win = timed_steps(dev, dist, res["run_all"], n_sus, 0)
        mhz = sampler.window(*win) if sampler else None
        sustained = {"ms_per_step": sus_ms, "steps": n_sus, "seconds": n_sus * sus_ms * 1e-3,
                     "value": layer_ops(layers, M) * n_gpus / (sus_ms * 1e-3) / 1e12, "unit": "TOPS",
                     "sm_mhz_median": mhz, "ms_times_mhz": (sus_ms * mhz) if mhz else None}
    burst_mhz = sampler.window(*res["window"]) if sampler else None
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["sm_mhz_timed_region"] = burst_mhz
    status = _lib.kernel_status()
    if status != 0:
        raise SystemExit("bench.py: a kernel reported a wait timeout (status %d)" % status)

    total_ops = layer_ops(layers, M) * n_gpus
    value = total_ops / (ms_step * 1e-3) / 1e12
    roofline = roofline_record(layers, M, res, peaks, peak_src, args.workload, int8_probe, args.steps * ms_step * 1e-3)
    line = {"metric": metric, "value": value, "unit": "TOPS", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int4 codes widened to int8, int32 accumulate, fp16 out",
            "data": "synthetic", "config": config,
            "tokens_per_s": M * n_gpus / (ms_step * 1e-3),
            "gpu_launches": res["launches_per_step"] * args.steps,
            "launch_mode": res["launch_mode"],
            "roofline": roofline,
            "kernel_ms": {"kernel_b_all_linears": res["gemm_ms"], "kernel_a_all_linears": res["quant_ms"],
                          "how": "each kernel family replayed alone as its own CUDA graph over the same buffers"},
            "sustained": sustained, "clocks": clocks}
    if res["quant_ms"]:
        qbytes = sum(bytes_quant(M, K) for (_, K, _, _) in layers)
        quant_gbs = qbytes / (res["quant_ms"] * 1e-3) / 1e9
        line["quant_kernel"] = {"bound": "hbm", "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": quant_gbs / peaks["hbm_gbs"], "ms_per_step": res["quant_ms"]}

    if not args.no_e2e:
        e2e_ms, h2d, d2h, h2d_ms, d2h_ms = e2e_run(qb, layers, M, dev, max(3, min(args.steps, 10)), 6, work)
        if dist is not None:
            t = torch.tensor([e2e_ms, h2d_ms, d2h_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms, h2d_ms, d2h_ms = (float(v) for v in t.tolist())
        line["e2e"] = {"value": total_ops / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "host_link_gbs": (h2d + d2h) / (e2e_ms * 1e-3) / 1e9,
                       "h2d_alone_gbs_per_rank": h2d / (h2d_ms * 1e-3) / 1e9,
                       "d2h_alone_gbs_per_rank": d2h / (d2h_ms * 1e-3) / 1e9,
                       "api": "torch.nn.Sequential(quarot_b200.nn.[Hadamard]Quantizer, quarot_b200.nn.Linear4bit) "
                              "with pinned host activations in and host fp16 results out"}
    del res, work
    torch.cuda.empty_cache()
    if not args.no_others:
        line["other_configs"] = other_configs(qb, dev, dist, world, rank, peaks, peak_src, args.workload, int8_probe)
        if dist is not None:
            line["parity"] = multi_gpu_parity(dev, world, rank, dist)
        if _lib.kernel_status() != 0:
            raise SystemExit("bench.py: a kernel reported a wait timeout in other_configs")
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = cpu_reference_run(layers, M, 2, 1, budget_s=12.0)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        emit(line)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
