#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path (Hadamard + int4 quantise + int4 GEMM + dequant).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one pass over the linears of one decoder layer for one batch of
token rows: per linear, kernel (a) (fused [Hadamard ->] absmax -> int4 pack) and
kernel (b) (tcgen05 int4 GEMM with the dequant epilogue).  The default workload is
the LLaMA-2-7B layer at prefill size (M = 2048 tokens): QKV 4096->12288, o_proj
4096->4096, gate/up 4096->22016 (quantiser only) and down_proj 11008->4096 with
the online Hadamard had_172 (x) Walsh_64.  Activations and weights are seeded
synthetic tensors with the benchmark's value distributions (quarot_b200/synth.py).

N > 1 (launched with torch.distributed.run, one rank per GPU): token rows are
sharded, weights replicated, no collective on the data path; every rank processes
M rows per step (weak scaling) and the reported value is the whole-job aggregate.

One JSON line is printed by rank 0.  --impl reference times the CPU restatement of
the upstream torch path (oracle/) on the host cores for the same metric and config.
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
            self.lines.append(line.strip())

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
        for line in self.lines:
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
def cpu_reference_run(layers, M_full, steps, warmup, budget_s=20.0):
    """Times the CPU restatement of the upstream torch path on a bounded sample of token rows.

    Weights are unpacked to int32 once, outside the timed region (as the fake-quant
    reference keeps them); per step and per linear: Hadamard (fp32 butterflies, cast
    to fp16), per-token scale, quantise, pack, unpack, int32 matmul, fp32 dequant.
    """
    from oracle import quarot_oracle as O
    from quarot_b200 import synth
    cores = torch.get_num_threads()
    # pick the sample so that one step costs about budget_s / (steps + warmup)
    a = torch.randint(-8, 8, (16, 4096), dtype=torch.int32)
    b = torch.randint(-8, 8, (1024, 4096), dtype=torch.int32)
    t0 = time.perf_counter()
    _ = a @ b.T
    rate = 2.0 * 16 * 1024 * 4096 / max(time.perf_counter() - t0, 1e-6)   # int ops / s
    per_token_ops = layer_ops(layers, 1)
    target = budget_s / max(steps + warmup, 1)
    ms = int(max(1, min(64, M_full, rate * target / per_token_ops)))
    data = []
    for (name, K, N, had) in layers:
        x = synth.activations(ms, K, seed=1234)
        w, sw = synth.weights(N, K, seed=4321)
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
            "ms_per_step_full": dt * 1e3 * (M_full / ms), "tokens_per_s": ms / dt}


# ------------------------------------------------------------------ device arm
def build_device_workload(layers, M, dev, nsets):
    import quarot_b200 as qb
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


def device_step(qb, work, set_idx, record=None):
    for L in work:
        if record is not None:
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
        if L["khad"] == 0 and L["x"][set_idx].shape[0] <= 2:
            # one or two token rows, no transform: the quantiser runs inside the weight-streaming kernel (one launch)
            if record is not None:
                e1.record()
            qb.quant_linear_i4(L["x"][set_idx], L["w"][set_idx], L["sw"][set_idx], out=L["out"])
        else:
            qb.hadamard_quant(L["x"][set_idx], L["table"], L["khad"], 1.0, out_q=L["q"], out_s=L["s"])
            if record is not None:
                e1.record()
            qb.linear_i4(L["q"], L["s"], L["w"][set_idx], L["sw"][set_idx], out=L["out"])
        if record is not None:
            e2.record()
            record.append((L["name"], e0, e1, e2))


def e2e_run(qb, layers, M, dev, steps, warmup, work):
    """Same step through the module API with HOST buffers: per linear, activations are copied
    from pinned host memory, pushed through Sequential([HadamardQuantizer|Quantizer], Linear4bit)
    and the fp16 result is copied back to pinned host memory.  Copies run on their own streams
    so that transfers of neighbouring linears overlap the kernels."""
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
        fin = torch.cuda.Event()
        fin.record(s_out)
        main.wait_event(fin)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    for _ in range(steps):
        step()
    e1.record(main)
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / steps, h2d_bytes, d2h_bytes


def colsplit_run(args, layers, M, dev, world, rank, dist):
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
        for _ in range(max(args.warmup, 3)):
            step(coll)
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step(coll)
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / args.steps
        if dist is not None:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        res[label] = ms
    return res


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
        for i in range(max(args.warmup, nsets)):
            step(i % nsets, fused)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(i % nsets, fused)
        e1.record()
        torch.cuda.synchronize(dev)
        res[label] = e0.elapsed_time(e1) / args.steps
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
        for i in range(max(args.warmup, 3)):
            fn(xs[i % nsets])
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(xs[i % nsets])
        e1.record()
        torch.cuda.synchronize(dev)
        res[label] = e0.elapsed_time(e1) / args.steps
    return res


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
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3

    from quarot_b200 import synth
    table_name, default_m = WORKLOADS[args.workload]
    layers = getattr(synth, table_name)
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
        print(json.dumps(line))
        return 0

    # ------------------------------------------------------------ our arm (GPU)
    import quarot_b200 as qb
    from quarot_b200 import _lib
    for kv in filter(None, os.environ.get("QR_TUNE", "").split(",")):   # experiments: QR_TUNE=gemm_2sm=0,gemm_pst=6
        k, v = kv.split("=")
        _lib.set_tuning(k, int(v))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
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
        print(json.dumps(line))
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
        print(json.dumps(line))
        return 0

    if args.workload == "llama2_70b_mlp_colsplit":
        res = colsplit_run(args, layers, M, dev, world, rank, dist)
        ops = layer_ops(layers, M)           # whole job: every output channel is computed exactly once
        # headline: the epilogue that stores into the peers' matrices where it ran (N > 1 with symmetric memory),
        # else compute + NCCL all-gather; the other variants are reported beside it
        ms = res.get("fused_peer_store_ms", res["compute_plus_allgather_ms"])
        tops = lambda t: ops / (t * 1e-3) / 1e12
        line = {"metric": metric, "value": tops(ms), "unit": "TOPS", "n_gpus": n_gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None,
                "dtype": "int4 codes widened to int8, int32 accumulate, fp16 out", "data": "synthetic",
                "config": dict(config, sharding="output channels split over ranks, every rank quantises all token rows; "
                                                "result assembled on every rank by " +
                                                ("tiled stores of the GEMM epilogue into the peers' matrices (NVLink)"
                                                 if "fused_peer_store_ms" in res else "an NCCL all-gather of the fp16 slabs")),
                "compute_only": {"ms_per_step": res["compute_ms"], "value": tops(res["compute_ms"]), "unit": "TOPS"},
                "nccl_allgather": {"ms_per_step": res["compute_plus_allgather_ms"],
                                   "value": tops(res["compute_plus_allgather_ms"]), "unit": "TOPS"},
                "fused_peer_store": (None if "fused_peer_store_ms" not in res else
                                     {"ms_per_step": res["fused_peer_store_ms"], "value": tops(res["fused_peer_store_ms"]),
                                      "unit": "TOPS"}),
                "exchanged_bytes_per_rank": sum(2 * M * (N // n_gpus) * (n_gpus - 1) for (_, _, N, _) in layers),
                "tokens_per_s": M / (ms * 1e-3), "gpu_launches": 2 * len(layers) * args.steps}
        if rank == 0:
            print(json.dumps(line))
        if dist is not None:
            dist.destroy_process_group()
        return 0

    nsets = 3
    work = build_device_workload(layers, M, dev, nsets)
    for i in range(max(args.warmup, nsets)):
        device_step(qb, work, i % nsets)
    torch.cuda.synchronize(dev)
    # The eight launches of a step are captured once per buffer set into CUDA graphs and replayed, so the
    # timed region measures the kernels and not the Python launch path (--no-graph times eager launches).
    graphs = None
    if not args.no_graph:
        try:
            graphs = []
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for sidx in range(nsets):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        device_step(qb, work, sidx)
                    graphs.append(g)
            torch.cuda.current_stream(dev).wait_stream(side)
            for i in range(args.warmup):
                graphs[i % nsets].replay()
            torch.cuda.synchronize(dev)
        except Exception as exc:   # capture is an optimisation of the harness, not of the kernels
            sys.stderr.write("bench.py: CUDA graph capture failed (%s); timing eager launches\n" % exc)
            graphs = None
            torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        if graphs is not None:
            graphs[i % nsets].replay()
        else:
            device_step(qb, work, i % nsets)
    e1.record()
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    ms_step = e0.elapsed_time(e1) / args.steps
    if dist is not None:
        t = torch.tensor([ms_step], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())

    # instrumented pass over the same steps: CUDA events around every kernel of the timed region
    rec = []
    for i in range(args.steps):
        device_step(qb, work, i % nsets, record=rec)
    torch.cuda.synchronize(dev)
    clocks = sampler.stop() if sampler else None
    per = {}
    for (name, a, b, c) in rec:
        d = per.setdefault(name, {"quant_ms": 0.0, "gemm_ms": 0.0, "n": 0})
        d["quant_ms"] += a.elapsed_time(b)
        d["gemm_ms"] += b.elapsed_time(c)
        d["n"] += 1
    for d in per.values():
        d["quant_ms"] /= d["n"]
        d["gemm_ms"] /= d["n"]
    status = _lib.kernel_status()
    if status != 0:
        raise SystemExit("bench.py: a kernel reported a wait timeout (status %d)" % status)

    total_ops = layer_ops(layers, M) * n_gpus
    value = total_ops / (ms_step * 1e-3) / 1e12
    peaks, peak_src = load_peaks()
    gemm_ms_total = sum(per[n]["gemm_ms"] for (n, _, _, _) in layers)
    quant_ms_total = sum(per[n]["quant_ms"] for (n, _, _, _) in layers)
    gemm_ops = layer_ops(layers, M)
    int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    achieved = gemm_ops / (gemm_ms_total * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "gemm_i4_kernel (4 launches per step, one per linear)",
                "achieved": achieved, "peak": int8_peak, "unit": "TOPS", "frac": achieved / int8_peak,
                "peak_source": "2 x bf16_tflops_sustained of MEASURED_PEAKS.json (%s): dense int8 runs at twice the "
                               "bf16 rate on these tensor cores; no int8 figure is in that file" % peak_src,
                "traffic": None,
                "frac_of_nominal_4500": achieved / 4500.0}
    qbytes = sum(bytes_quant(M, K) for (_, K, _, _) in layers)
    quant_gbs = qbytes / (quant_ms_total * 1e-3) / 1e9
    line = {"metric": metric, "value": value, "unit": "TOPS", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int4 codes widened to int8, int32 accumulate, fp16 out",
            "data": "synthetic", "config": config,
            "tokens_per_s": M * n_gpus / (ms_step * 1e-3),
            "gpu_launches": sum(1 if (L["khad"] == 0 and M <= 2) else 2 for L in work) * args.steps,
            "launch_mode": "cuda_graph_replay" if graphs is not None else "eager",
            "roofline": roofline,
            "quant_kernel": {"bound": "hbm", "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": quant_gbs / peaks["hbm_gbs"], "ms_per_step": quant_ms_total},
            "kernel_ms": per, "clocks": clocks}

    if not args.no_e2e:
        e2e_ms, h2d, d2h = e2e_run(qb, layers, M, dev, max(3, min(args.steps, 10)), 6, work)
        if dist is not None:
            t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        line["e2e"] = {"value": total_ops / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "host_link_gbs": (h2d + d2h) / (e2e_ms * 1e-3) / 1e9,
                       "api": "torch.nn.Sequential(quarot_b200.nn.[Hadamard]Quantizer, quarot_b200.nn.Linear4bit) "
                              "with pinned host activations in and host fp16 results out"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = cpu_reference_run(layers, M, 2, 1, budget_s=12.0)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
