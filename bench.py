"""Benchmark of the quantized matrix-product hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0).  Workloads (synthetic data, seeded):
  decode_8b   (default) configuration 3: Llama-8B-shape decoder, Q4_K attention/FFN weights and a
              Q6_K output projection drawn N(0, 0.02) and encoded on the device, f16 KV cache.
              A 4096-token random prompt is prefilled, then one step = one greedy decode token.
              `roofline` times the dominant kernel (the Q4_K mat-vec) alone over one token's
              matrices: that figure is the Q4_K GEMV HBM GB/s of the headline metric.
  decode_70b  configuration 5 at batch 1 on one GPU (39 GB of Q4_K weights).
  gemv_q4_k   configuration 1: Q4_K 4096x4096 mat-vec, x ~ N(0,1) quantized to Q8_K.
              One step = one mat-vec over each of COPIES distinct weight copies
              (COPIES x 9.4 MB > the 126 MB L2, so every step streams from HBM).
  gemv_q8_0   configuration 2: Q8_0 14336x4096, token batch --ncols in {1, 8, 64}.
  prefill_q4_k configuration 4: the three FFN products of a 2048-token batch on the tensor cores.
  load_gguf   a GGUF file of --layers Llama-8B-shape layers: open + parse + upload to HBM (GB/s).
`value` is measured with operands resident in HBM; `e2e` through the same C-ABI
calls with host (pinned) activation and result buffers, copies inside the timed
region.  `--impl reference` times the reference's own AVX2 kernels
(oracle/_ref, compiled from the reference's headers) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC_GEMV = "Q4_K GEMV HBM GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def ncu_traffic(kernel_key):
    """DRAM bytes per launch from the committed ncu summary, when one exists."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f).get(kernel_key)
    return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl")
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------ GEMV workloads
def gemv_spec(args):
    import emel_cpp_b200 as eb
    if args.workload == "gemv_q4_k":
        t, k, m, n = eb.Q4_K, args.cols or 4096, args.rows or 4096, args.ncols
        name = f"cfg1: Q4_K {m}x{k} mat-vec, x~N(0,1) -> Q8_K" + (f", token batch {n}" if n > 1 else "")
    else:
        t, k, m, n = eb.Q8_0, 4096, 14336, args.ncols
        name = f"cfg2: Q8_0 14336x4096, token batch {n}"
    wbytes = m * eb.row_bytes(t, k)
    copies = max(4, int(np.ceil(640e6 / wbytes)))     # > 5x the 126 MB L2
    return dict(type=t, k=k, m=m, n=n, name=name, wbytes=wbytes, copies=copies,
                alg_bytes=wbytes + 4 * k * n + 4 * m * n)


def run_gemv(args):
    import torch
    import emel_cpp_b200 as eb

    rank, world, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sp = gemv_spec(args)
    t, k, m, n, copies = sp["type"], sp["k"], sp["m"], sp["n"], sp["copies"]
    be = eb.Backend(local)
    stream = torch.cuda.ExternalStream(be.stream(), device=dev)

    # weights: `copies` distinct matrices, N(0, 0.02) encoded on the device (each rank its own)
    wdev = be.alloc(copies * sp["wbytes"])
    for c in range(copies):
        assert be.synth_fill(wdev + c * sp["wbytes"], t, m * k, 1000 + rank * 100 + c, 0.02, 0)
    xdev, ydev = be.alloc(4 * k * n), be.alloc(4 * m * n)
    assert be.synth_fill(xdev, eb.F32, k * n, 7 + rank, 1.0, 0) and be.sync()
    x_host = torch.empty(k * n, dtype=torch.float32).pin_memory()
    y_host = torch.empty(m * n, dtype=torch.float32).pin_memory()
    assert be.to_host(x_host.numpy(), xdev)

    ops_dev = [eb.mul_mat_op(wdev + c * sp["wbytes"], t, k, m, xdev, n, ydev) for c in range(copies)]
    ops_host = [eb.mul_mat_op(wdev + c * sp["wbytes"], t, k, m, x_host, n, y_host) for c in range(copies)]
    src1_view = eb.dense_view(xdev, eb.F32, [n, k])

    def step_dev():
        for op in ops_dev:
            assert be.mul_mat(op)

    def step_host():
        for op in ops_host:
            assert be.mul_mat(op)

    def step_kernel_only():
        for op in ops_dev:
            assert be.mul_mat_prepared(op)

    def capture(fn):
        """One step recorded as a CUDA graph: replay costs one launch per step."""
        fn()
        be.sync()
        d0 = be.diagnostics()["kernel_launches"]
        assert be.graph_begin()
        fn()
        g = be.graph_end()
        return g, be.diagnostics()["kernel_launches"] - d0

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        be.sync()
        barrier(world)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0 = be.diagnostics()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        be.sync()
        torch.cuda.synchronize()
        barrier(world)
        d1 = be.diagnostics()
        ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
        return ms, {k_: d1[k_] - d0[k_] for k_ in d1}

    g_dev, launches_per_step = capture(step_dev)
    assert be.prepare_rhs(src1_view, t)
    g_k, klaunches_per_step = capture(step_kernel_only)
    with ClockSampler(local) as clk:
        ms, _ = timed(lambda: be.graph_launch(g_dev), args.steps, args.warmup)
        assert be.prepare_rhs(src1_view, t)
        ms_k, _ = timed(lambda: be.graph_launch(g_k), args.steps, args.warmup)
        ms_e, de = timed(step_host, args.steps, args.warmup)
    clocks = clk.summary()
    be.graph_destroy(g_dev)
    be.graph_destroy(g_k)
    dd = {"kernel_launches": launches_per_step * args.steps}

    total_bytes = sp["alg_bytes"] * copies * args.steps * world
    value = total_bytes / (ms * 1e-3) / 1e9
    e2e = total_bytes / (ms_e * 1e-3) / 1e9
    launches = copies * args.steps
    kernel_gbs = sp["alg_bytes"] / (ms_k * 1e-3 / launches) / 1e9
    peaks, peak_kind = measured_peaks()
    kname = {eb.Q4_K: "gemv_stream_q4_k", eb.Q8_0: "gemv_stream_q8_0"}[t] + f"_n{n}"
    line = {
        "metric": METRIC_GEMV if args.workload == "gemv_q4_k" else "Q8_0 GEMV HBM GB/s",
        "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 6), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 dot (dp4a) + f32 scales", "data": "synthetic",
        "config": {"workload": sp["name"], "rows": m, "cols": k, "tokens": n, "weight_copies_per_step": copies,
                   "launch": "each step is one CUDA-graph replay of the step's C-ABI calls", "l2_policy": f"inputs larger than L2: {copies} distinct weight copies = {copies * sp['wbytes'] / 1e6:.0f} MB per step",
                   "parallelism": f"{world} independent row-shard replicas, no collective"},
        "pct_of_8tbs_nominal": round(100 * kernel_gbs / NOMINAL_HBM_GBS, 2),
        "e2e": {"value": round(e2e, 2), "unit": "GB/s", "h2d_bytes_per_step": de["h2d_bytes"] // args.steps,
                "d2h_bytes_per_step": de["d2h_bytes"] // args.steps},
        "gpu_launches": int(dd["kernel_launches"]),
        "roofline": {"bound": "hbm", "kernel": kname, "achieved": round(kernel_gbs, 2), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(kernel_gbs / peaks["hbm_gbs"], 4), "peak_source": f"of {peak_kind}",
                     "us_per_launch": round(ms_k * 1e3 / launches, 3), "algorithmic_bytes_per_launch": sp["alg_bytes"],
                     "traffic": ncu_traffic(kname)},
        "clocks": clocks,
    }
    flops = 2.0 * m * k * n
    if flops / sp["alg_bytes"] > peaks["bf16_tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9):
        # past the ridge point the product is bound by the tensor pipe, not by HBM (configuration 2 at 512 tokens)
        tf = flops / (ms_k * 1e-3 / launches) / 1e12
        line["dtype"] = "int8 mma.sync (one 32-weight block per instruction) + f32 scales"
        line["roofline"] = {"bound": "tensor", "kernel": f"gemm_q8_mma_n{n}", "achieved": round(tf, 2), "peak": peaks["bf16_tflops"],
                            "unit": "TFLOP/s", "frac": round(tf / peaks["bf16_tflops"], 4),
                            "peak_source": f"of {peak_kind} (cuBLAS bf16 burst)", "us_per_launch": round(ms_k * 1e3 / launches, 3),
                            "flops_per_launch": flops, "traffic": None}
    elif n >= 3 and t == eb.Q8_0:   # the library's threshold for the mma.sync kernel (kGemmQ8MmaMinCols)
        line["dtype"] = "int8 mma.sync (one 32-weight block per instruction) + f32 scales"
        line["roofline"]["kernel"] = f"gemm_q8_mma_n{n}"
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline_gemv(be, sp, wdev, x_host.numpy().copy(), budget_s=args.cpu_budget)
        print(json.dumps(line), flush=True)
    be.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def cpu_baseline_gemv(be, sp, wdev, x, budget_s=8.0, lanes=None):
    """The reference's AVX2 op_mul_mat (oracle/_ref; the C port where that was never built) on the
    same weight bytes and activations, timed on this host for a bounded sample."""
    from oracle import bindings as ob
    lib = ob.ref()
    kind = "reference" if lib is not None else "port"
    lib = lib or ob.port()
    t, k, m, n = sp["type"], sp["k"], sp["m"], sp["n"]
    w = np.zeros(sp["wbytes"], np.uint8)
    assert be.to_host(w, wdev)
    y = np.zeros((m, n), np.float32)
    op = ob.mul_mat_op(w, t, k, m, x, n, y)
    cores = lanes or min(8, os.cpu_count() or 1)
    kw = {"route": "avx2", "lanes": cores} if kind == "reference" else {}
    if kind == "port":
        cores = 1
    assert lib.mul_mat(op, **kw)            # warm-up
    reps, t0 = 0, time.perf_counter()
    while True:
        assert lib.mul_mat(op, **kw)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 2000:
            break
    gbs = sp["alg_bytes"] * reps / dt / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{reps} x {sp['name']} in {dt:.1f} s, AVX2/FMA route, row-sliced over {cores} threads",
            "us_per_op": round(dt / reps * 1e6, 1)}


def run_reference_gemv(args):
    """--impl reference: the reference's own CPU kernels for the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import emel_cpp_b200 as eb
    from oracle import bindings as ob
    sp = gemv_spec(args)
    t, k, m, n = sp["type"], sp["k"], sp["m"], sp["n"]
    lib = ob.ref()
    kind = "reference" if lib is not None else "port"
    lib = lib or ob.port()
    rng = np.random.Generator(np.random.PCG64(1000))
    # weights: random block bytes with sane scales (the CPU arm's time does not depend on the values)
    w = rng.integers(0, 256, size=sp["wbytes"], dtype=np.uint8)
    bb = eb.BLOCK_BYTES[t]
    blocks = w.reshape(-1, bb)
    for off in ({eb.Q4_K: (0, 2), eb.Q6_K: (208,), eb.Q8_0: (0,), eb.Q4_0: (0,)}[t]):
        blocks[:, off] = rng.integers(0, 256, size=blocks.shape[0])
        blocks[:, off + 1] = rng.integers(0x18, 0x30, size=blocks.shape[0])
    x = rng.standard_normal((k, n), dtype=np.float32)
    y = np.zeros((m, n), np.float32)
    op = ob.mul_mat_op(w, t, k, m, x, n, y)
    lanes = min(8, os.cpu_count() or 1)   # the reference's own maximum lane count (src/emel/kernel/matmul/guards.hpp:12-14)
    kw = {"route": "avx2", "lanes": lanes} if kind == "reference" else {}
    per_step = sp["copies"]               # a step is the same number of mat-vecs as on the GPU arm
    for _ in range(args.warmup):
        assert lib.mul_mat(op, **kw)
    t0 = time.perf_counter()
    for _ in range(args.steps * per_step):
        assert lib.mul_mat(op, **kw)
    dt = time.perf_counter() - t0
    gbs = sp["alg_bytes"] * args.steps * per_step / dt / 1e9
    line = {"impl": "reference", "metric": METRIC_GEMV if args.workload == "gemv_q4_k" else "Q8_0 GEMV HBM GB/s",
            "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot (AVX2 maddubs) + f32 scales", "data": "synthetic",
            "config": {"workload": sp["name"], "rows": m, "cols": k, "tokens": n, "weight_copies_per_step": sp["copies"],
                       "launch": "each step is that many op_mul_mat calls on the host",
                       "l2_policy": "one weight matrix reused (the CPU kernels are compute-bound)",
                       "parallelism": f"{lanes} host threads (row slices, the reference's maximum lane count)"},
            "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": lanes if kind == "reference" else 1, "kind": kind,
                             "sample": f"{args.steps} steps of {per_step} mat-vecs, measured"},
            "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ prompt-processing products (configuration 4)
def prefill_spec(args):
    n = args.ncols if args.ncols > 1 else 2048
    return dict(n=n, n_embd=4096, n_ff=14336,
                name=f"cfg4: {n} tokens x (gate, up 14336x4096 + down 4096x14336) Q4_K, activations -> Q8_K",
                flops=2.0 * n * 3 * 4096 * 14336)


def run_prefill(args):
    """One step = the three FFN matrix products of one layer for a token batch (gate and up share the
    quantized activations).  The dominant kernel is the tcgen05 int8 kernel; its roofline is the tensor
    pipe, reported against the measured bf16 GEMM peak (the int8 pipe's nominal peak is twice that)."""
    import torch
    import emel_cpp_b200 as eb

    rank, world, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sp = prefill_spec(args)
    n, ke, kf = sp["n"], sp["n_embd"], sp["n_ff"]
    be = eb.Backend(local)
    stream = torch.cuda.ExternalStream(be.stream(), device=dev)
    t = eb.Q4_K
    wg, wu, wd = (be.alloc(kf * eb.row_bytes(t, ke)), be.alloc(kf * eb.row_bytes(t, ke)), be.alloc(ke * eb.row_bytes(t, kf)))
    for i, (w, m, k) in enumerate(((wg, kf, ke), (wu, kf, ke), (wd, ke, kf))):
        assert be.synth_fill(w, t, m * k, 3000 + 10 * rank + i, 0.02, 0)
    x, h = be.alloc(4 * ke * n), be.alloc(4 * kf * n)
    assert be.synth_fill(x, eb.F32, ke * n, 11 + rank, 1.0, 0) and be.synth_fill(h, eb.F32, kf * n, 12 + rank, 1.0, 0)
    yg, yu, yd = be.alloc(4 * kf * n), be.alloc(4 * kf * n), be.alloc(4 * ke * n)
    x_host = torch.empty(ke * n, dtype=torch.float32).pin_memory()
    h_host = torch.empty(kf * n, dtype=torch.float32).pin_memory()
    y_host = torch.empty(kf * n, dtype=torch.float32).pin_memory()
    assert be.to_host(x_host.numpy(), x) and be.to_host(h_host.numpy(), h) and be.sync()
    op_g, op_u, op_d = (eb.mul_mat_op(wg, t, ke, kf, x, n, yg), eb.mul_mat_op(wu, t, ke, kf, x, n, yu),
                        eb.mul_mat_op(wd, t, kf, ke, h, n, yd))
    xv, hv = eb.dense_view(x, eb.F32, [n, ke]), eb.dense_view(h, eb.F32, [n, kf])

    def step_dev():            # quantize once per distinct right-hand side, then the products
        assert be.prepare_rhs(xv, t) and be.mul_mat_prepared(op_g) and be.mul_mat_prepared(op_u)
        assert be.prepare_rhs(hv, t) and be.mul_mat_prepared(op_d)

    def step_host():           # host activations in, host results out, through the plain op_mul_mat call
        assert be.mul_mat(eb.mul_mat_op(wg, t, ke, kf, x_host, n, y_host))
        assert be.mul_mat(eb.mul_mat_op(wu, t, ke, kf, x_host, n, y_host))
        assert be.mul_mat(eb.mul_mat_op(wd, t, kf, ke, h_host, n, y_host[:ke * n]))

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        be.sync()
        barrier(world)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0 = be.diagnostics()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        be.sync()
        torch.cuda.synchronize()
        barrier(world)
        d1 = be.diagnostics()
        return max_over_ranks(e0.elapsed_time(e1), world, dev), {k_: d1[k_] - d0[k_] for k_ in d1}

    l0 = be.diagnostics()["kernel_launches"]
    step_dev()
    be.sync()
    launches_per_step = be.diagnostics()["kernel_launches"] - l0
    assert be.graph_begin()
    step_dev()
    g = be.graph_end()
    # the products alone (activations already quantized): gate + up share one graph, timed per launch
    assert be.prepare_rhs(xv, t)
    assert be.graph_begin()
    assert be.mul_mat_prepared(op_g) and be.mul_mat_prepared(op_u)
    gk = be.graph_end()
    with ClockSampler(local) as clk:
        ms, dd = timed(lambda: be.graph_launch(g), args.steps, args.warmup)
        assert be.prepare_rhs(xv, t)
        ms_k, _ = timed(lambda: be.graph_launch(gk), args.steps, args.warmup)
        e_steps = max(1, min(args.steps, 4))
        ms_e, de = timed(step_host, e_steps, 1)
    clocks = clk.summary()
    peaks, peak_kind = measured_peaks()
    tflops = sp["flops"] * args.steps * world / (ms * 1e-3) / 1e12
    tflops_e = sp["flops"] * e_steps * world / (ms_e * 1e-3) / 1e12
    k_flops = 2.0 * n * ke * kf                                  # one 14336x4096 product
    k_tflops = k_flops / (ms_k * 1e-3 / (2 * args.steps)) / 1e12
    line = {
        "metric": "prefill GEMM TFLOP/s", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 tcgen05.mma (s32 accumulators in TMEM) + f32 block scales", "data": "synthetic",
        "config": {"workload": sp["name"], "tokens": n, "launch": "each step is one CUDA-graph replay: 2 activation quantizers + 3 products",
                   "l2_policy": f"inputs larger than L2: {(4 * (ke + kf) * n + 3 * kf * eb.row_bytes(t, ke)) / 1e6:.0f} MB of operands, "
                                f"{4 * (2 * kf + ke) * n / 1e6:.0f} MB of results per step",
                   "parallelism": "single GPU" if world == 1 else f"{world} independent replicas, no collective"},
        "e2e": {"value": round(tflops_e, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": de["h2d_bytes"] // e_steps,
                "d2h_bytes_per_step": de["d2h_bytes"] // e_steps},
        "gpu_launches": int(launches_per_step * args.steps),
        "roofline": {"bound": "tensor", "kernel": "gemm_q4k_tc", "achieved": round(k_tflops, 2), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(k_tflops / peaks["bf16_tflops"], 4),
                     "peak_source": f"of {peak_kind} (cuBLAS bf16 burst; the kernel's MMAs are int8 and issue two per useful one)",
                     "us_per_launch": round(ms_k * 1e3 / (2 * args.steps), 2), "flops_per_launch": k_flops, "traffic": None},
        "clocks": clocks,
    }
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline_prefill(sp, args.cpu_budget)
        print(json.dumps(line), flush=True)
    be.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def cpu_baseline_prefill(sp, budget_s, lanes=None):
    """The reference's AVX2 op_mul_mat on a bounded sample: the gate product for 16 of the tokens."""
    import emel_cpp_b200 as eb
    from oracle import bindings as ob
    lib = ob.ref()
    kind = "reference" if lib is not None else "port"
    lib = lib or ob.port()
    k, m, n = sp["n_embd"], sp["n_ff"], 16
    rng = np.random.Generator(np.random.PCG64(5))
    w = rng.integers(0, 256, size=m * eb.row_bytes(eb.Q4_K, k), dtype=np.uint8).reshape(-1, eb.BLOCK_BYTES[eb.Q4_K])
    w[:, 1] = rng.integers(0x18, 0x30, size=w.shape[0])
    w[:, 3] = rng.integers(0x18, 0x30, size=w.shape[0])
    x, y = rng.standard_normal((k, n), dtype=np.float32), np.zeros((m, n), np.float32)
    op = ob.mul_mat_op(w.reshape(-1), eb.Q4_K, k, m, x, n, y)
    lanes = lanes or min(8, os.cpu_count() or 1)
    kw = {"route": "avx2", "lanes": lanes} if kind == "reference" else {}
    assert lib.mul_mat(op, **kw)
    reps, t0 = 0, time.perf_counter()
    while True:
        assert lib.mul_mat(op, **kw)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 200:
            break
    tf = 2.0 * k * m * n * reps / dt / 1e12
    return {"value": round(tf, 5), "unit": "TFLOP/s", "cores": lanes if kind == "reference" else 1, "kind": kind,
            "sample": f"{reps} x (14336x4096 Q4_K product for {n} tokens) in {dt:.1f} s, AVX2/FMA route, row-sliced over {lanes} threads"}


def run_reference_prefill(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sp = prefill_spec(args)
    t0 = time.perf_counter()
    res = [cpu_baseline_prefill(sp, 2.0, lanes=min(os.cpu_count() or 1, 8)) for _ in range(max(1, min(args.steps, 5)))]
    v = float(np.median([r["value"] for r in res]))
    line = {"impl": "reference", "metric": "prefill GEMM TFLOP/s", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sp["flops"] / (v * 1e12) * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot (AVX2 maddubs) + f32 scales",
            "data": "synthetic", "config": {"workload": sp["name"], "tokens": sp["n"]},
            "cpu_baseline": dict(res[0], value=v),
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)



# ------------------------------------------------------------------ GGUF file -> HBM
def load_spec(args):
    layers = args.layers
    per_layer = [("attn_q", 4096, 4096), ("attn_k", 4096, 1024), ("attn_v", 4096, 1024), ("attn_output", 4096, 4096),
                 ("ffn_gate", 4096, 14336), ("ffn_up", 4096, 14336), ("ffn_down", 14336, 4096)]
    return dict(layers=layers, per_layer=per_layer,
                name=f"GGUF file of {layers} Llama-8B-shape layers (Q4_K matrices, f32 norms): open + parse + upload every tensor")


def write_load_file(sp, path, seed=20):
    """Streams a GGUF v3 file to `path`: random block bytes (the loader never decodes them)."""
    from emel_cpp_b200 import gguf_image as gi
    rng = np.random.default_rng(seed)
    pool = rng.integers(0, 256, size=64 << 20, dtype=np.uint8)
    tensors = []
    for l in range(sp["layers"]):
        tensors.append((f"blk.{l}.attn_norm.weight", (4096,), 0, 4096 * 4))
        tensors.append((f"blk.{l}.ffn_norm.weight", (4096,), 0, 4096 * 4))
        for stem, k, m in sp["per_layer"]:
            tensors.append((f"blk.{l}.{stem}.weight", (k, m), 12, k // 256 * 144 * m))
    head = bytearray(b"GGUF" + np.array([3], "<u4").tobytes() + np.array([len(tensors), 2], "<u8").tobytes())
    head += gi.kv("general.architecture", gi.T_STRING, "llama") + gi.kv("general.alignment", gi.T_UINT32, 32)
    off = 0
    for name, dims, t, nbytes in tensors:
        head += gi.tensor_info(name, dims, t, off)
        off += gi.pad(nbytes, 32)
    head += b"\0" * (gi.pad(len(head), 32) - len(head))
    with open(path, "wb") as fh:
        fh.write(head)
        at = 0
        for _name, _dims, _t, nbytes in tensors:
            left = gi.pad(nbytes, 32)
            while left:
                n = min(left, pool.size - at)
                fh.write(pool[at:at + n].data)
                at = (at + n) % pool.size
                left -= n
    return len(head) + off


def load_dir():
    for d in ("/dev/shm", tempfile.gettempdir()):
        if os.path.isdir(d) and os.access(d, os.W_OK):
            return tempfile.mkdtemp(prefix="emelb_gguf_", dir=d)
    return tempfile.mkdtemp(prefix="emelb_gguf_")


def reference_parse_us(path, repeats=5):
    """-> (reference us, this library us, kind): probe + parse of the file's metadata by the reference's
    own functions (oracle/_ref; the oracle port when that was not built) and by emelb_gguf_open_image,
    both on an in-memory image of the file's size whose tensor data is left zero (neither reads it)."""
    import ctypes as C
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import gguf
    from oracle import bindings as ob, gguf_oracle as go
    with gguf.File(path) as f:
        meta_end = f.data_section_offset
    buf = np.zeros(os.path.getsize(path), np.uint8)
    with open(path, "rb") as fh:
        buf[:meta_end] = np.frombuffer(fh.read(meta_end), np.uint8)
    ref = ob.ref()
    t_ref, t_lib = [], []
    for _ in range(repeats):
        t0 = time.perf_counter()
        err = ref.f("gguf_parse")(buf.ctypes.data, buf.size, None, None, None) if ref is not None else go.parse(buf.data)[0]
        t_ref.append(time.perf_counter() - t0)
        assert err == 0, err
        h = C.c_void_p()
        t0 = time.perf_counter()
        err = eb.lib().emelb_gguf_open_image(buf.ctypes.data, buf.size, C.byref(h))
        t_lib.append(time.perf_counter() - t0)
        assert err == 0, err
        eb.lib().emelb_gguf_close(h)
    return float(np.median(t_ref) * 1e6), float(np.median(t_lib) * 1e6), ("reference" if ref is not None else "port")


def run_load(args):
    import torch
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import gguf
    rank, world, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    be = eb.Backend(local)
    sp = load_spec(args)
    d = load_dir()
    path = os.path.join(d, f"bench_{rank}.gguf")
    try:
        file_bytes = write_load_file(sp, path)
        steps, warmup = min(args.steps, 8), args.warmup

        def one_load(mode):
            """mode: None = the default route (one pipelined pass over the file); "each" = the same route, one
            call per tensor; "plain" / "register" = the alternative routes of the library, whole file."""
            assert be.set_upload_route(mode if mode in ("plain", "register") else "ring")
            t0 = time.perf_counter()
            f = gguf.File(path)
            t1 = time.perf_counter()
            n = f.requirements.tensor_count
            lib, h, bh = eb.lib(), f.handle, be.handle
            if mode == "each":
                for i in range(n):
                    err = lib.emelb_gguf_upload(bh, h, i, 100000 + i, None)
                    assert err == 0, (i, err)
            else:
                err = lib.emelb_gguf_upload_all(bh, h, 100000)
                assert err == 0, err
            be.sync()
            t2 = time.perf_counter()
            return f, n, t1 - t0, t2 - t0

        def unload(f, n, check=False):
            if check:      # bytes in HBM == bytes in the file, for three tensors
                for i in (0, n // 2, n - 1):
                    rec = f.tensor(i)
                    st = be.state(100000 + i)
                    got = np.empty(rec["data_size"], np.uint8)
                    assert be.to_host(got, st.buffer, rec["data_size"])
                    want = np.ctypeslib.as_array((C.c_uint8 * rec["data_size"]).from_address(rec["data"]))
                    assert np.array_equal(got, want), f"tensor {i} differs after upload"
            for i in range(n):
                be.evict(100000 + i)
            f.close()

        import ctypes as C
        results = {}
        with ClockSampler(local) as clocks:
            for mode in (None, "each", "plain", "register"):
                for _ in range(warmup if mode is None else 1):
                    f, n, _p, _t = one_load(mode)
                    unload(f, n)
                barrier(world)
                parse_s, total_s = [], []
                for k in range(steps if mode is None else min(steps, 3)):
                    f, n, p, t = one_load(mode)
                    parse_s.append(p)
                    total_s.append(t)
                    unload(f, n, check=(k == 0))
                results[{None: "staged", "each": "staged_per_tensor"}.get(mode, mode)] = (float(np.mean(total_s)), float(np.median(parse_s)))
            assert be.set_upload_route("ring")
        sec = max_over_ranks(results["staged"][0], world, f"cuda:{local}")
        if rank != 0:
            return
        gbs = file_bytes * world / sec / 1e9
        ref_us, lib_us, kind = reference_parse_us(path)
        peaks, peak_kind = measured_peaks()
        peak = float(peaks["hbm_gbs"])
        line = {"metric": "GGUF file to HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "u8", "data": "synthetic",
                "config": {"workload": sp["name"], "file_bytes": file_bytes, "tensors": n, "file_dir": os.path.dirname(path),
                           "timer": "host wall clock around the synchronous open + upload calls (page cache warm)",
                           "open_file_us": results["staged"][1] * 1e6, "parse_us": lib_us,
                           "routes_gbs": {k: file_bytes / v[0] / 1e9 for k, v in results.items()},
                           "upload_threads": min(16, os.cpu_count() or 1)},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": file_bytes, "d2h_bytes_per_step": 0},
                "gpu_launches": 0,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                             "note": f"copy-engine transfers only, no kernel: bounded by the host link, not by HBM ({peak_kind} HBM peak shown)"},
                "cpu_baseline": {"value": ref_us, "unit": "us per probe + parse of the same metadata", "cores": 1, "kind": kind,
                                 "sample": "median of 5 parses; the reference maps the file and does not copy tensor data"},
                "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    finally:
        be.close()
        try:
            os.unlink(path)
            os.rmdir(d)
        except OSError:
            pass


def run_reference_load(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sp = load_spec(args)
    d = load_dir()
    path = os.path.join(d, "bench_ref.gguf")
    try:
        write_load_file(sp, path)
        us, _lib_us, kind = reference_parse_us(path, repeats=max(3, min(args.steps, 9)))
        line = {"impl": "reference", "metric": "GGUF probe + parse us", "value": us, "unit": "us", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
                "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": {"workload": sp["name"]},
                "cpu_baseline": {"value": us, "unit": "us", "cores": 1, "kind": kind, "sample": "probe + parse of the file's metadata"},
                "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
    finally:
        try:
            os.unlink(path)
            os.rmdir(d)
        except OSError:
            pass


# ------------------------------------------------------------------ decode workload (configurations 3 and 5)
DECODE_SHAPES = {
    "decode_8b": dict(n_layer=32, n_embd=4096, n_head=32, n_head_kv=8, head_dim=128, n_ff=14336, n_vocab=128256,
                      prompt=4096, name="cfg3: Llama-8B shape, Q4_K attn/FFN + Q6_K output, greedy decode after a 4096-token prompt, f16 KV"),
    "decode_70b": dict(n_layer=80, n_embd=8192, n_head=64, n_head_kv=8, head_dim=128, n_ff=28672, n_vocab=128256,
                       prompt=8192 - 160, name="cfg5: Llama-70B shape, Q4_K weights, batch-1 decode at context 8192, f16 KV"),
}


MIX_Q6_K = False   # set by --mix


def decode_tensors(sh, out_type):
    """(layer, role, K, M, type) of every matrix, in the roles of include/emelb_llama.h."""
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import llama as el
    qd, kvd = sh["n_head"] * sh["head_dim"], sh["n_head_kv"] * sh["head_dim"]
    per_layer = [(el.ATTN_Q, sh["n_embd"], qd), (el.ATTN_K, sh["n_embd"], kvd), (el.ATTN_V, sh["n_embd"], kvd),
                 (el.ATTN_OUT, qd, sh["n_embd"]), (el.FFN_GATE, sh["n_embd"], sh["n_ff"]), (el.FFN_UP, sh["n_embd"], sh["n_ff"]),
                 (el.FFN_DOWN, sh["n_ff"], sh["n_embd"])]
    out = [(-1, el.TOKEN_EMBD, sh["n_embd"], sh["n_vocab"], eb.Q4_K), (-1, el.OUTPUT, sh["n_embd"], sh["n_vocab"], out_type)]
    for l in range(sh["n_layer"]):
        # --mix: the value and down projections of every other layer are Q6_K, as quantization mixes of the Q4_K_M
        # kind have them
        out += [(l, role, k, m, eb.Q6_K if MIX_Q6_K and l % 2 == 0 and role in (el.ATTN_V, el.FFN_DOWN) else eb.Q4_K)
                for role, k, m in per_layer]
    return out


def build_decode_session(be, sh, out_type, n_ctx, rank, G, dist=None, seed0=5000, peer=True):
    """A decoder session of shape `sh` with synthetic weights (N(0, 0.02) encoded on the device, norm
    weights 1.0).  G > 1: this rank's row interval of every matrix, the joins over peer stores."""
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import llama as el
    cfg = el.config(sh["n_layer"], sh["n_embd"], sh["n_head"], sh["n_head_kv"], sh["head_dim"], sh["n_ff"], sh["n_vocab"], n_ctx,
                    shard_rank=rank if G > 1 else 0, shard_count=G)
    sess = el.Session(be, cfg)
    peer_joins = False
    if G > 1 and peer:
        handles = [None] * G
        dist.all_gather_object(handles, sess.exchange_export())
        assert sess.exchange_attach(handles), sess.last_error
        dist.barrier()          # every rank has mapped its peers before anybody's first join
        peer_joins = True
    info = dict(weight_bytes=0, q4k_bytes=0, q4k_ops=[], peer_joins=peer_joins, allocs=[], tensors=[], norm_ones=None)
    r = rank if G > 1 else 0
    for i, (layer, role, k, m, t) in enumerate(decode_tensors(sh, out_type)):
        row0 = 0
        if role != el.TOKEN_EMBD:
            row0, m = el.shard_rows(m, r, G)     # this rank's rows of the same seeded matrix
        nbytes = m * eb.row_bytes(t, k)
        d = be.alloc(nbytes)
        info["allocs"].append(d)
        assert be.synth_fill(d, t, m * k, seed0 + i, 0.02, row0 * k), be.last_error
        assert sess.bind_matrix(layer, role, d, t), sess.last_error
        info["tensors"].append((layer, role, d, t, nbytes))
        if role != el.TOKEN_EMBD:
            info["weight_bytes"] += nbytes
            if t == eb.Q4_K and layer >= 0:
                info["q4k_bytes"] += nbytes
                info["q4k_ops"].append((layer, role, d, t, k, m))
    ones = be.alloc(4 * sh["n_embd"])
    info["allocs"].append(ones)
    info["norm_ones"] = ones
    assert be.to_device(ones, np.ones(sh["n_embd"], np.float32))
    assert sess.bind_norm(-1, el.OUTPUT_NORM, ones)
    for l in range(sh["n_layer"]):
        assert sess.bind_norm(l, el.ATTN_NORM, ones) and sess.bind_norm(l, el.FFN_NORM, ones)
    assert be.sync()
    return sess, info


def release_decode_session(be, sess, info, world):
    barrier(world)              # no rank unmaps an exchange arena while a peer may still store into it
    sess.exchange_detach()
    barrier(world)              # ... nor frees one that a peer still maps
    sess.close()
    for d in info["allocs"]:
        be.free(d)


def time_cfg1_matvec(be, timed_region, copies=68):
    """Configuration 1 inside the decode run: the 4096 x 4096 Q4_K mat-vec over `copies` distinct weight copies
    (640 MB > L2), activations already quantized, one CUDA-graph replay per pass.  -> (us per launch, bytes)."""
    import emel_cpp_b200 as eb
    k = m = 4096
    wbytes = m * eb.row_bytes(eb.Q4_K, k)
    w = be.alloc(copies * wbytes)
    for c in range(copies):
        assert be.synth_fill(w + c * wbytes, eb.Q4_K, m * k, 900 + c, 0.02, 0)
    x, y = be.alloc(4 * k), be.alloc(4 * m)
    assert be.synth_fill(x, eb.F32, k, 11, 1.0, 0) and be.sync()
    ops = [eb.mul_mat_op(w + c * wbytes, eb.Q4_K, k, m, x, 1, y) for c in range(copies)]
    assert be.prepare_rhs(eb.dense_view(x, eb.F32, [1, k]), eb.Q4_K)
    for op in ops[:4]:
        assert be.mul_mat_prepared(op)
    be.sync()
    assert be.graph_begin()
    for op in ops:
        assert be.mul_mat_prepared(op)
    g = be.graph_end()
    for _ in range(3):
        be.graph_launch(g)
    ms, _ = timed_region(lambda: [be.graph_launch(g) for _ in range(5)])
    be.graph_destroy(g)
    for d in (w, x, y):
        be.free(d)
    return ms * 1e3 / (5 * copies), wbytes + 4672 + 4 * m


def run_decode_batch(args):
    """--batch B > 1: B sequences decoded together (BASELINE configuration 5's batch-16 decode, or the 8B shape).
    Every sequence gets its own random prompt of the configured length; a step = one token for each sequence."""
    import torch
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import llama as el

    rank, world, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sh = DECODE_SHAPES[args.workload]
    out_type = eb.Q6_K if args.workload == "decode_8b" else eb.Q4_K
    steps, warmup, B = args.steps, args.warmup, args.batch
    prompt_len = sh["prompt"] if args.prompt is None else args.prompt
    n_ctx = ((prompt_len + warmup + steps + 15) // 16) * 16
    be = eb.Backend(local)
    stream = torch.cuda.ExternalStream(be.stream(), device=dev)
    shard = world > 1
    dist = None
    if shard:
        import torch.distributed as dist
        box = [eb.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        assert be.comm_init(rank, world, box[0]), be.last_error
    G, r = (world, rank) if shard else (1, 0)
    sess, info = build_decode_session(be, sh, out_type, n_ctx, r, G, dist, peer=False)
    assert sess.set_sequences(B), sess.last_error
    rng = np.random.Generator(np.random.PCG64(42))
    t0 = time.perf_counter()
    first, pos = [], []
    for j in range(B):
        prompt = rng.integers(0, sh["n_vocab"], size=prompt_len, dtype=np.int32)
        assert sess.select_sequence(j)
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        first.append(int(prompt[-1]))
        pos.append(prompt_len - 1)
    prefill_s = time.perf_counter() - t0

    def timed_region(fn):
        be.sync()
        barrier(world)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        out = fn()
        e1.record(stream)
        be.sync()
        torch.cuda.synchronize()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world, dev), out

    with ClockSampler(local) as clk:
        w_ids = sess.generate_batch(first, pos, warmup)
        ms, ids = timed_region(lambda: sess.generate_batch(w_ids[-1], [p + warmup for p in pos], steps))
        launches = sess.batch_launches_per_step()
        # end to end: one C-ABI call per step, B token ids in, B next ids out (host round trip every step)
        d0 = be.diagnostics()

        def loop():
            t, o = list(w_ids[-1]), []
            for i in range(steps):
                t = list(sess.decode_batch(t, [p + warmup + i for p in pos]))
                o.append(t)
            return o
        ms_e, ids_e = timed_region(loop)
        d1 = be.diagnostics()
        assert [list(x) for x in ids] == ids_e, "device-fed and host-fed batch loops disagree"
        # the same sequences one at a time, for the ratio
        assert sess.select_sequence(0)
        w1 = sess.generate(first[0], pos[0], warmup)
        ms1, ids1 = timed_region(lambda: sess.generate(int(w1[-1]), pos[0] + warmup, min(steps, 32)))
        assert list(ids1) == [int(x[0]) for x in ids[:len(ids1)]], "sequence 0 decodes differently alone"
    clocks = clk.summary()
    tok_s = steps * B / (ms * 1e-3)
    kv_bytes_per_pos = sh["n_layer"] * 2 * sh["n_head_kv"] * sh["head_dim"] * 2
    ctx_mid = prompt_len + warmup + steps // 2
    bytes_per_step = info["weight_bytes"] * (world if shard else 1) + kv_bytes_per_pos * ctx_mid * B
    peaks, peak_kind = measured_peaks()
    gbs = bytes_per_step / (ms / steps * 1e-3) / 1e9 / (world if shard else 1)
    line = {
        "metric": "decode tok/s", "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 5), "higher_is_better": True, "scaling": "strong" if shard else "weak", "vs_baseline": None,
        "dtype": "int8 dot (mma.sync / dp4a) + f32 scales; f16 KV", "data": "synthetic",
        "config": {"workload": sh["name"].replace("batch-1", f"batch-{B}"), "batch": B, "prompt_tokens": prompt_len, "decoded_tokens_per_sequence": steps,
                   "n_ctx": n_ctx, "launch": "one CUDA-graph replay per step; the next token ids are fed back on the device",
                   "l2_policy": f"inputs larger than L2: {bytes_per_step / 1e9:.2f} GB of weights and KV rows read per step",
                   "parallelism": "single GPU" if world == 1 else f"matrices row-sharded over {world} GPUs, NCCL all-gather joins of the batch tensors",
                   "kernel_launches_per_step": launches, "prefill_s": round(prefill_s, 2)},
        "hbm_gbs_effective": round(gbs, 1),
        "e2e": {"value": round(steps * B / (ms_e * 1e-3), 2), "unit": "tok/s", "h2d_bytes_per_step": 8 * B,
                "d2h_bytes_per_step": (d1["d2h_bytes"] - d0["d2h_bytes"]) // steps},
        "gpu_launches": launches * steps,
        "roofline": {"bound": "hbm", "kernel": "whole step (weights once + every sequence's KV rows)", "achieved": round(gbs, 2),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4), "peak_source": f"of {peak_kind}",
                     "algorithmic_bytes_per_step": int(bytes_per_step), "traffic": None},
        "one_sequence_alone": {"tok_s": round(len(ids1) / (ms1 * 1e-3), 2), "same_tokens": True},
        "cpu_baseline": None, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    release_decode_session(be, sess, info, world)


def run_decode_streamed(args):
    """--layer-window S: the decode workload with the layers' matrices kept in page-locked host memory and streamed
    through a window of S layer slots in HBM (include/emelb_window.h) -- the arrangement for a model whose layers do
    not fit the HBM left for weights.  The resident session runs first on the same weights; the streamed session
    must produce the same tokens.  The bound is the host-to-device copy rate, measured here with one plain copy
    of 1 GB from the same page-locked buffer."""
    import torch
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import llama as el
    from emel_cpp_b200 import window as ew

    assert args.gpus == 1, "the layer window is a one-GPU arrangement"
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    sh = DECODE_SHAPES[args.workload]
    out_type = eb.Q6_K if args.workload == "decode_8b" else eb.Q4_K
    slots, depth = args.layer_window, max(1, args.layer_window // 2)
    steps, warmup, B = min(args.steps, 16), 1, max(1, args.batch)
    prompt_len = 512 if args.prompt is None else args.prompt
    n_ctx = ((prompt_len + warmup + steps + 15) // 16) * 16
    be = eb.Backend(0)
    stream = torch.cuda.ExternalStream(be.stream(), device=dev)

    def timed_region(fn):
        be.sync()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        out = fn()
        e1.record(stream)
        be.sync()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    rng = np.random.Generator(np.random.PCG64(42))
    prompts = [rng.integers(0, sh["n_vocab"], size=prompt_len, dtype=np.int32) for _ in range(B)]

    def run(sess):
        """-> prefill ms (sequence 0), decode ms, ids"""
        assert sess.set_sequences(B), sess.last_error
        pre_ms = None
        for j in range(B):
            assert sess.select_sequence(j)
            ms, ok = timed_region(lambda: sess.prefill(prompts[j][:-1], 0))
            assert ok, sess.last_error
            pre_ms = ms if pre_ms is None else pre_ms
        first, pos = [int(p[-1]) for p in prompts], [prompt_len - 1] * B
        if B == 1:
            w = sess.generate(first[0], pos[0], warmup)
            ms, ids = timed_region(lambda: sess.generate(int(w[-1]), pos[0] + warmup, steps))
            return pre_ms, ms, [int(x) for x in w] + [int(x) for x in ids]
        w = sess.generate_batch(first, pos, warmup)
        ms, ids = timed_region(lambda: sess.generate_batch(w[-1], [p + warmup for p in pos], steps))
        return pre_ms, ms, [list(map(int, x)) for x in w] + [list(map(int, x)) for x in ids]

    sess, info = build_decode_session(be, sh, out_type, n_ctx, 0, 1)
    res_pre, res_ms, res_ids = run(sess)
    sess.close()
    # the layers' matrices -> one page-locked host image, packed like a file; their device copies are freed
    layer_tensors = [t for t in info["tensors"] if t[0] >= 0]
    offs, at = {}, 4096
    for layer, role, d, t, nbytes in layer_tensors:
        offs[(layer, role)] = at
        at += (nbytes + 4095) // 4096 * 4096
    image = torch.empty(at, dtype=torch.uint8, pin_memory=True)
    for layer, role, d, t, nbytes in layer_tensors:
        o = offs[(layer, role)]
        assert be.to_host(image[o:o + nbytes].numpy(), d, nbytes)
        be.free(d)
        info["allocs"].remove(d)
    layer_bytes = sum(t[4] for t in layer_tensors)
    layers = [[(l * 16 + role, offs[(l, role)], nbytes) for (layer, role, d, t, nbytes) in layer_tensors if layer == l] for l in range(sh["n_layer"])]
    _o, sizes, cap = ew.plan_layers(layers)
    win = ew.LayerWindow(be)
    assert win.bind(image, layers, slots * cap, slots, depth), win.last_error
    assert win.bound["streaming_active"], "the layers fit the budget: nothing to stream"
    sess = el.Session(be, el.config(sh["n_layer"], sh["n_embd"], sh["n_head"], sh["n_head_kv"], sh["head_dim"], sh["n_ff"], sh["n_vocab"], n_ctx))
    assert sess.set_window(win), sess.last_error
    base = image.data_ptr()
    for layer, role, d, t, nbytes in info["tensors"]:
        assert sess.bind_matrix(layer, role, d if layer < 0 else base + offs[(layer, role)], t), sess.last_error
    assert sess.bind_norm(-1, el.OUTPUT_NORM, info["norm_ones"])
    for l in range(sh["n_layer"]):
        assert sess.bind_norm(l, el.ATTN_NORM, info["norm_ones"]) and sess.bind_norm(l, el.FFN_NORM, info["norm_ones"])
    # the copy rate the stream is bounded by: 1 GB of the same buffer in one copy
    probe_bytes = min(1 << 30, at)
    probe = be.alloc(probe_bytes)
    host_view = image[:probe_bytes].numpy()
    assert be.to_device(probe, host_view)
    copy_ms, ok = timed_region(lambda: be.to_device(probe, host_view))
    assert ok
    be.free(probe)
    h2d_peak = probe_bytes / (copy_ms * 1e-3) / 1e9
    with ClockSampler(0) as clk:
        win_pre, win_ms, win_ids = run(sess)
    assert win_ids == res_ids, "the streamed session decodes differently from the resident one"
    st = win.stats()
    tok_s = steps * B / (win_ms * 1e-3)
    gbs = layer_bytes * steps / (win_ms * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s, layers streamed from host memory", "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(win_ms / steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 dot + f32 scales; f16 KV", "data": "synthetic",
        "config": {"workload": sh["name"].replace("batch-1", f"batch-{B}") + f", layers streamed through {slots} slots", "batch": B,
                   "window_slots": slots, "prefetch_depth": depth, "prompt_tokens": prompt_len, "decoded_tokens_per_sequence": steps,
                   "slot_bytes": cap, "layer_bytes_per_step": layer_bytes, "hbm_for_layers": slots * cap,
                   "source_page_locked": win.bound["source_page_locked"], "launch": "plain launches; copies ordered by events",
                   "l2_policy": f"inputs larger than L2: {layer_bytes / 1e9:.2f} GB cross PCIe and are read per step"},
        "same_tokens_as_resident": True,
        "resident": {"tok_s": round(steps * B / (res_ms * 1e-3), 2), "prefill_tok_s": round((prompt_len - 1) / (res_pre * 1e-3), 1)},
        "prefill_tok_s": round((prompt_len - 1) / (win_pre * 1e-3), 1),
        "roofline": {"bound": "pcie", "kernel": "slot loads (one copy per matrix)", "achieved": round(gbs, 2), "peak": round(h2d_peak, 2),
                     "unit": "GB/s", "frac": round(gbs / h2d_peak, 4), "peak_source": "one 1 GB page-locked copy timed in this run", "traffic": None},
        "window": st, "gpu_launches": sess.launches_per_token() * steps if B == 1 else sess.batch_launches_per_step() * steps,
        "e2e": None, "cpu_baseline": None, "clocks": clk.summary(),
    }
    print(json.dumps(line), flush=True)
    sess.close()
    win.close()
    for d in info["allocs"]:
        be.free(d)


def run_decode(args):
    import torch
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import llama as el

    rank, world, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sh = DECODE_SHAPES[args.workload]
    out_type = eb.Q6_K if args.workload == "decode_8b" else eb.Q4_K
    steps, warmup = args.steps, args.warmup
    prompt_len = sh["prompt"] if args.prompt is None else args.prompt
    n_ctx = ((prompt_len + warmup + steps + 15) // 16) * 16
    be = eb.Backend(local)
    stream = torch.cuda.ExternalStream(be.stream(), device=dev)
    # N > 1: ONE sequence with every matrix row-sharded over the N GPUs (the multi-GPU design of this path);
    # --replicas runs N independent sequences instead
    shard = world > 1 and not args.replicas
    dist = None
    if world > 1:
        import torch.distributed as dist
    if shard:
        box = [eb.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        assert be.comm_init(rank, world, box[0]), be.last_error
    G, r = (world, rank) if shard else (1, 0)
    sess, info = build_decode_session(be, sh, out_type, n_ctx, r, G, dist, peer=args.join == "peer")
    if args.one_kernel:
        assert sess.set_step_mode(1)
    peer_joins, weight_bytes, q4k_bytes, q4k_ops = info["peer_joins"], info["weight_bytes"], info["q4k_bytes"], info["q4k_ops"]

    def timed_region(fn):
        be.sync()
        barrier(world)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        out = fn()
        e1.record(stream)
        be.sync()
        torch.cuda.synchronize()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world, dev), out

    def decode_run(sess, prompt, n_steps, n_warm, host_loop=True):
        """prefill (twice: the first pass also sizes the batch buffers), then the device-fed greedy loop and,
        optionally, the loop with a host round trip per token.  -> dict"""
        pos0 = len(prompt) - 1
        t0 = time.perf_counter()
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        first = time.perf_counter() - t0
        t0 = time.perf_counter()
        assert sess.prefill(prompt[:-1], 0), sess.last_error
        warm = time.perf_counter() - t0
        warm_ids = sess.generate(int(prompt[-1]), pos0, n_warm)
        ms, ids = timed_region(lambda: sess.generate(int(warm_ids[-1]), pos0 + n_warm, n_steps))
        out = dict(ms=ms, ids=list(ids), prefill_s=first, prefill_warm_s=warm, launches=sess.launches_per_token())
        if host_loop:
            # end to end: one C-ABI call per token, token id in, next token id out (host round trip every step)
            d0 = be.diagnostics()
            tok = int(prompt[-1])
            for i in range(n_warm):
                tok = sess.decode(tok, pos0 + i)

            def loop():
                t, o = tok, []
                for i in range(n_steps):
                    t = sess.decode(t, pos0 + n_warm + i)
                    o.append(t)
                return o
            ms_e, ids_e = timed_region(loop)
            d1 = be.diagnostics()
            out.update(ms_e=ms_e, ids_e=list(ids_e), d2h=(d1["d2h_bytes"] - d0["d2h_bytes"]) // (n_steps + n_warm))
        return out

    prompt = np.random.Generator(np.random.PCG64(42 + (0 if shard else rank))).integers(0, sh["n_vocab"], size=prompt_len, dtype=np.int32)
    extras = {}
    with ClockSampler(local) as clk:
        res = decode_run(sess, prompt, steps, warmup)
        assert res["ids"] == res["ids_e"], "device-fed and host-fed greedy loops disagree"
        ms, ms_e = res["ms"], res["ms_e"]
        # the dominant kernel alone: every Q4_K layer matrix of one token, activations already quantized
        x8 = be.alloc(4 * sh["n_ff"])
        assert be.synth_fill(x8, eb.F32, sh["n_ff"], 9, 1.0, 0)
        # launched the way the decode step launches them: Q, K, V of a layer in one launch, gate and up in one
        # launch (emelb_mul_mat_prepared_group), Wo and down on their own
        ybuf = be.alloc(4 * (2 * sh["n_ff"] + 2 * sh["n_embd"]))
        by_k = {}
        per_layer = {}
        for layer, role, d, t, k, m in q4k_ops:
            per_layer.setdefault(layer, {})[role] = (d, t, k, m)
        for layer in sorted(per_layer):
            roles = per_layer[layer]
            for group in ((el.ATTN_Q, el.ATTN_K, el.ATTN_V), (el.ATTN_OUT,), (el.FFN_GATE, el.FFN_UP), (el.FFN_DOWN,)):
                if any(role not in roles for role in group):
                    continue            # --mix: a Q6_K matrix in the group
                ops, off = [], 0
                for role in group:
                    d, t, k, m = roles[role]
                    ops.append(eb.mul_mat_op(d, t, k, m, x8, 1, ybuf + 4 * off))
                    off += m
                by_k.setdefault(roles[group[0]][2], []).append(ops)
        graphs = []

        def run_group(ops):
            assert (be.mul_mat_prepared(ops[0]) if len(ops) == 1 else be.mul_mat_prepared_group(ops)), be.last_error

        for k, groups in by_k.items():
            assert be.prepare_rhs(eb.dense_view(x8, eb.F32, [1, k]), eb.Q4_K)
            for ops in groups[:4]:
                run_group(ops)
            be.sync()
            assert be.graph_begin()
            for ops in groups:
                run_group(ops)
            graphs.append((k, be.graph_end(), len(groups)))
        ms_k, n_k = 0.0, 0
        for k, g, n_ops in graphs:
            assert be.prepare_rhs(eb.dense_view(x8, eb.F32, [1, k]), eb.Q4_K)
            for _ in range(3):
                be.graph_launch(g)
            t_ms, _ = timed_region(lambda: [be.graph_launch(g) for _ in range(5)])
            ms_k += t_ms / 5
            n_k += n_ops
            be.graph_destroy(g)
        # configuration 1, the mat-vec the headline metric is quoted on first
        cfg1_us, cfg1_bytes = time_cfg1_matvec(be, timed_region)
        # the same session through the one-kernel step (every layer of a token in one persistent kernel)
        if not shard and not args.one_kernel and args.workload == "decode_8b":
            assert sess.set_step_mode(1)
            w_ids = sess.generate(int(prompt[-1]), prompt_len - 1, warmup)
            ms1, ids1 = timed_region(lambda: sess.generate(int(w_ids[-1]), prompt_len - 1 + warmup, steps))
            if sess.launches_per_token() < res["launches"]:
                extras["one_kernel_step"] = {"tok_s": round(steps * (1 if shard else world) / (ms1 * 1e-3), 2),
                                             "kernel_launches_per_token": sess.launches_per_token(),
                                             "same_tokens_as_launch_chain": list(ids1) == res["ids"]}
            assert sess.set_step_mode(0)
        if world > 1 and world <= 4 and shard and peer_joins:
            # the same session with the joins inside the neighbouring kernels instead of one join kernel each (run on
            # the rank counts this form has been validated on: 2 and 4)
            assert sess.set_join_fusion(True)
            w_ids = sess.generate(int(prompt[-1]), prompt_len - 1, warmup)
            ms_j, ids_j = timed_region(lambda: sess.generate(int(w_ids[-1]), prompt_len - 1 + warmup, steps))
            extras["joins_in_kernels"] = {"tok_s": round(steps / (ms_j * 1e-3), 2), "kernel_launches_per_token": sess.launches_per_token(),
                                          "same_tokens": list(ids_j) == res["ids"],
                                          "note": "producers push their interval (f32 rows or Q8_K planes) and raise a flag, consumers wait in their prologue"}
            assert sess.set_join_fusion(False)
        if world > 1 and shard:
            # beside the headline: N independent replicas of the same model (no collective), and configuration 5
            # (70B shape) row-sharded over the same N GPUs with a shortened prompt
            release_decode_session(be, sess, info, world)
            sess = None
            s2, i2 = build_decode_session(be, sh, out_type, n_ctx, 0, 1)
            p2 = np.random.Generator(np.random.PCG64(42 + rank)).integers(0, sh["n_vocab"], size=prompt_len, dtype=np.int32)
            r2 = decode_run(s2, p2, min(steps, 32), warmup, host_loop=False)
            extras["replicas"] = {"tok_s": round(min(steps, 32) * world / (r2["ms"] * 1e-3), 2), "sequences": world,
                                  "parallelism": f"{world} independent replicas (one sequence per GPU), no collective"}
            release_decode_session(be, s2, i2, 1)
            sh5 = DECODE_SHAPES["decode_70b"]
            p_len5, st5 = 512, min(steps, 16)
            s5, i5 = build_decode_session(be, sh5, eb.Q4_K, ((p_len5 + warmup + st5 + 15) // 16) * 16, rank, world, dist, seed0=7000)
            p5 = np.random.Generator(np.random.PCG64(45)).integers(0, sh5["n_vocab"], size=p_len5, dtype=np.int32)
            r5 = decode_run(s5, p5, st5, warmup, host_loop=False)
            extras["cfg5_sharded"] = {"tok_s": round(st5 / (r5["ms"] * 1e-3), 2), "workload": sh5["name"], "prompt_tokens": p_len5,
                                      "decoded_tokens": st5, "kernel_launches_per_token": r5["launches"],
                                      "note": "prompt shortened from 8032 to 512 tokens to bound the run"}
            release_decode_session(be, s5, i5, world)
    clocks = clk.summary()

    seqs = 1 if shard else world
    tok_s = steps * seqs / (ms * 1e-3)
    tok_s_e2e = steps * seqs / (ms_e * 1e-3)
    kv_bytes_per_pos = sh["n_layer"] * 2 * sh["n_head_kv"] * sh["head_dim"] * 2
    ctx_mid = prompt_len + warmup + steps // 2
    bytes_per_token = weight_bytes * (world if shard else 1) + kv_bytes_per_pos * ctx_mid
    peaks, peak_kind = measured_peaks()
    kernel_gbs = q4k_bytes / (ms_k * 1e-3) / 1e9
    cfg1_gbs = cfg1_bytes / (cfg1_us * 1e-6) / 1e9
    line = {
        "metric": "decode tok/s", "value": round(tok_s, 2), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 5), "higher_is_better": True, "scaling": "strong" if shard else "weak", "vs_baseline": None,
        "dtype": "int8 dot (dp4a) + f32 scales; f16 KV", "data": "synthetic",
        "config": {"workload": sh["name"] + (" (--mix: attn_v and ffn_down of every other layer Q6_K)" if MIX_Q6_K else ""),
                   "prompt_tokens": prompt_len, "decoded_tokens": steps, "n_ctx": n_ctx,
                   "launch": ("one persistent kernel per token plus the output head" if args.one_kernel else "one CUDA-graph replay per token")
                             + "; the next token id is fed back on the device",
                   "l2_policy": f"inputs larger than L2: {weight_bytes * (world if shard else 1) / 1e9:.2f} GB of weights streamed per token",
                   "parallelism": "single GPU" if world == 1 else (
                       f"one sequence, matrices row-sharded over {world} GPUs, 4 joins of f32 row intervals per layer "
                       f"({'peer stores over NVLink, one kernel per join' if peer_joins else 'NCCL all-gather'}; "
                       "the prompt's batch joins are NCCL all-gathers)" if shard
                       else f"{world} independent replicas (one sequence per GPU), no collective"),
                   "kernel_launches_per_token": res["launches"],
                   "prefill_s": round(res["prefill_s"], 3),
                   "prefill_tok_s": round((prompt_len - 1) / res["prefill_warm_s"], 1),
                   "prefill": "prompt tokens in batches of up to 2048: tcgen05 Q4_K products, mma.sync batch attention"
                              + (", row intervals joined by NCCL all-gather" if shard else "")},
        "hbm_gbs_effective": round(bytes_per_token * tok_s / seqs / 1e9, 1),
        "q4_k_gemv_hbm_gbs": round(kernel_gbs, 1), "pct_of_8tbs_nominal": round(100 * kernel_gbs / NOMINAL_HBM_GBS, 2),
        "e2e": {"value": round(tok_s_e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": res["d2h"]},
        "gpu_launches": res["launches"] * steps,
        "roofline": {"bound": "hbm", "kernel": "gemv_stream_q4_k_n1", "achieved": round(kernel_gbs, 2), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(kernel_gbs / peaks["hbm_gbs"], 4), "peak_source": f"of {peak_kind}",
                     "us_per_launch": round(ms_k * 1e3 / n_k, 3), "algorithmic_bytes_per_launch": q4k_bytes // n_k,
                     "launches_timed": n_k,
                     # ncu capture of the 14336x4096 launch, scaled by bytes (traffic grows with the weight bytes)
                     "traffic": (lambda rr: None if rr is None else int(rr * (q4k_bytes // n_k)))(ncu_traffic("q4_k_n1_traffic_over_algorithmic"))},
        # configuration 1 (the 4096 x 4096 Q4_K mat-vec BASELINE's metric names first), timed in the same run
        "roofline_cfg1": {"bound": "hbm", "kernel": "gemv_stream_q4_k_n1", "workload": "cfg1: Q4_K 4096x4096 mat-vec, 68 weight copies (640 MB > L2)",
                          "achieved": round(cfg1_gbs, 2), "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(cfg1_gbs / peaks["hbm_gbs"], 4),
                          "peak_source": f"of {peak_kind}", "us_per_launch": round(cfg1_us, 3), "algorithmic_bytes_per_launch": cfg1_bytes,
                          "traffic": ncu_traffic("gemv_stream_q4_k_n1")},
        "clocks": clocks,
    }
    line.update(extras)
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline_decode(sh, out_type, budget_s=args.cpu_budget)
        print(json.dumps(line), flush=True)
    if sess is not None:
        release_decode_session(be, sess, info, world)
    be.close()
    if world > 1:
        dist.destroy_process_group()


class CpuDecoder:
    """The reference's CPU kernels driven through one whole decode token of shape `sh`: per layer the seven
    mat-vecs (AVX2/FMA route, row-sliced over `lanes` threads as kernel::matmul does) and the flash attention
    over `ctx` cached tokens (single-threaded, as in the reference), then the output projection.  The weight
    bytes of ONE layer are reused for every layer (random block bytes with sane scales): the kernels' time does
    not depend on the values, and 4.4 GB of distinct host weights would only add set-up time."""

    def __init__(self, sh, out_type, lanes, ctx):
        import emel_cpp_b200 as eb
        from oracle import bindings as ob
        lib = ob.ref()
        self.kind = "reference" if lib is not None else "port"
        self.lib = lib or ob.port()
        self.sh, self.lanes = sh, lanes
        rng = np.random.Generator(np.random.PCG64(1))

        def blocks(t, k, m):
            w = rng.integers(0, 256, size=m * eb.row_bytes(t, k), dtype=np.uint8).reshape(-1, eb.BLOCK_BYTES[t])
            for off in ({eb.Q4_K: (0, 2), eb.Q6_K: (208,)}[t]):
                w[:, off + 1] = rng.integers(0x18, 0x30, size=w.shape[0])
            return w.reshape(-1)

        qd, kvd = sh["n_head"] * sh["head_dim"], sh["n_head_kv"] * sh["head_dim"]
        mats = [(sh["n_embd"], qd), (sh["n_embd"], kvd), (sh["n_embd"], kvd), (qd, sh["n_embd"]),
                (sh["n_embd"], sh["n_ff"]), (sh["n_embd"], sh["n_ff"]), (sh["n_ff"], sh["n_embd"])]
        self.keep, self.layer_ops = [], []
        for k, m in mats:
            w, x, y = blocks(eb.Q4_K, k, m), rng.standard_normal(k, dtype=np.float32), np.zeros(m, np.float32)
            self.keep += [w, x, y]
            self.layer_ops.append(ob.mul_mat_op(w, eb.Q4_K, k, m, x, 1, y))
        w, x, y = blocks(out_type, sh["n_embd"], sh["n_vocab"]), rng.standard_normal(sh["n_embd"], dtype=np.float32), np.zeros(sh["n_vocab"], np.float32)
        self.keep += [w, x, y]
        self.head_op = ob.mul_mat_op(w, out_type, sh["n_embd"], sh["n_vocab"], x, 1, y)
        hd, T = sh["head_dim"], ctx
        q = rng.standard_normal((sh["n_head"], hd), dtype=np.float32)
        kc = (rng.standard_normal((sh["n_head_kv"], T, hd), dtype=np.float32) * 0.5).astype(np.float16).view(np.uint16)
        vc = rng.standard_normal((sh["n_head_kv"], T, hd), dtype=np.float32).astype(np.float16).view(np.uint16)
        dst = np.zeros((sh["n_head"], hd), np.float32)
        self.keep += [q, kc, vc, dst]
        self.fop = ob.flash_op(q, kc, vc, dst, hd, sh["n_head"], sh["n_head_kv"], T, T, scale=float(hd) ** -0.5, masked_total=T)
        self.kw = {"route": "avx2", "lanes": lanes} if self.kind == "reference" else {}
        self.fkw = {"route": "avx2"} if self.kind == "reference" else {}

    def layer(self):
        for op in self.layer_ops:
            assert self.lib.mul_mat(op, **self.kw)
        assert self.lib.flash_attn(self.fop, **self.fkw)

    def token(self):
        for _ in range(self.sh["n_layer"]):
            self.layer()
        assert self.lib.mul_mat(self.head_op, **self.kw)


def cpu_baseline_decode(sh, out_type, budget_s=8.0):
    """Beside the GPU number: the reference's CPU kernels on this host, min(8, cores) lanes (the reference's own
    maximum lane count, src/emel/kernel/matmul/guards.hpp:12-14), timed on a bounded sample."""
    lanes = min(8, os.cpu_count() or 1)
    dec = CpuDecoder(sh, out_type, lanes, sh["prompt"])
    dec.layer()
    t0 = time.perf_counter()
    dec.layer()
    one = time.perf_counter() - t0
    reps = int(max(1, min(sh["n_layer"], budget_s / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        dec.layer()
    t_layer = (time.perf_counter() - t0) / reps
    t0 = time.perf_counter()
    assert dec.lib.mul_mat(dec.head_op, **dec.kw)
    t_head = time.perf_counter() - t0
    sec = sh["n_layer"] * t_layer + t_head
    # the serial route beside it: one kernel actor, one core (two layers and the head's share, scaled)
    one_core = None
    if dec.kind == "reference" and lanes > 1:
        d1 = CpuDecoder(sh, out_type, 1, sh["prompt"])
        d1.layer()
        t0 = time.perf_counter()
        d1.layer()
        t1 = time.perf_counter() - t0
        one_core = {"value": round(1.0 / (sh["n_layer"] * t1 + t_head * lanes), 4), "unit": "tok/s", "cores": 1,
                    "sample": "one layer on one thread x the layer count + the output projection's 8-lane time x 8"}
    return {"value": round(1.0 / sec, 4), "unit": "tok/s", "cores": lanes if dec.kind == "reference" else 1, "kind": dec.kind,
            "one_core": one_core,
            "sample": f"mean of {reps} layers (7 mat-vecs + attention over {sh['prompt']} tokens each) x {sh['n_layer']} layers + one "
                      f"output projection; AVX2/FMA route, mat-vecs row-sliced over {lanes} threads, attention single-threaded "
                      "as in the reference"}


def run_reference_decode(args):
    """--impl reference: every step is one whole decode token on the host cores (CpuDecoder), measured, not scaled."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    sh = DECODE_SHAPES[args.workload]
    import emel_cpp_b200 as eb
    out_type = eb.Q6_K if args.workload == "decode_8b" else eb.Q4_K
    lanes = min(8, os.cpu_count() or 1)
    ctx = sh["prompt"] if args.prompt is None else args.prompt
    dec = CpuDecoder(sh, out_type, lanes, ctx)
    for _ in range(args.warmup):
        dec.token()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        dec.token()
    dt = time.perf_counter() - t0
    v = round(args.steps / dt, 4)
    n_ctx = ((ctx + args.warmup + args.steps + 15) // 16) * 16
    line = {"impl": "reference", "metric": "decode tok/s", "value": v, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot (AVX2 maddubs) + f32 scales; f16 KV", "data": "synthetic",
            "config": {"workload": sh["name"], "prompt_tokens": ctx, "decoded_tokens": args.steps, "n_ctx": n_ctx,
                       "launch": "one whole token per step on the host: 7 mat-vecs + attention per layer, then the output projection",
                       "l2_policy": "one layer's weight bytes reused for every layer (compute-bound kernels)",
                       "parallelism": f"{lanes} host threads (the reference's maximum lane count), attention single-threaded",
                       "kernel_launches_per_token": 0, "prefill_s": None, "prefill_tok_s": None, "prefill": "not run: the KV cache holds random rows"},
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": lanes if dec.kind == "reference" else 1, "kind": dec.kind,
                             "sample": f"{args.steps} whole tokens after {args.warmup} warm-up tokens, attention over {ctx} cached tokens"},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_8b", choices=["decode_8b", "decode_70b", "gemv_q4_k", "gemv_q8_0", "prefill_q4_k", "load_gguf"])
    ap.add_argument("--layers", type=int, default=16, help="load_gguf: layers in the synthetic file (122.7 MB each)")
    ap.add_argument("--prompt", type=int, default=None, help="prompt length override for the decode workloads")
    ap.add_argument("--ncols", type=int, default=1)
    ap.add_argument("--rows", type=int, default=None, help="row count override for gemv_q4_k")
    ap.add_argument("--cols", type=int, default=None, help="column count override for gemv_q4_k")
    ap.add_argument("--cpu-budget", type=float, default=8.0)
    ap.add_argument("--replicas", action="store_true",
                    help="decode workloads at --gpus N > 1: N independent sequences (one per GPU, no collective) instead of "
                         "ONE sequence with every matrix row-sharded over the N GPUs")
    ap.add_argument("--shard", action="store_true", help="accepted for compatibility: sharding is what --gpus N > 1 does")
    ap.add_argument("--join", default="peer", choices=["peer", "nccl"],
                    help="sharded decode: join the ranks' row intervals by peer stores over NVLink (default) or by NCCL all-gathers")
    ap.add_argument("--batch", type=int, default=1, help="decode workloads: sequences decoded together (one token each per step)")
    ap.add_argument("--layer-window", type=int, default=0,
                    help="decode workloads, one GPU: keep the layers' matrices in page-locked host memory and stream them "
                         "through a window of this many layer slots in HBM (2-8); prints its own line")
    ap.add_argument("--one-kernel", action="store_true",
                    help="decode workloads: run the headline through the one-kernel step (every layer of a token in one "
                         "persistent kernel) instead of the launch chain")
    ap.add_argument("--mix", action="store_true",
                    help="decode workloads: attn_v and ffn_down of every other layer as Q6_K instead of Q4_K")
    args = ap.parse_args()
    global MIX_Q6_K
    MIX_Q6_K = args.mix
    args.warmup = max(3, args.warmup)
    decode = args.workload.startswith("decode")
    if args.workload == "prefill_q4_k":
        (run_reference_prefill if args.impl == "reference" else run_prefill)(args)
    elif args.workload == "load_gguf":
        (run_reference_load if args.impl == "reference" else run_load)(args)
    elif args.impl == "reference":
        (run_reference_decode if decode else run_reference_gemv)(args)
    elif decode and args.layer_window > 0:
        run_decode_streamed(args)
    else:
        (run_decode_batch if decode and args.batch > 1 else run_decode if decode else run_gemv)(args)


if __name__ == "__main__":
    main()
