"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Headline: the int4 group-quantized decode GEMV of the benchmark's second configuration (W u4 [14336, 4096], group
128, bf16 scales, x bf16 [M=1, 4096]), reported as achieved HBM GB/s = algorithmic bytes / device time. A STEP is
eight passes over 8 resident copies of the weights (64 GEMV launches, captured in one CUDA graph): the copies hold
242 MB > the 126 MB L2, so every launch streams its weights from HBM. W warm-up steps, then exactly K timed steps, CUDA events on the launching
stream, max over ranks.

For N > 1 the linear is sharded column-parallel: every rank owns a [14336, 4096] shard of a 14336*N-row linear (weak
scaling) and each launch's bf16 outputs are all-gathered by the launch itself: the reduction that produces an output
stores it into every rank's gather buffer (peer stores over NVLink, bounded completion checks), verified once against
NCCL's all-gather before timing. The same run also measures, at every N, the two sharded configurations of the path and
prints them under `secondary`: the expert-parallel MoE FFN layer (config 4, 4096 tokens in total, strong scaling) and
the column-parallel int8 linear (config 5, N sharded over the ranks, peer-store gather of the int32 outputs).

`--impl reference` times the reference bench's CPU loop (oracle/cpu_baseline.cpp) on all host cores over the same
workload: a step is the same 64 GEMVs.
"""
from __future__ import annotations

import argparse
import ctypes as C
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

N_OUT, K_IN, GROUP = 14336, 4096, 128
COPIES = 8
PASSES = 8                # a step runs the GEMV over every weight copy this many times: 64 launches in one graph
LAUNCHES = COPIES * PASSES
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
METRIC = "int4_decode_gemv_hbm_gbs"


def workload_name(m: int) -> str:
    return f"int4 group-quantized decode GEMV M={m} N={N_OUT} K={K_IN} g={GROUP} (config 2), step = {LAUNCHES} launches over {COPIES} rotating weight copies"


def algorithmic_bytes(m: int, n: int = N_OUT, k: int = K_IN, group: int = GROUP) -> int:
    """Packed weights + bf16 scales + bf16 x + bf16 y, each touched once."""
    return n * k // 2 + n * (k // group) * 2 + m * k * 2 + m * n * 2


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "kind": "measured"}
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def cpu_model() -> str:
    try:
        with open("/proc/cpuinfo") as fh:
            for line in fh:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def summary(self, lo: int = 0, hi: int | None = None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        rows = self.rows[lo:hi] or self.rows[-3:]
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is not None:
            time.sleep(0.12)
            self.proc.terminate()


# ---------------------------------------------------------------------------------------------------------------------
# CPU arm: the reference bench's own loop on the host cores
# ---------------------------------------------------------------------------------------------------------------------
def cpu_step_inputs(m: int):
    import numpy as np

    from vyre_b200 import synth

    x, w, s = synth.int4_linear_inputs(m, N_OUT, K_IN, seed=0)
    return synth.bf16_bits_to_f32(x).reshape(m, K_IN).astype(np.float32), w, s


def cpu_gemv_times(m: int, samples: int, warmup: int = 1):
    """Seconds per GEMV of the reference's CPU loop over the full [14336, 4096] weights, one value per sample."""
    import oracle

    xf, w, s = cpu_step_inputs(m)
    for _ in range(warmup):
        oracle.cpu_baseline_int4_gemv(xf, w, s, m, N_OUT, K_IN)
    out = []
    for _ in range(samples):
        t0 = time.perf_counter()
        oracle.cpu_baseline_int4_gemv(xf, w, s, m, N_OUT, K_IN)
        out.append(time.perf_counter() - t0)
    return out, oracle.num_threads()


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    m = args.m
    # a step is what the native arm's step is: COPIES GEMVs over the full weights (the CPU has no L2 to defeat, the same
    # weights serve every pass)
    per_gemv, threads = cpu_gemv_times(m, samples=(args.steps + args.warmup) * LAUNCHES, warmup=1)
    timed = per_gemv[args.warmup * LAUNCHES:]
    step_s = sum(timed) / max(1, args.steps)
    gbs = LAUNCHES * algorithmic_bytes(m) / step_s / 1e9
    sample = (f"{args.steps} steps x {LAUNCHES} full GEMVs (rows [0,{N_OUT}) x K={K_IN}) of the reference bench's f32 loop "
              f"(vyre-bench/src/cases/quantized_linear.rs:447-463 restated for the row-major layout), -O3, OpenMP over rows")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16xint4->f32", "data": "synthetic",
        "config": {"workload": workload_name(m)},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample,
                         "cpu_model": cpu_model(), "ms_per_gemv_median": round(statistics.median(timed) * 1e3, 3)},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
FP32_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12  # 74.4

def event_time_us(fn, reps: int, warm: int, stream=None):
    """Average device time of fn() in microseconds over `reps` calls after `warm` untimed ones (CUDA events on the stream)."""
    import torch

    stream = stream or torch.cuda.current_stream()
    with torch.cuda.stream(stream):
        for _ in range(warm):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
    stream.synchronize()
    return a.elapsed_time(b) * 1e3 / max(1, reps)


def tensor_peak(int8: bool) -> float:
    """Measured tensor-pipe peak of this GPU in T(FL)OP/s: tcgen05.mma from shared-memory operands only."""
    import torch

    from vyre_b200 import ffi

    L = ffi.lib()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops = C.c_double(0.0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def launch():
        ffi.check(L.vyb_k_tensor_peak(1 if int8 else 0, 4096, stream, C.c_void_p(status.data_ptr()), C.byref(ops)))

    us = event_time_us(launch, reps=5, warm=2)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    return ops.value / (us * 1e-6) / 1e12


def measure_prefill(shape, steps: int, warmup: int, peaks: dict, check: bool = True) -> dict:
    """Config 3: int4 prefill GEMM on tcgen05 (kernel-level launches), with a tile checked against torch in f32."""
    import torch

    from vyre_b200 import ffi

    L = ffi.lib()
    m, n, k = shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
    s = (torch.rand((n, k // GROUP), device="cuda") * 0.019 + 0.001).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

    def launch():
        ffi.check(L.vyb_k_int4_prefill_gemm(x.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(), m, n, k, GROUP,
                                            ffi.DT_BF16, stream, C.c_void_p(status.data_ptr())))

    us = event_time_us(launch, steps, warmup)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    tflops = 2.0 * m * n * k / (us * 1e-6) / 1e12
    out = {"tflops": round(tflops, 1), "us_per_launch": round(us, 1),
           "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": round(tflops / peaks["bf16_tflops"], 4), "peak_kind": f"cuBLAS bf16 burst, of {peaks['kind']}",
                        "frac_of_sustained": round(tflops / peaks["bf16_tflops_sustained"], 4),
                        "kernel": "int4_gemm_pair_kernel", "us_per_launch": round(us, 1), "algorithmic_flops_per_launch": 2 * m * n * k}}
    if check:
        rows, cols = min(m, 128), min(n, 256)
        lo, hi = (w[:cols] & 0xF).float() - 8.0, (w[:cols] >> 4).float() - 8.0
        wq = torch.stack([lo, hi], dim=2).reshape(cols, k)
        wd = (wq * s[:cols].float().repeat_interleave(GROUP, dim=1)).to(torch.bfloat16).float()  # the tile the tensor core sees
        want = x[:rows].float() @ wd.T
        got = y[:rows, :cols].float()
        err = float(((got - want).abs() / want.abs().clamp_min(1e-2 * want.pow(2).mean().sqrt())).max())
        out["parity_tile"] = {"rows": rows, "cols": cols, "max_rel_err_vs_torch_f32": round(err, 5), "ok": err <= 1e-2}
        assert err <= 1e-2, f"prefill GEMM tile disagrees with torch: {err}"
    return out


def measure_int8(shape, steps: int, warmup: int, i8_peak: float, peaks: dict) -> dict:
    """Config 5 on one GPU: int8 x int8 -> int32 GEMM on tcgen05, a tile checked exactly."""
    import torch

    from vyre_b200 import ffi

    L = ffi.lib()
    m, n, k = shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda")
    y = torch.empty((m, n), dtype=torch.int32, device="cuda")

    def launch():
        ffi.check(L.vyb_k_int8_gemm_i32(a.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, stream, C.c_void_p(status.data_ptr())))

    us = event_time_us(launch, steps, warmup)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    tops = 2.0 * m * n * k / (us * 1e-6) / 1e12
    want = (a[:64].double() @ w[:128].double().T).to(torch.int64)  # exact: sums far below 2^53
    exact = bool(torch.equal(y[:64, :128].to(torch.int64), want))
    assert exact, "int8 GEMM tile is not bit-exact"
    return {"tops": round(tops, 1), "us_per_launch": round(us, 1), "parity_tile": {"rows": 64, "cols": 128, "bit_exact_vs_f64": exact},
            "roofline": {"bound": "tensor", "achieved": round(tops, 1), "peak": round(i8_peak, 1), "unit": "TOP/s",
                         "frac": round(tops / i8_peak, 4), "peak_kind": "tcgen05 kind::i8 from shared-memory operands, measured in this run",
                         "frac_of_2x_bf16_burst": round(tops / (2 * peaks["bf16_tflops"]), 4), "kernel": "int8_gemm_pair_kernel",
                         "us_per_launch": round(us, 1), "algorithmic_ops_per_launch": 2 * m * n * k}}


def measure_int8_weight_only(peaks: dict, reps: int = 200) -> dict:
    """Config 1 (the reference-runnable case): f32 activations [16, 1024], int8 weights [1024, 1024] with per-channel f32
    scales, dequantised on the fly. 1 MB of weights: a latency-sized launch, timed back to back over 16 rotating weight copies
    and checked in full against torch f32 on the device."""
    import numpy as np
    import torch

    from vyre_b200 import ffi, synth

    L = ffi.lib()
    m, n, k = 16, 1024, 1024
    x_np, w_np, s_np = synth.int8_weight_only_inputs(m, n, k, seed=0)
    x, sc = torch.from_numpy(x_np).cuda(), torch.from_numpy(s_np).cuda()
    ws = [torch.from_numpy(np.roll(w_np, c, axis=0)).cuda() for c in range(16)]
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    it = [0]

    def launch():
        c = it[0] % len(ws)
        it[0] += 1
        ffi.check(L.vyb_k_int8_weight_only_linear(x.data_ptr(), ws[c].data_ptr(), sc.data_ptr(), y.data_ptr(), m, n, k, stream))

    us = event_time_us(launch, reps, 20)
    it[0] = 0
    launch()
    torch.cuda.synchronize()
    want = x.double() @ (ws[0].double() * sc.double()[:, None]).T
    err = float(((y.double() - want).abs().max() / want.abs().max()).item())
    assert err <= 1e-4, f"int8 weight-only linear disagrees with f64: {err}"
    abytes = n * k + n * 4 + m * k * 4 + m * n * 4
    gbs = abytes / (us * 1e-6) / 1e9
    return {"shape": {"m": m, "n": n, "k": k}, "us_per_launch": round(us, 2), "gflops": round(2.0 * m * n * k / (us * 1e-6) / 1e9, 1),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                         "algorithmic_bytes_per_launch": abytes, "kernel": "int8_weight_only_tiled_kernel",
                         "note": "1.2 MB per launch: launch latency, not bandwidth, bounds this configuration; the weights fit L2"},
            "parity": {"max_rel_err_vs_f64_full_output": err, "tolerance": 1e-4}}


def measure_dropin_1m(local_rank: int, samples: int = 30, shape=(256, 4096, 64, 256), peaks: dict | None = None) -> dict:
    """The one workload the reference publishes on this path, through the reference's own operator id and layout:
    `nn.linear_4bit_affine_grouped.1m` (vyre-bench/src/cases/quantized_linear.rs:30-40: in_dim 256, out_dim 4096, group 64,
    batch 256), every buffer resident, device time of one dispatch from the events that bracket it in the contract path
    (the reference samples device timestamps the same way, over the same buffers again and again)."""
    import numpy as np

    import vyre_b200 as vb

    k, n, g, b = shape
    rng = np.random.default_rng(16)
    x = rng.standard_normal(b * k).astype(np.float32)
    packed = rng.integers(0, 2**32, size=(k // 8) * n, dtype=np.uint32)
    scale = rng.uniform(1e-3, 2e-2, size=(k // g) * n).astype(np.float32)
    zp = rng.integers(0, 16, size=(k // g) * n, dtype=np.uint32)
    bias = rng.standard_normal(n).astype(np.float32)
    dev = vb.Device.acquire(local_rank)
    sess = vb.ArtifactSession.compile(vb.linear_4bit_affine_grouped_batched("x", "w", "scale", "zp", "b", "out", k, n, g, b), dev)
    handles = [dev.resident_from(a) for a in (x, packed, scale, zp, bias)] + [dev.allocate_resident(b * n * 4)]
    bs = vb.BindingSet(sess.artifact.digest())
    for slot, h in enumerate(handles):
        bs.insert_resident(slot, h)
    ns = []
    for i in range(samples + 5):
        done = sess.submit(bs, leave_resident=True).wait()
        if i >= 5:
            ns.append(done.device_ns)
        del done
    got = dev.download_resident(handles[5], b * n * 4).view(np.float32)
    # two batch rows against numpy in f64 (the full comparison with the oracle is a GPU test)
    nib = ((packed.reshape(k // 8, 1, n) >> (4 * np.arange(8, dtype=np.uint32)).reshape(1, 8, 1)) & 0xF).reshape(k, n).astype(np.float64)
    wd = (nib - np.repeat(zp.reshape(k // g, n), g, axis=0)) * np.repeat(scale.reshape(k // g, n).astype(np.float64), g, axis=0)
    err = 0.0
    for row in (0, b - 1):
        want = x[row * k:(row + 1) * k].astype(np.float64) @ wd + bias
        err = max(err, float(np.abs(got[row * n:(row + 1) * n] - want).max()))
    assert err <= 1e-4, f"dropin 1m disagrees with the f64 restatement: {err}"
    for h in handles:
        dev.free_resident(h)
    variant = sess.kernel_variant()
    dev.release()
    ns.sort()
    p50 = ns[len(ns) // 2]
    macs = k * n * b
    # algorithmic bytes of one dispatch: packed words, both sidecars, bias, activations in, outputs out
    abytes = (k // 8) * n * 4 + 2 * (k // g) * n * 4 + n * 4 + b * k * 4 + b * n * 4
    if shape != (256, 4096, 64, 256):
        gbs = abytes / (p50 * 1e-9) / 1e9
        return {"case": f"linear_4bit_affine_grouped K={k} N={n} g={g} B={b}", "op_id": "vyre-libs::nn::linear_4bit_affine_grouped",
                "kernel_variant": variant, "device_us_per_dispatch": {"p50": round(p50 / 1e3, 2), "min": round(ns[0] / 1e3, 2), "samples": len(ns)},
                "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"] if peaks else None, "unit": "GB/s",
                             "frac": round(gbs / peaks["hbm_gbs"], 4) if peaks else None, "algorithmic_bytes_per_dispatch": abytes,
                             "kernel": "affine_grouped_decode_kernel" if b <= 4 else "affine_grouped_fast_kernel",
                             "note": "one dispatch per sample between two events (event overhead included); the 33 MB of weights fit L2"},
                "parity": {"max_abs_err_vs_f64_two_rows": err, "tolerance": 1e-4}}
    return {"case": "nn.linear_4bit_affine_grouped.1m", "op_id": "vyre-libs::nn::linear_4bit_affine_grouped",
            "shape": {"in_dim": k, "out_dim": n, "group": g, "batch": b}, "kernel_variant": variant,
            "device_us_per_dispatch": {"p50": round(p50 / 1e3, 2), "min": round(ns[0] / 1e3, 2), "p99": round(ns[-1] / 1e3, 2), "samples": len(ns)},
            "device_ns_per_batch_item_p50": round(p50 / b, 1), "tflops_effective": round(2.0 * macs / (p50 * 1e-9) / 1e12, 2),
            "published_reference": {"device_us_per_dispatch": 214.5, "ns_per_batch_item_p50": 838, "gpu": "RTX 5090 (not this hardware)",
                                    "speedup_vs_published": round(214.5e3 / p50, 1)},
            "roofline": {"bound": "fp32", "achieved": round(2.0 * macs / (p50 * 1e-9) / 1e12, 2), "peak": FP32_TFLOPS_NOMINAL, "unit": "TFLOP/s",
                         "frac": round(2.0 * macs / (p50 * 1e-9) / 1e12 / FP32_TFLOPS_NOMINAL, 4),
                         "peak_kind": "nominal: 148 SMs x 128 FMA lanes x 2 x 1.965 GHz (no measured f32 peak on file)",
                         "kernel": "affine_grouped_fast_kernel", "algorithmic_flops_per_dispatch": 2 * macs, "algorithmic_bytes_per_dispatch": abytes,
                         "note": "0.54 GFLOP over 5.2 MB that stay in L2: bound by the f32 pipe, not by HBM (5.2 MB at the measured HBM peak is 0.8 us)"},
            "l2_policy": "buffers of 5 MB stay in L2, as in the reference's own sample loop",
            "parity": {"max_abs_err_vs_f64_two_rows": err, "tolerance": 1e-4},
            "api": "ArtifactSession.submit with resident bindings, leave_resident; Completion.device_ns",
            "device_ns_samples": ns}


def measure_k_quant(local_rank: int, peaks: dict, samples: int = 20, shape=(4096, 4096)) -> list:
    """GGML K-quant fused linears (vyre-libs/src/nn/quant/ggml.rs:338-385) at a decode shape through the reference's op ids:
    buffers resident, device time of one dispatch from the events of the contract path, one f64 check per run."""
    import numpy as np

    import vyre_b200 as vb

    in_dim, out_dim = shape
    out = []
    dev = vb.Device.acquire(local_rank)
    for bits, build, name in ((4, vb.q4_k_linear, "q4_k_linear"), (2, vb.q2_k_linear, "q2_k_linear")):
        rng = np.random.default_rng(bits)
        block, wpb = (32, 4) if bits == 4 else (16, 1)
        blocks = in_dim * out_dim // block
        packed = rng.integers(0, 2**32, size=blocks * wpb, dtype=np.uint32)
        scales = rng.uniform(0.01, 0.2, size=blocks).astype(np.float32)
        mins = (-rng.uniform(0.0, 1.0, size=blocks)).astype(np.float32)
        x, b = rng.standard_normal(in_dim).astype(np.float32), rng.standard_normal(out_dim).astype(np.float32)
        sess = vb.ArtifactSession.compile(build("x", "p", "s", "m", "b", "o", in_dim, out_dim), dev)
        handles = [dev.resident_from(a) for a in (x, packed, scales, mins, b)] + [dev.allocate_resident(out_dim * 4)]
        bs = vb.BindingSet(sess.artifact.digest())
        for slot, h in enumerate(handles):
            bs.insert_resident(slot, h)
        ns = []
        for i in range(samples + 3):
            done = sess.submit(bs, leave_resident=True).wait()
            if i >= 3:
                ns.append(done.device_ns)
            del done
        got = dev.download_resident(handles[5], out_dim * 4).view(np.float32)
        vpw = 32 // bits
        q = ((packed.reshape(-1, 1) >> (bits * np.arange(vpw, dtype=np.uint32))) & ((1 << bits) - 1)).reshape(in_dim, out_dim)
        deq = q.astype(np.float64) * np.repeat(scales.astype(np.float64), block).reshape(in_dim, out_dim) + \
            np.repeat(mins.astype(np.float64), block).reshape(in_dim, out_dim)
        want = x.astype(np.float64) @ deq + b
        err = float(np.abs(got - want).max() / np.abs(want).max())
        assert err <= 1e-4, f"{name} disagrees with the f64 restatement: {err}"
        for h in handles:
            dev.free_resident(h)
        ns.sort()
        p50 = ns[len(ns) // 2]
        abytes = packed.nbytes + scales.nbytes + mins.nbytes + x.nbytes + b.nbytes + out_dim * 4
        gbs = abytes / (p50 * 1e-9) / 1e9
        out.append({"case": f"{name} in={in_dim} out={out_dim}", "op_id": f"vyre-libs::quant::{name}", "kernel_variant": sess.kernel_variant(),
                    "device_us_per_dispatch": {"p50": round(p50 / 1e3, 2), "min": round(ns[0] / 1e3, 2), "samples": len(ns)},
                    "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": round(gbs / peaks["hbm_gbs"], 4), "algorithmic_bytes_per_dispatch": abytes,
                                 "kernel": "k_quant_linear_fast_kernel",
                                 "note": "one dispatch per sample between two events (event overhead included); the buffers fit L2"},
                    "parity": {"max_rel_err_vs_f64": err, "tolerance": 1e-4}})
    dev.release()
    return out


def measure_residual_block(peaks: dict, rows: int = 1, hidden: int = 4096, inter: int = 14336, layers: int = 3, reps: int = 30) -> dict:
    """The decode residual block (vyre-libs/src/nn/model/dense_gated_mlp.rs:168-370 over int4 projections): RMSNorm, gate /
    up projections, SwiGLU, down projection, residual add, `layers` blocks in a row with weights of their own (together
    larger than L2), one CUDA graph. Timed twice: every operator its own launch (six per block), and with the norm in the
    gate / up launches, SwiGLU in the up launch's stores and the residual add in the down launch's (three per block, one
    programmatic chain). Both must give the same bits."""
    import numpy as np
    import torch

    from vyre_b200 import ffi, synth

    L = ffi.lib()
    bf16 = ffi.DT_BF16
    rng = np.random.default_rng(11)
    dev16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()  # noqa: E731
    weights, host0 = [], {}
    for layer in range(layers):
        nw_np = synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))
        ent = {"nw": dev16(nw_np)}
        if layer == 0:
            host0["post_attention_layernorm.weight"] = nw_np
        for name, (n, k) in {"gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}.items():
            _, w, sc = synth.int4_linear_inputs(1, n, k, seed=17 * layer + len(name))
            ent[name] = (torch.from_numpy(w).cuda(), dev16(sc))
            if layer == 0:
                host0[f"mlp.{name}_proj.qweight"], host0[f"mlp.{name}_proj.scales"] = w.view(np.uint32), sc
        weights.append(ent)
    x0_np = synth.f32_to_bf16_bits((rng.standard_normal((rows, hidden)) * 2).astype(np.float32))
    x0 = dev16(x0_np)
    stream_h = [dev16(np.zeros((rows, hidden), np.uint16)) for _ in range(layers + 1)]
    normed, act, down = (dev16(np.zeros((rows, d), np.uint16)) for d in (hidden, inter, hidden))
    gate, up = (dev16(np.zeros((rows, inter), np.uint16)) for _ in range(2))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    sp, st = C.c_void_p(side.cuda_stream), C.c_void_p(status.data_ptr())
    flags = ffi.LAUNCH_CONSTANT_WEIGHTS
    eps = C.c_float(1e-6)

    def gemv(x, ws, y, n, k):
        ffi.check(L.vyb_k_int4_gemv_ex(x.data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(), y.data_ptr(), rows, n, k, GROUP, bf16, flags, sp, st))

    def block(x, ws, y, n, k, nw=None, res=None, gate_in=None):
        opt = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
        ffi.check(L.vyb_k_int4_linear_block(x.data_ptr(), opt(nw), eps, ws[0].data_ptr(), ws[1].data_ptr(), opt(gate_in), opt(res),
                                            y.data_ptr(), rows, n, k, GROUP, flags, sp, st))

    def separate():
        for i, w in enumerate(weights):
            h, out = stream_h[i], stream_h[i + 1]
            ffi.check(L.vyb_k_rms_norm(h.data_ptr(), w["nw"].data_ptr(), normed.data_ptr(), rows, hidden, eps, bf16, sp))
            gemv(normed, w["gate"], gate, inter, hidden)
            gemv(normed, w["up"], up, inter, hidden)
            ffi.check(L.vyb_k_swiglu(gate.data_ptr(), up.data_ptr(), act.data_ptr(), rows * inter, bf16, sp))
            gemv(act, w["down"], down, hidden, inter)
            ffi.check(L.vyb_k_residual_add(h.data_ptr(), down.data_ptr(), out.data_ptr(), rows * hidden, bf16, sp))

    def fused():
        for i, w in enumerate(weights):
            h, out = stream_h[i], stream_h[i + 1]
            if rows <= 2:
                block(h, w["gate"], gate, inter, hidden, nw=w["nw"])
                block(h, w["up"], act, inter, hidden, nw=w["nw"], gate_in=gate)
            else:  # three and four rows run gate / up on the f16 tensor path, which takes neither norm nor SwiGLU
                ffi.check(L.vyb_k_rms_norm(h.data_ptr(), w["nw"].data_ptr(), normed.data_ptr(), rows, hidden, eps, bf16, sp))
                gemv(normed, w["gate"], gate, inter, hidden)
                gemv(normed, w["up"], up, inter, hidden)
                ffi.check(L.vyb_k_swiglu(gate.data_ptr(), up.data_ptr(), act.data_ptr(), rows * inter, bf16, sp))
            block(act, w["down"], out, hidden, inter, res=h)

    results, finals = {}, []
    for name, body, launches in (("separate_launches", separate, 6), ("fused_launches", fused, 3 if rows <= 2 else 5)):
        stream_h[0].copy_(x0)
        with torch.cuda.stream(side):
            body()  # first launches configure the kernels and make the long-row workspace; must precede capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                body()
        us = event_time_us(graph.replay, reps=reps, warm=3, stream=side) / layers
        finals.append(stream_h[layers].clone())
        results[name] = {"launches_per_block": launches, "us_per_block": round(us, 2)}
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert torch.equal(finals[0], finals[1]), "the fused block's output differs from the separate operators'"
    # the same block through the contract path: the reference's ProgramGraph (six nodes) and the graph the fusion pass makes
    # of it (three nodes), every node a submission on resident buffers; host time of a run, input uploaded, output read back
    import time

    import vyre_b200 as vb

    device = vb.Device.acquire(torch.cuda.current_device())
    graph6 = vb.quantized_gated_mlp_graph(vb.QuantizedGatedMlpSpec(rows, hidden, inter, GROUP, norm_eps=1e-6))
    graph3, taken = graph6.fuse_linear_blocks()
    contract, outs = {}, []
    for name, g in (("program_graph", graph6), ("fused_graph", graph3)):
        sess = vb.GraphSession(g, device)
        for cname, data in host0.items():
            sess.set_constant(cname, data)
        for _ in range(3):
            out = sess.run({"residual": x0_np})["mlp.block_output"]
        t0 = time.perf_counter()
        for _ in range(20):
            out = sess.run({"residual": x0_np})["mlp.block_output"]
        contract[name] = {"nodes": len(g.nodes()), "host_us_per_run": round((time.perf_counter() - t0) / 20 * 1e6, 1)}
        outs.append(out)
        # without the host between the nodes: prepared binding sets, each ordered on the device behind the one before
        for _ in range(3):
            chained = sess.run_chained({"residual": x0_np})["mlp.block_output"]
        t0 = time.perf_counter()
        for _ in range(20):
            chained = sess.run_chained({"residual": x0_np})["mlp.block_output"]
        contract[name]["chained_host_us_per_run"] = round((time.perf_counter() - t0) / 20 * 1e6, 1)
        assert chained == out, "the chained run's block output differs"
        sess.close()
    device.release()
    assert outs[0] == outs[1], "the fused graph's block output differs from the ProgramGraph's"
    assert outs[0] == stream_h[1].cpu().numpy().tobytes(), "the graph's block output differs from the kernel-level chain's first block"
    wbytes = 3 * (hidden * inter // 2 + hidden * inter // GROUP * 2)
    abytes = wbytes + rows * (4 * hidden + 4 * inter) * 2 + 2 * hidden * 2  # weights, scales; residual (read 3x, written once), norm weight 2x, gate / up written and read
    gbs = abytes / (results["fused_launches"]["us_per_block"] * 1e-6) / 1e9
    return {"case": f"residual block rows={rows} hidden={hidden} inter={inter}, {layers} blocks per graph ({layers * wbytes >> 20} MiB of weights)",
            **results, "same_bits": True, "contract_path": {**contract, "nodes_taken_in": taken},
            "speedup": round(results["separate_launches"]["us_per_block"] / results["fused_launches"]["us_per_block"], 3),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(gbs / peaks["hbm_gbs"], 4), "algorithmic_bytes_per_block": abytes,
                         "kernel": "int4_gemv_halfsm_kernel (fused whole-row and k-block forms)"}}


def metric_stats(samples) -> dict:
    """vyre-bench MetricStats (vyre-bench/SCHEMA.md, `MetricStats` object) of integer samples."""
    v = sorted(int(x) for x in samples)
    n = len(v)
    pick = lambda q: v[min(n - 1, int(q * n))]  # noqa: E731
    mean = sum(v) / n
    sd = (sum((x - mean) ** 2 for x in v) / n) ** 0.5
    return {"samples": n, "min": v[0], "max": v[-1], "mean": mean, "median": v[n // 2], "p90": pick(0.90), "p95": pick(0.95),
            "p99": pick(0.99), "p999": pick(0.999), "p9999": pick(0.9999), "stddev": sd, "cv": sd / mean if mean else 0.0,
            "determinism_cv": None}


def vyre_bench_result(m: int, kernel_us: float, timed_launches: int, peak_gbs: float, dropin: dict, cpu: dict | None, wall_s: float) -> dict:
    """The two cases of this run in the reference bench's own result shape (vyre-bench/SCHEMA.md `vyre-bench.result.v1`,
    metric keys of vyre-bench/src/runner/execute/metric_keys.rs:520-541): the headline GEMV and the reference's published
    case. The GEMV's per-launch time is an average over a graph replay, so its statistics collapse to that value."""
    import torch

    gemv_ns = int(round(kernel_us * 1e3))
    gemv_gbs = algorithmic_bytes(m) / gemv_ns
    cases = [{
        "id": f"nn.linear_int4_grouped_rowmajor.decode_m{m}", "status": "passed", "correctness": "approximate",
        "wall_ns": metric_stats([gemv_ns]), "artifacts": [], "contract": None, "competitors": None,
        "speedup": (cpu["ms_per_gemv"] * 1e6 / gemv_ns) if cpu else None,
        "metrics": {"kernel_execute_ns": dict(metric_stats([gemv_ns]), samples=timed_launches),
                    "bytes_touched": metric_stats([algorithmic_bytes(m)]),
                    "device_gb_s_x1000": metric_stats([round(gemv_gbs * 1000)]),
                    "roofline_mem_pct_x1000": metric_stats([round(100000 * gemv_gbs / peak_gbs)])}}]
    ns = dropin["device_ns_samples"]
    abytes = dropin["roofline"]["algorithmic_bytes_per_dispatch"]
    cases.append({
        "id": "nn.linear_4bit_affine_grouped.1m", "status": "passed", "correctness": "approximate", "wall_ns": metric_stats(ns),
        "artifacts": [], "contract": None, "competitors": None, "speedup": None,
        "metrics": {"kernel_execute_ns": metric_stats(ns), "bytes_touched": metric_stats([abytes]),
                    "device_gb_s_x1000": metric_stats([round(1000 * abytes / x) for x in ns]),
                    "roofline_mem_pct_x1000": metric_stats([round(100000 * (abytes / x) / peak_gbs) for x in ns])}})
    prop = torch.cuda.get_device_properties(0)
    return {"schema": "vyre-bench.result.v1", "run_id": "vyre-b200.bench", "suite": "gpu", "features": ["backend:cuda-b200"],
            "environment": {"cpu_model": cpu_model(), "gpu_name": prop.name, "gpu_memory_mb": prop.total_memory // (1 << 20),
                            "cuda_version": torch.version.cuda, "os": sys.platform},
            "cases": cases,
            "summary": {"total_cases": len(cases), "passed": len(cases), "failed": 0, "total_time_ns": int(wall_s * 1e9), "cache_hit_rate": 1.0}}


def moe_inputs(tokens, hidden, inter, experts_local, experts, seed_rank):
    import torch

    torch.manual_seed(1234 + seed_rank)
    x = torch.randn((tokens, hidden), device="cuda").to(torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(7)  # the router is replicated: same values on every rank
    wr = (torch.randn((experts, hidden), device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    # expert weights depend on the GLOBAL expert index only, so that a token's result is the same at every world size
    w13, s13, w2, s2 = [], [], [], []
    first = seed_rank * experts_local
    for e in range(first, first + experts_local):
        ge = torch.Generator(device="cuda").manual_seed(100 + e)
        w13.append(torch.randint(0, 256, (2, inter, hidden // 2), dtype=torch.uint8, device="cuda", generator=ge))
        s13.append((torch.rand((2, inter, hidden // GROUP), device="cuda", generator=ge) * 0.019 + 0.001).to(torch.bfloat16))
        w2.append(torch.randint(0, 256, (hidden, inter // 2), dtype=torch.uint8, device="cuda", generator=ge))
        s2.append((torch.rand((hidden, inter // GROUP), device="cuda", generator=ge) * 0.019 + 0.001).to(torch.bfloat16))
    return x, wr, torch.stack(w13), torch.stack(s13), torch.stack(w2), torch.stack(s2)


def measure_moe(world: int, rank: int, dist, steps: int, warmup: int, peaks: dict) -> dict:
    """Config 4: 4096 tokens in total, 8 experts top-2, expert-parallel over the ranks with device-side dispatch and
    combine over peer memory (one GPU: the fused single-GPU layer). Tokens/s over all ranks; a sample of rank 0's
    outputs is compared with the single-GPU layer run on the same tokens and experts when the weights fit."""
    import torch

    from vyre_b200 import ffi, sharding

    L = ffi.lib()
    tokens_total, inter, hidden, experts, topk = 4096, 14336, 4096, 8, 2
    local = experts // world
    tokens = tokens_total // world
    torch.manual_seed(99)
    x_all = torch.randn((tokens_total, hidden), device="cuda").to(torch.bfloat16)  # same on every rank
    x = x_all[rank * tokens:(rank + 1) * tokens].contiguous()
    _, wr, w13, s13, w2, s2 = moe_inputs(1, hidden, inter, local, experts, rank)
    stream = torch.cuda.current_stream()
    if world == 1:
        need = C.c_uint64(0)
        ffi.check(L.vyb_k_moe_ffn_int4_scratch_bytes(tokens, hidden, inter, experts, topk, C.byref(need)))
        scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
        out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
        ridx = torch.empty((tokens, topk), dtype=torch.int32, device="cuda")
        rw = torch.empty((tokens, topk), dtype=torch.float32, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")

        def step():
            ffi.check(L.vyb_k_moe_ffn_int4(x.data_ptr(), wr.data_ptr(), w13.data_ptr(), s13.data_ptr(), w2.data_ptr(),
                                           s2.data_ptr(), out.data_ptr(), ridx.data_ptr(), rw.data_ptr(), scratch.data_ptr(),
                                           need.value, tokens, hidden, inter, experts, topk, GROUP,
                                           C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))
            return out
    else:
        ops = sharding.DeviceExpertParallel(wr, w13, s13, w2, s2, hidden, inter, experts, topk, tokens_local_max=tokens,
                                            tokens_total=tokens_total, group_size=GROUP)
        status = ops.status
        # one layer = eleven launches ordered by cross-GPU arrival counters; replayed as one CUDA graph, as a serving loop would
        ops.forward(x)
        torch.cuda.synchronize()
        layer = torch.cuda.CUDAGraph()
        with torch.cuda.graph(layer):
            y_static = ops.forward(x)[0]

        def step():
            layer.replay()
            return y_static

    for _ in range(max(3, warmup)):
        step()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        y = step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    if dist:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    assert status.cpu().tolist() == [0, 0, 0, 0], "a bounded device-side wait ran out in the MoE layer"
    # a checksum of the first 64 output rows of the whole batch: the same tokens meet the same experts at every world
    # size, and every row is computed by the same kernel arithmetic wherever it runs, so the value must not depend on N
    digest = None
    if rank == 0:
        import hashlib

        digest = hashlib.sha256(y[:64].view(torch.int16).cpu().numpy().tobytes()).hexdigest()[:16]
    flops = 2.0 * tokens_total * topk * 3 * inter * hidden
    tflops = flops / (ms * 1e-3) / 1e12
    return {"tokens_per_s": round(tokens_total / (ms * 1e-3)), "ms_per_layer": round(ms, 4), "expert_tflops": round(tflops, 1),
            "parallelism": "single GPU, fused layer" if world == 1 else f"expert-parallel x{world}, device-side dispatch/combine over peer memory (NVLink)",
            "scaling": "strong", "tokens_total": tokens_total, "first_64_rows_sha256_16": digest,
            "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": round(peaks["bf16_tflops"] * world, 1), "unit": "TFLOP/s",
                         "frac": round(tflops / (peaks["bf16_tflops"] * world), 4), "peak_kind": f"{world} x cuBLAS bf16 burst, of {peaks['kind']}",
                         "kernel": "int4_gemm_pair_kernel (grouped, two launches per layer)", "us_per_launch": None}}


def measure_colpar_int8(world: int, rank: int, dist, steps: int, warmup: int, i8_peak: float) -> dict:
    """Config 5: X bf16 [4096, 8192] quantised per token, W int8 [28672, 8192] sharded by rows over the ranks, int32
    outputs gathered into the full [4096, 28672] on every rank by peer stores (chunks over M overlap GEMM and gather)."""
    import torch

    from vyre_b200 import ffi, sharding

    L = ffi.lib()
    m, n, k = 4096, 28672, 8192
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    torch.manual_seed(5)
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    gather = sharding.PeerColumnGather(m, n, 4, multiple=16)
    w = torch.randint(-127, 128, (gather.end - gather.begin, k), dtype=torch.int8, device="cuda")  # this rank's rows
    xq = torch.empty((m, k), dtype=torch.int8, device="cuda")
    sc = torch.empty(m, dtype=torch.float32, device="cuda")
    cur = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    ffi.check(L.vyb_k_quantize_per_token_int8(x.data_ptr(), xq.data_ptr(), sc.data_ptr(), m, k, C.c_void_p(cur.cuda_stream)))
    y_local = torch.empty((m, w.shape[0]), dtype=torch.int32, device="cuda")

    def compute_only():
        ffi.check(L.vyb_k_int8_gemm_i32(xq.data_ptr(), w.data_ptr(), y_local.data_ptr(), m, w.shape[0], k,
                                        C.c_void_p(cur.cuda_stream), C.c_void_p(status.data_ptr())))

    def gather_only():
        gather.push(y_local, 0, cur.cuda_stream, status)
        gather.wait(cur.cuda_stream, status)

    def total():  # one kernel: the GEMM's epilogue stores every tile into every rank's output
        return sharding.column_parallel_int8_linear(gather, xq, w, status)

    def chunked():  # four row chunks, a copy kernel on a side stream behind each
        return sharding.column_parallel_int8_linear(gather, xq, w, status, chunks=4, side_stream=side, fused=False)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        if dist:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.barrier()
        return ms

    ms_compute = timed(compute_only)
    ms_gather = timed(gather_only)
    ms_total = timed(total)
    ms_chunked = timed(chunked)
    full, _ = total()
    compute_only()
    mine = y_local
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0], "a bounded device-side wait ran out in the column-parallel gather"
    own_ok = bool(torch.equal(full[:, gather.begin:gather.end], mine))
    want = (xq[:64].double() @ w[:128].double().T).to(torch.int64)
    exact = bool(torch.equal(mine[:64, :128].to(torch.int64), want))
    assert own_ok and exact, "column-parallel int8 linear: gathered block or GEMM tile is wrong"
    ops = 2.0 * m * n * k
    tops = ops / (ms_total * 1e-3) / 1e12
    return {"tops": round(tops, 1), "ms_compute": round(ms_compute, 4), "ms_gather": round(ms_gather, 4), "ms_total": round(ms_total, 4),
            "ms_total_chunked_copy_kernel": round(ms_chunked, 4), "tops_compute_only": round(ops / (ms_compute * 1e-3) / 1e12, 1), "scaling": "strong",
            "parallelism": f"N sharded over {world} rank(s); GEMM and gather are one kernel: the tcgen05 epilogue stores every tile into every rank's output (peer stores over NVLink)",
            "gather_bytes_received_per_rank": int(m * n * 4 * (world - 1) / world),
            "parity": {"own_block_in_gathered_output": own_ok, "gemm_tile_bit_exact_vs_f64": exact},
            "roofline": {"bound": "tensor", "achieved": round(tops, 1), "peak": round(i8_peak * world, 1), "unit": "TOP/s",
                         "frac": round(tops / (i8_peak * world), 4), "peak_kind": f"{world} x tcgen05 kind::i8 peak measured in this run",
                         "kernel": "int8_gemm_pair_kernel (gathering epilogue)", "us_per_launch": round(ms_total * 1e3, 1)}}


def run_native(args) -> None:
    import numpy as np
    import torch

    import vyre_b200 as vb
    from vyre_b200 import ffi, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist  # noqa: PLW0642

        # the collectives here move a few KB: in-switch reduction buys nothing, and without it no rank's memory is
        # bound to an NVLink multicast object while the ranks leave one after the other
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = ffi.lib()
    m = args.m
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    peaks = measured_peaks()
    t_run0 = time.perf_counter()

    # ---- resident inputs: COPIES distinct weight sets so that consecutive launches never hit L2 ----------------------
    x_np, w_np, s_np = synth.int4_linear_inputs(m, N_OUT, K_IN, seed=rank)
    x = torch.from_numpy(x_np.view(np.int16)).cuda()
    ws, ss = [], []
    for c in range(COPIES):
        ws.append(torch.from_numpy(np.roll(w_np, c, axis=0)).cuda())
        ss.append(torch.from_numpy(np.roll(s_np, c, axis=0).view(np.int16)).cuda())
    y = torch.zeros((m, N_OUT), dtype=torch.bfloat16, device="cuda")
    pag = None
    if world > 1:
        from vyre_b200 import sharding

        pag = sharding.PeerAllGather(m, N_OUT)  # the all-gather is this library's own, by peer stores over NVLink, not NCCL
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    gemv_flags = ffi.LAUNCH_CONSTANT_WEIGHTS

    def launch(c: int, out=None, xin=None, mm=None):
        # weights are graph constants: the launch may overlap the tail of the previous one
        ffi.check(L.vyb_k_int4_gemv_ex((x if xin is None else xin).data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(),
                                       (y if out is None else out).data_ptr(), m if mm is None else mm, N_OUT, K_IN, GROUP,
                                       ffi.DT_BF16, gemv_flags, C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

    def capture(body):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g, stream=stream):
                body()
        return g

    with torch.cuda.stream(stream):
        for c in range(COPIES):  # first launches configure the kernels; must precede graph capture
            launch(c)
    stream.synchronize()

    def step_body():
        if pag is None:
            for c in range(LAUNCHES):
                launch(c % COPIES)
            return
        # GEMV and all-gather are one kernel and one programmatic chain: launch c writes buffer half c % 2 on this rank and,
        # by peer stores over NVLink from the same kernel, on every other rank. The replay ends with the bounded wait for its
        # own gathers. (The pipelined form, where launch c + 1 carries launch c's outputs over, measured no faster.)
        for c in range(LAUNCHES):
            pag.gemv(c & 1, x, ws[c % COPIES], ss[c % COPIES], K_IN, stream.cuda_stream, status, gemv_flags)
        pag.wait(stream.cuda_stream, status)

    graph = capture(step_body)
    with torch.cuda.stream(stream):
        graph.replay()
    stream.synchronize()
    if pag is not None:
        # the gathered result of the graph's last launch (half 1) against NCCL's all-gather of the plain kernel's output
        launch(COPIES - 1)
        stream.synchronize()
        want_all = torch.empty((world, m, N_OUT), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(want_all.view(-1), y.view(-1))
        torch.cuda.synchronize()
        assert torch.equal(pag.halves()[1].view(torch.int16), want_all.view(torch.int16)), "peer-store all-gather differs from NCCL"
        y = pag.halves()[1][rank]
    y_ref = y.clone()

    for _ in range(warmup):
        with torch.cuda.stream(stream):
            graph.replay()
    stream.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    lo = sampler.mark()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(steps):
            graph.replay()
        end.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    hi = sampler.mark()
    elapsed_ms = start.elapsed_time(end)
    if dist:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    assert status.cpu().tolist() == [0, 0, 0, 0], "a bounded device-side wait ran out during the bench"
    assert torch.equal(y, y_ref), "non-deterministic GEMV output during the bench"
    ms_per_step = elapsed_ms / steps
    step_bytes = LAUNCHES * algorithmic_bytes(m)
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- kernel-only time of the dominant kernel (no collective), for the roofline: a longer region of its own, so
    # that the figure does not hang on the few hundred microseconds of a 20-step run; clocks sampled across it
    kgraph = capture(lambda: [launch(c % COPIES) for c in range(LAUNCHES)])
    k_lo = sampler.mark()
    kernel_reps = args.kernel_reps or max(steps, 60)
    kernel_us = event_time_us(kgraph.replay, reps=kernel_reps, warm=3, stream=stream) / LAUNCHES
    if rank == 0:
        time.sleep(0.06)
    k_hi = sampler.mark()
    achieved = algorithmic_bytes(m) / (kernel_us * 1e-6) / 1e9
    extra = {}
    if rank == 0:
        for mm in (2, 4, 8):
            xm_np, _, _ = synth.int4_linear_inputs(mm, 16, K_IN, seed=3)
            xm = torch.from_numpy(xm_np.view(np.int16)).cuda()
            ym = torch.zeros((mm, N_OUT), dtype=torch.bfloat16, device="cuda")
            for c in range(COPIES):
                launch(c, ym, xm, mm)
            stream.synchronize()
            g2 = capture(lambda: [launch(c % COPIES, ym, xm, mm) for c in range(LAUNCHES)])
            us = event_time_us(g2.replay, reps=min(40, kernel_reps), warm=3, stream=stream) / LAUNCHES
            gbs = algorithmic_bytes(mm) / (us * 1e-6) / 1e9
            extra[f"m{mm}"] = {"us_per_launch": round(us, 3), "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peaks["hbm_gbs"], 4)}
            del g2
        # the down projection of the same feed-forward block: N=4096, K=14336 (the same bytes of weights and scales read as
        # [4096, 14336 / 2] and [4096, 112]); rows longer than 4096 are cut into k blocks inside one launch
        dn, dk = K_IN, N_OUT
        xd = torch.from_numpy(synth.int4_linear_inputs(1, 16, dk, seed=4)[0].view(np.int16)).cuda()
        yd = torch.zeros((1, dn), dtype=torch.bfloat16, device="cuda")

        def launch_down(c):
            ffi.check(L.vyb_k_int4_gemv_ex(xd.data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(), yd.data_ptr(), 1, dn, dk, GROUP,
                                           ffi.DT_BF16, gemv_flags, C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

        with torch.cuda.stream(stream):
            for c in range(COPIES):
                launch_down(c)
        stream.synchronize()
        g3 = capture(lambda: [launch_down(c % COPIES) for c in range(LAUNCHES)])
        us = event_time_us(g3.replay, reps=min(40, kernel_reps), warm=3, stream=stream) / LAUNCHES
        gbs = algorithmic_bytes(1, n=dn, k=dk) / (us * 1e-6) / 1e9
        extra["m1_n4096_k14336"] = {"us_per_call": round(us, 3), "launches_per_call": 1, "k_blocks": 7, "gbs": round(gbs, 1),
                                    "frac_of_measured_peak": round(gbs / peaks["hbm_gbs"], 4)}
        del g3
        # whole rows of 2048: the same bytes read as [28672, 2048 / 2] and [28672, 16] (six pipeline stages of half-size tiles)
        hn, hk = 2 * N_OUT, K_IN // 2
        # (seed 6: the row of seed 5 holds an element 2^-20 below its group's largest, which sends one warp through the wide
        # activation conversion and costs that launch 1.1 us of prologue: 7.3 us instead of 6.2 us)
        xh2 = torch.from_numpy(synth.int4_linear_inputs(1, 16, hk, seed=6)[0].view(np.int16)).cuda()
        yh2 = torch.zeros((1, hn), dtype=torch.bfloat16, device="cuda")

        def launch_half(c):
            ffi.check(L.vyb_k_int4_gemv_ex(xh2.data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(), yh2.data_ptr(), 1, hn, hk, GROUP,
                                           ffi.DT_BF16, gemv_flags, C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

        with torch.cuda.stream(stream):
            for c in range(COPIES):
                launch_half(c)
        stream.synchronize()
        g4 = capture(lambda: [launch_half(c % COPIES) for c in range(LAUNCHES)])
        us = event_time_us(g4.replay, reps=min(40, kernel_reps), warm=3, stream=stream) / LAUNCHES
        gbs = algorithmic_bytes(1, n=hn, k=hk) / (us * 1e-6) / 1e9
        extra["m1_n28672_k2048"] = {"us_per_call": round(us, 3), "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peaks["hbm_gbs"], 4)}
        del g4
    clocks_headline = sampler.summary(lo, hi) if rank == 0 else None
    clocks_kernel = sampler.summary(k_lo, k_hi) if rank == 0 else None

    # ---- the sharded configurations of the path, at this N (every rank takes part) ------------------------------------
    del graph, kgraph
    torch.cuda.synchronize()
    secondary = {}
    i8_peak = tensor_peak(True)
    s_lo = sampler.mark()
    secondary["moe_ep_config4"] = measure_moe(world, rank, dist, steps=5, warmup=3, peaks=peaks)
    torch.cuda.empty_cache()
    secondary["int8_colpar_config5"] = measure_colpar_int8(world, rank, dist, steps=5, warmup=2, i8_peak=i8_peak)
    torch.cuda.empty_cache()
    s_hi = sampler.mark()

    # All ranks leave the process group together, right after the collective work; what follows on rank 0 is single-GPU.
    if dist:
        pag = None
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        dist = None
    if rank != 0:
        return

    secondary["tensor_peaks_measured_in_run"] = {"int8_tops": round(i8_peak, 1), "bf16_tflops": round(tensor_peak(False), 1),
                                                 "how": "tcgen05.mma 128x256 tiles from shared-memory operands, one CTA per SM"}
    secondary["int4_prefill_gemm_config3"] = measure_prefill([2048, 14336, 4096], 20, 5, peaks)
    secondary["int8_gemm_config5_single_gpu"] = measure_int8([4096, 28672, 8192], 10, 3, i8_peak, peaks)
    secondary["int8_weight_only_config1"] = measure_int8_weight_only(peaks)
    secondary["dropin_1m"] = measure_dropin_1m(local_rank)
    secondary["dropin_decode_shape"] = measure_dropin_1m(local_rank, shape=(K_IN, N_OUT, GROUP, 1), peaks=peaks)
    secondary["k_quant_linear"] = measure_k_quant(local_rank, peaks)
    secondary["residual_block_m1"] = measure_residual_block(peaks)
    secondary["clocks_during_secondary"] = sampler.summary(s_lo, sampler.mark())
    torch.cuda.empty_cache()

    # ---- end to end through the contract path: host x -> submit -> wait -> host y, weights resident ------------------
    # one prepared binding set per weight copy (validated once, one graph launch per submission); the activations of
    # every step are copied in from pinned host memory and the outputs read back to host memory inside the timed region
    dev = vb.Device.acquire(local_rank)
    prog = vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, K_IN, N_OUT, GROUP, ffi.DT_BF16)
    sess = vb.ArtifactSession.compile(prog, dev)
    hw = [dev.resident_from(np.roll(w_np, c, axis=0).view(np.uint32)) for c in range(COPIES)]
    hs = [dev.resident_from(np.roll(s_np, c, axis=0)) for c in range(COPIES)]
    x_pinned = torch.from_numpy(x_np.view(np.int16).copy()).pin_memory().numpy().view(np.uint16)
    preps = []
    for c in range(COPIES):
        bs = vb.BindingSet(sess.artifact.digest())
        bs.insert_host(0, x_pinned)
        bs.insert_resident(1, hw[c])
        bs.insert_resident(2, hs[c])
        preps.append(sess.prepare(bs))
    depth = 4
    e2e_steps = max(2, min(steps, 100))

    def e2e_step(keep):
        inflight, last = [], None
        for c in range(LAUNCHES):
            inflight.append(preps[c % COPIES].submit({0: x_pinned}))
            if len(inflight) == depth:
                last = inflight.pop(0).wait()
                keep[0] += float(last.output_view(3, np.uint16)[0])
                del last
        while inflight:
            last = inflight.pop(0).wait()
            keep[0] += float(last.output_view(3, np.uint16)[0])
            if inflight:
                del last
        return last

    keep = [0.0]
    for _ in range(max(3, min(warmup, 5))):
        del_last = e2e_step(keep)
        del del_last
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        last = e2e_step(keep)
        if _ != e2e_steps - 1:
            del last
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    got_last = np.frombuffer(last.output(3), np.uint16).reshape(m, N_OUT)
    want_last = y_ref.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got_last, want_last), "contract path and kernel-level path disagree"
    del last
    e2e = {"value": step_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(LAUNCHES * x_pinned.nbytes),
           "d2h_bytes_per_step": int(LAUNCHES * m * N_OUT * 2), "us_per_step": round(e2e_s * 1e6, 2),
           "us_per_submission": round(e2e_s * 1e6 / LAUNCHES, 2), "steps": e2e_steps, "in_flight": depth, "n_gpus_measured": 1,
           "api": "ArtifactSession.prepare + PreparedSubmission.submit / Submission.wait (vyb_prepare, vyb_prepared_submit, "
                  "vyb_submission_wait), weights resident, rank 0's GPU"}
    for p in preps:
        p.free()
    for h in hw + hs:
        dev.free_resident(h)
    dev.release()
    sampler.stop()

    cpu = None
    if world == 1:
        per_gemv, cpu_threads = cpu_gemv_times(m, samples=9, warmup=1)
        med = statistics.median(per_gemv)
        cpu = {"value": algorithmic_bytes(m) / med / 1e9, "unit": "GB/s", "cores": cpu_threads, "kind": "port",
               "sample": f"median of 9 full GEMVs M={m} (rows [0,{N_OUT}) x K={K_IN}) of the reference bench's f32 loop "
                         "(vyre-bench/src/cases/quantized_linear.rs:447-463 restated for the row-major layout), -O3, OpenMP over rows",
               "ms_per_gemv": round(med * 1e3, 3), "cpu_model": cpu_model()}

    launches_per_step = LAUNCHES + (1 if world > 1 else 0)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16xint4->f32", "data": "synthetic",
        "config": {"workload": workload_name(m)},
        "run": {"per_gpu_shard": [N_OUT, K_IN],
                "parallelism": f"column-parallel x{world}" + (" + all-gather by peer stores over NVLink from the GEMV kernel itself, one launch" if world > 1 else ""),
                "l2_policy": f"inputs larger than L2: {COPIES} rotating weight copies = {COPIES * (N_OUT * K_IN // 2) / 1e6:.0f} MB",
                "launch": f"CUDA graph of {LAUNCHES} launches per step ({PASSES} passes over the {COPIES} copies), programmatic dependent launch (constant weights)"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(m), "traffic_source": "recorded constant from an ncu capture (profiles/), not measured in this run",
                     "peak_kind": f"of {peaks['kind']}", "kernel": "int4_gemv_halfsm_kernel",
                     "us_per_launch": round(kernel_us, 3), "algorithmic_bytes_per_launch": algorithmic_bytes(m),
                     "timed_launches": kernel_reps * LAUNCHES, "frac_of_nominal_8tbs": achieved / 8000.0, "clocks": clocks_kernel},
        "e2e": e2e, "gpu_launches": steps * launches_per_step, "clocks": clocks_headline, "other_batches": extra,
        "secondary": secondary,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    line["vyre_bench"] = vyre_bench_result(m, kernel_us, kernel_reps * LAUNCHES, peaks["hbm_gbs"], secondary["dropin_1m"], cpu,
                                           time.perf_counter() - t_run0)
    del secondary["dropin_1m"]["device_ns_samples"]
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the decode GEMV, from one ncu capture of the M=1 case over
# 8 rotating weight copies (summary kept under profiles/); other batches were not captured.
NCU_DRAM_BYTES_PER_LAUNCH = {1: 30331648}


def run_quick(args) -> None:
    """A few plain launches of one kernel; prints one short JSON line (the cases profiled under ncu)."""
    import numpy as np
    import torch

    from vyre_b200 import ffi, synth

    peaks = measured_peaks()
    if args.case == "prefill":
        print(json.dumps({"quick": True, "case": "prefill", "shape": args.shape, **measure_prefill(args.shape, args.steps, args.warmup, peaks)}))
        return
    if args.case == "int8gemm":
        print(json.dumps({"quick": True, "case": "int8gemm", "shape": args.shape,
                          **measure_int8(args.shape, args.steps, args.warmup, 2 * peaks["bf16_tflops"], peaks)}))
        return
    if args.case == "dropin":
        first = measure_dropin_1m(0)
        first.pop("device_ns_samples", None)
        print(json.dumps({"quick": True, "k_quant": measure_k_quant(0, peaks), "dropin_1m": first,
                          "dropin_decode_shape": [measure_dropin_1m(0, shape=(K_IN, N_OUT, GROUP, bb), peaks=peaks) for bb in (1, 4, 8)]}))
        return
    if args.case == "block":
        print(json.dumps({"quick": True, "case": "block", **measure_residual_block(peaks, rows=args.m, reps=args.steps)}))
        return
    if args.case == "peak":
        print(json.dumps({"quick": True, "case": "peak", "int8_tops": tensor_peak(True), "bf16_tflops": tensor_peak(False)}))
        return
    L = ffi.lib()
    m = args.m
    n_out = args.rows or N_OUT
    k_in = args.k or K_IN
    x_np, w_np, s_np = synth.int4_linear_inputs(m, n_out, k_in, seed=0)
    x = torch.from_numpy(x_np.view(np.int16)).cuda()
    copies = max(1, args.copies)
    ws = [torch.from_numpy(np.roll(w_np, c, axis=0)).cuda() for c in range(copies)]
    ss = [torch.from_numpy(np.roll(s_np, c, axis=0).view(np.int16)).cuda() for c in range(copies)]
    y = torch.zeros((m, n_out), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    it = [0]

    def launch(stream=None):
        c = it[0] % copies
        it[0] += 1
        ffi.check(L.vyb_k_int4_gemv_ex(x.data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(), y.data_ptr(), m, n_out, k_in,
                                       GROUP, ffi.DT_BF16, ffi.LAUNCH_CONSTANT_WEIGHTS,
                                       C.c_void_p(stream or torch.cuda.current_stream().cuda_stream), C.c_void_p(status.data_ptr())))

    if args.graph:
        # the headline's launch pattern for any batch and row count: a graph of LAUNCHES launches, replayed `steps` times
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(copies):
                launch(side.cuda_stream)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(LAUNCHES):
                    launch(side.cuda_stream)
            for _ in range(max(3, args.warmup)):
                graph.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side)
            for _ in range(args.steps):
                graph.replay()
            b.record(side)
        side.synchronize()
        us = a.elapsed_time(b) * 1e3 / (args.steps * LAUNCHES)
    else:
        us = event_time_us(launch, args.steps, args.warmup)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    gbs = algorithmic_bytes(m, n=n_out, k=k_in) / (us * 1e-6) / 1e9
    print(json.dumps({"quick": True, "m": m, "rows": n_out, "k": k_in, "graph": bool(args.graph), "steps": args.steps, "copies": copies,
                      "us_per_launch": round(us, 3), "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peaks["hbm_gbs"], 4)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--m", type=int, default=1, help="decode batch (1, 4 or 8)")
    ap.add_argument("--case", default="gemv", choices=["gemv", "prefill", "int8gemm", "peak", "dropin", "block"], help="kernel exercised by --quick")
    ap.add_argument("--shape", type=int, nargs=3, default=[2048, 14336, 4096], metavar=("M", "N", "K"),
                    help="GEMM shape for --quick --case prefill|int8gemm")
    ap.add_argument("--kernel-reps", type=int, default=0,
                    help="graph replays of the kernel-only roofline region (0: max(steps, 60)); small values shorten a profiler's launch list")
    ap.add_argument("--copies", type=int, default=COPIES,
                    help="weight copies rotated in --quick mode (1 keeps the weights L2-resident: compute-bound check)")
    ap.add_argument("--rows", type=int, default=0, help="weight rows N in --quick --case gemv (0: the configuration's 14336)")
    ap.add_argument("--k", type=int, default=0, help="row length K in --quick --case gemv (0: the configuration's 4096)")
    ap.add_argument("--graph", action="store_true",
                    help="--quick --case gemv: time replays of a CUDA graph of 64 launches (the headline's launch pattern) instead of single launches")
    ap.add_argument("--quick", action="store_true",
                    help="kernel-only run without graphs, end-to-end leg or CPU baseline (the case profiled under ncu)")
    args = ap.parse_args()
    if args.impl == "reference":
        # torchrun exports OMP_NUM_THREADS=1 to its workers: the CPU arm uses every host core, like the reference's rayon pool
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        if args.steps == 200 and args.warmup == 20:
            args.steps, args.warmup = 5, 1
        run_reference(args)
    elif args.quick:
        if args.steps == 200 and args.warmup == 20:
            args.steps, args.warmup = 16, 8
        run_quick(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
