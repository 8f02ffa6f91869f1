"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Headline (N=1): the int4 group-quantized decode GEMV of the benchmark's second configuration
(W u4 [14336, 4096], group 128, bf16 scales, x bf16 [M=1, 4096]), reported as achieved HBM GB/s =
algorithmic bytes per launch / device time per launch. A step is one GEMV launch over one batch of
activations; launches rotate over 8 resident copies of the weights (242 MB > the 126 MB L2) so every step
streams its weights from HBM. Timing is CUDA events on the launching stream, max over ranks.

For N > 1 the linear is sharded column-parallel: every rank owns a [14336, 4096] shard of a 14336*N-row
linear (weak scaling) and each step's bf16 outputs are all-gathered by this library's own peer-store kernel over
NVLink (one CTA on a side stream, bounded completion checks), overlapped with the next GEMV and verified once
against NCCL's all-gather before timing.

`--impl reference` times the CPU restatement of the reference engine (oracle/) on the host cores over a bounded
row sample of the same workload.
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_OUT, K_IN, GROUP = 14336, 4096, 128
COPIES = 8
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(m: int, n: int = N_OUT, k: int = K_IN, group: int = GROUP) -> int:
    """Packed weights + bf16 scales + bf16 x + bf16 y, each touched once."""
    return n * k // 2 + n * (k // group) * 2 + m * k * 2 + m * n * 2


def measured_peaks() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self, lo: int = 0, hi: int | None = None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
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


def cpu_reference_rate(m: int, budget_s: float, steps: int | None = None, warmup: int = 0):
    """Times the CPU restatement of the reference engine on a bounded row sample of the GEMV workload.
    Returns (GB/s, seconds per step, sample description, threads)."""
    import oracle
    from vyre_b200 import synth

    threads = oracle.num_threads()
    x, w, s = synth.int4_linear_inputs(m, N_OUT, K_IN, seed=0)
    probe_rows = 512
    t0 = time.perf_counter()
    oracle.int4_rowmajor_linear(x, w[:probe_rows], s[:probe_rows], m, probe_rows, K_IN)
    per_row = (time.perf_counter() - t0) / probe_rows
    if steps is None:
        rows, reps = N_OUT, max(3, int(budget_s / max(per_row * N_OUT, 1e-6)))
        reps = min(reps, 200)
    else:
        rows = int(max(16, min(N_OUT, budget_s / max(1, steps + warmup) / max(per_row, 1e-9))))
        reps = steps
    for _ in range(warmup if steps is not None else 1):
        oracle.int4_rowmajor_linear(x, w[:rows], s[:rows], m, rows, K_IN)
    t0 = time.perf_counter()
    for _ in range(reps):
        oracle.int4_rowmajor_linear(x, w[:rows], s[:rows], m, rows, K_IN)
    dt = (time.perf_counter() - t0) / reps
    gbs = algorithmic_bytes(m, n=rows) / dt / 1e9
    sample = f"{reps} x int4 GEMV M={m} on rows [0,{rows}) of {N_OUT} x K={K_IN} (f64-accumulating oracle, OpenMP over rows)"
    return gbs, dt, sample, threads


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    gbs, dt, sample, threads = cpu_reference_rate(1, budget_s=120.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "int4_decode_gemv_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16xint4->f32", "data": "synthetic",
        "config": {"workload": "int4 group-quantized decode GEMV M=1 N=14336 K=4096 g=128 (config 2), CPU row sample"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum per launch of int4_gemv_kernel, from one ncu capture of the M=1
# case over 8 rotating weight copies (summary kept under profiles/); other batches were not captured.
NCU_DRAM_BYTES_PER_LAUNCH = {1: 30346368}


def measure_case(case: str, shape, steps: int, warmup: int) -> dict:
    """Times plain launches of one of the tensor-core paths (prefill GEMM, int8 GEMM, fused MoE layer) with CUDA events."""
    import torch

    from vyre_b200 import ffi

    L = ffi.lib()
    m, n, k = shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    if case == "prefill":
        x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
        w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda")
        s = (torch.rand((n, k // GROUP), device="cuda") * 0.019 + 0.001).to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

        def launch():
            ffi.check(L.vyb_k_int4_prefill_gemm(x.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(), m, n, k, GROUP,
                                                ffi.DT_BF16, stream, C.c_void_p(status.data_ptr())))
        unit, scale = "TFLOP/s", 1e12
    elif case == "moe":
        # --shape TOKENS INTER HIDDEN; 8 experts, top-2 (config 4 is --shape 4096 14336 4096)
        experts, topk = 8, 2
        tokens, inter, hidden = m, n, k
        x = torch.randn((tokens, hidden), device="cuda").to(torch.bfloat16)
        wr = (torch.randn((experts, hidden), device="cuda") * 0.02).to(torch.bfloat16)
        w13 = torch.randint(0, 256, (experts, 2, inter, hidden // 2), dtype=torch.uint8, device="cuda")
        s13 = (torch.rand((experts, 2, inter, hidden // GROUP), device="cuda") * 0.019 + 0.001).to(torch.bfloat16)
        w2 = torch.randint(0, 256, (experts, hidden, inter // 2), dtype=torch.uint8, device="cuda")
        s2 = (torch.rand((experts, hidden, inter // GROUP), device="cuda") * 0.019 + 0.001).to(torch.bfloat16)
        out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
        ridx = torch.empty((tokens, topk), dtype=torch.int32, device="cuda")
        rw = torch.empty((tokens, topk), dtype=torch.float32, device="cuda")
        need = C.c_uint64(0)
        ffi.check(L.vyb_k_moe_ffn_int4_scratch_bytes(tokens, hidden, inter, experts, topk, C.byref(need)))
        scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")

        def launch():
            ffi.check(L.vyb_k_moe_ffn_int4(x.data_ptr(), wr.data_ptr(), w13.data_ptr(), s13.data_ptr(), w2.data_ptr(),
                                           s2.data_ptr(), out.data_ptr(), ridx.data_ptr(), rw.data_ptr(),
                                           scratch.data_ptr(), need.value, tokens, hidden, inter, experts, topk, GROUP,
                                           stream, C.c_void_p(status.data_ptr())))
        unit, scale = "TFLOP/s", 1e12 / (3 * topk)  # 3 projections per (token, expert) pair: rate counts expert flops
    else:
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda")
        y = torch.empty((m, n), dtype=torch.int32, device="cuda")

        def launch():
            ffi.check(L.vyb_k_int8_gemm_i32(a.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, stream,
                                            C.c_void_p(status.data_ptr())))
        unit, scale = "TOP/s", 1e12
    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        launch()
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / max(1, steps)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    line = {"quick": True, "case": case, "shape": [m, n, k], "steps": steps, "us_per_launch": us,
            "rate": 2.0 * m * n * k / (us * 1e-6) / scale, "unit": unit}
    if case == "moe":
        line["tokens_per_s"] = m / (us * 1e-6)
    return line


def run_quick_gemm(args) -> None:
    """The cases profiled under ncu; one JSON line."""
    print(json.dumps(measure_case(args.case, args.shape, args.steps, args.warmup)))


def run_quick(args) -> None:
    """A few plain launches of the decode GEMV over rotating weight copies; prints one short JSON line."""
    import torch

    from vyre_b200 import ffi, synth

    if args.case != "gemv":
        return run_quick_gemm(args)
    L = ffi.lib()
    m = args.m
    x_np, w_np, s_np = synth.int4_linear_inputs(m, N_OUT, K_IN, seed=0)
    x = torch.from_numpy(x_np.view(np.int16)).cuda()
    copies = max(1, args.copies)
    ws = [torch.from_numpy(np.roll(w_np, c, axis=0)).cuda() for c in range(copies)]
    ss = [torch.from_numpy(np.roll(s_np, c, axis=0).view(np.int16)).cuda() for c in range(copies)]
    y = torch.zeros((m, N_OUT), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def launch(i: int):
        c = i % copies
        ffi.check(L.vyb_k_int4_gemv_ex(x.data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(), y.data_ptr(), m, N_OUT, K_IN,
                                       GROUP, ffi.DT_BF16, ffi.LAUNCH_CONSTANT_WEIGHTS, C.c_void_p(stream),
                                       C.c_void_p(status.data_ptr())))

    for i in range(args.warmup):
        launch(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        launch(i)
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / max(1, args.steps)
    assert status.cpu().tolist() == [0, 0, 0, 0]
    print(json.dumps({"quick": True, "m": m, "steps": args.steps, "copies": copies, "us_per_launch": us,
                      "gbs": algorithmic_bytes(m) / (us * 1e-6) / 1e9}))


def run_native(args) -> None:
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
    steps = max(COPIES, (args.steps // COPIES) * COPIES)
    warmup = max(3 * COPIES, ((args.warmup + COPIES - 1) // COPIES) * COPIES)

    # ---- resident inputs: COPIES distinct weight sets so that consecutive steps never hit L2 -------------------
    x_np, w_np, s_np = synth.int4_linear_inputs(m, N_OUT, K_IN, seed=rank)
    x = torch.from_numpy(x_np.view(np.int16)).cuda()
    ws, ss = [], []
    for c in range(COPIES):
        ws.append(torch.from_numpy(np.roll(w_np, c, axis=0)).cuda())
        ss.append(torch.from_numpy(np.roll(s_np, c, axis=0).view(np.int16)).cuda())
    y = torch.zeros((m, N_OUT), dtype=torch.bfloat16, device="cuda")
    # N > 1: the all-gather is this library's peer-store kernel over NVLink (symmetric memory), not NCCL
    pag = None
    if world > 1:
        from vyre_b200 import sharding

        pag = sharding.PeerAllGather(m, N_OUT)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()

    side = torch.cuda.Stream()
    # with a concurrent push kernel the GEMV leaves one SM free: sharing an SM with the weight stream (140 KB of bulk
    # copies in flight) made every memory access of the push wait microseconds
    gemv_flags = ffi.LAUNCH_CONSTANT_WEIGHTS | (ffi.LAUNCH_LEAVE_ONE_SM if world > 1 else 0)

    def launch(c: int, out=None):
        # weights are graph constants: the launch may overlap the tail of the previous one (see the header)
        ffi.check(L.vyb_k_int4_gemv_ex(x.data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(), (y if out is None else out).data_ptr(), m, N_OUT, K_IN,
                                       GROUP, ffi.DT_BF16, gemv_flags,
                                       C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

    with torch.cuda.stream(stream):
        for c in range(COPIES):  # first launches configure the kernel; must precede graph capture
            launch(c)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            if pag is None:
                for c in range(COPIES):
                    launch(c)
            else:
                # GEMV c writes this rank's slice of buffer half c % 2; a one-CTA push kernel on a side stream copies
                # it to every peer and signals them while GEMV c+1 already runs; GEMV c+2 (same half) waits for it.
                pushed = [None] * COPIES
                for c in range(COPIES):
                    half = c & 1
                    if c >= 2:
                        stream.wait_event(pushed[c - 2])
                    launch(c, pag.local_slice(half))
                    ready = torch.cuda.Event()
                    ready.record(stream)
                    side.wait_event(ready)
                    pag.push(half, side.cuda_stream, status)
                    pushed[c] = torch.cuda.Event()
                    pushed[c].record(side)
                stream.wait_stream(side)
                # the replay ends with the bounded wait for its own gathers: nothing is left in flight
                pag.wait(stream.cuda_stream, status)
    # parity guard inside the bench: the last copy's output must match the contract path bit for bit
    with torch.cuda.stream(stream):
        graph.replay()
    stream.synchronize()
    if pag is not None:
        # the gathered result of the graph's last step (odd step index: half 1) against NCCL's all-gather of the
        # plain kernel's output for the same weight copy
        launch(COPIES - 1)
        stream.synchronize()
        want_all = torch.empty((world, m, N_OUT), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(want_all.view(-1), y.view(-1))
        torch.cuda.synchronize()
        assert torch.equal(pag.halves()[1].view(torch.int16), want_all.view(torch.int16)), "peer-store all-gather differs from NCCL"
        y = pag.halves()[1][rank]
    y_ref = y.clone()

    for _ in range(warmup // COPIES):
        with torch.cuda.stream(stream):
            graph.replay()
    stream.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    # the barrier comes after the sampler's start-up so that every rank enters the timed region together
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    lo = sampler.mark()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(steps // COPIES):
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
    clocks = sampler.stop(lo, hi) if rank == 0 else None
    assert status.cpu().tolist() == [0, 0, 0, 0], "a bounded device-side wait ran out during the bench"
    assert torch.equal(y, y_ref), "non-deterministic GEMV output during the bench"

    ms_per_step = elapsed_ms / steps
    bytes_per_step = algorithmic_bytes(m)
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # All ranks leave the process group together, right after the timed region: the captured graph holds NCCL work
    # and must be gone before the communicator is; what follows on rank 0 is single-GPU work without collectives.
    if dist:
        del graph
        torch.cuda.synchronize()
        pag = None
        dist.barrier()
        dist.destroy_process_group()
        dist = None
    if rank != 0:
        return

    # ---- kernel-only time of the dominant kernel (no collective), for the roofline --------------------------------
    kgraph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(kgraph, stream=stream):
            for c in range(COPIES):
                launch(c)
    ksteps = min(steps, 40000)
    ks, ke = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(4):
            kgraph.replay()
        ks.record(stream)
        for _ in range(ksteps // COPIES):
            kgraph.replay()
        ke.record(stream)
    stream.synchronize()
    kernel_us = ks.elapsed_time(ke) * 1e3 / ksteps
    peak, peak_kind = measured_peaks()
    achieved = bytes_per_step / (kernel_us * 1e-6) / 1e9

    extra = {}
    for mm in (4, 8):
        xm_np, _, _ = synth.int4_linear_inputs(mm, 16, K_IN, seed=3)
        xm = torch.from_numpy(xm_np.view(np.int16)).cuda()
        ym = torch.zeros((mm, N_OUT), dtype=torch.bfloat16, device="cuda")
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g2, stream=stream):
                for c in range(COPIES):
                    ffi.check(L.vyb_k_int4_gemv_ex(xm.data_ptr(), ws[c].data_ptr(), ss[c].data_ptr(), ym.data_ptr(), mm,
                                                   N_OUT, K_IN, GROUP, ffi.DT_BF16, ffi.LAUNCH_CONSTANT_WEIGHTS,
                                                   C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))
            for _ in range(4):
                g2.replay()
            ks.record(stream)
            for _ in range(2000 // COPIES):
                g2.replay()
            ke.record(stream)
        stream.synchronize()
        us = ks.elapsed_time(ke) * 1e3 / (2000 // COPIES * COPIES)
        extra[f"m{mm}"] = {"us_per_launch": round(us, 3), "gbs": round(algorithmic_bytes(mm) / (us * 1e-6) / 1e9, 1),
                           "frac_of_measured_peak": round(algorithmic_bytes(mm) / (us * 1e-6) / 1e9 / peak, 4)}

    # ---- end to end through the contract path: host x -> submit -> wait -> host y, weights resident ---------------
    dev = vb.Device.acquire(local_rank)
    prog = vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, K_IN, N_OUT, GROUP, ffi.DT_BF16)
    sess = vb.ArtifactSession.compile(prog, dev)
    hw = [dev.resident_from(np.roll(w_np, c, axis=0).view(np.uint32)) for c in range(COPIES)]
    hs = [dev.resident_from(np.roll(s_np, c, axis=0)) for c in range(COPIES)]
    x_pinned = torch.from_numpy(x_np.view(np.int16).copy()).pin_memory().numpy().view(np.uint16)
    depth = 4
    e2e_steps = max(depth * COPIES, min(steps, 4000))

    # one prepared binding set per weight copy: the activation buffer is the same pinned array every step (a serving
    # loop rewrites it in place), so the sets are built once and only submitted in the timed loop
    sets = []
    for c in range(COPIES):
        bs = vb.BindingSet(sess.artifact.digest())
        bs.insert_host(0, x_pinned)
        bs.insert_resident(1, hw[c])
        bs.insert_resident(2, hs[c])
        sets.append(bs)

    def submit(i: int):
        return sess.submit(sets[i % COPIES])

    inflight, checksum, last = [], 0.0, None
    for i in range(depth * COPIES):  # warm-up
        submit(i).wait()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        inflight.append(submit(i))
        if len(inflight) == depth:
            last = inflight.pop(0).wait()
            checksum += float(last.output_view(3, np.uint16)[0])
    while inflight:
        last = inflight.pop(0).wait()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    got_last = np.frombuffer(last.output(3), np.uint16).reshape(m, N_OUT)
    want_last = y_ref.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got_last, want_last), "contract path and kernel-level path disagree"
    e2e = {"value": world * bytes_per_step / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(x_pinned.nbytes),
           "d2h_bytes_per_step": int(m * N_OUT * 2), "us_per_step": round(e2e_s * 1e6, 2), "in_flight": depth,
           "api": "ArtifactSession.submit/wait (vyb_submit, vyb_submission_wait), weights resident"}
    for h in hw + hs:
        dev.free_resident(h)
    dev.release()

    # ---- the other configurations of the path, kernel-level, a few launches each (reported beside the headline) -----
    secondary = {}
    try:
        bf16_peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        bf16_peak = 1590.0
    c3 = measure_case("prefill", [2048, 14336, 4096], 20, 5)
    secondary["int4_prefill_gemm_config3"] = {"tflops": round(c3["rate"], 1), "us_per_launch": round(c3["us_per_launch"], 1),
                                              "frac_of_bf16_burst_peak": round(c3["rate"] / bf16_peak, 3)}
    c5 = measure_case("int8gemm", [4096, 28672, 8192], 10, 3)
    secondary["int8_gemm_config5"] = {"tops": round(c5["rate"], 1), "us_per_launch": round(c5["us_per_launch"], 1),
                                      "frac_of_2x_bf16_burst_peak": round(c5["rate"] / (2 * bf16_peak), 3)}
    c4 = measure_case("moe", [4096, 14336, 4096], 5, 2)
    secondary["moe_ffn_config4"] = {"tokens_per_s": round(c4["tokens_per_s"]), "ms_per_layer": round(c4["us_per_launch"] / 1e3, 3),
                                    "expert_tflops": round(c4["rate"], 1)}
    torch.cuda.empty_cache()

    cpu_gbs, cpu_dt, cpu_sample, cpu_threads = cpu_reference_rate(m, budget_s=12.0)

    line = {
        "metric": "int4_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16xint4->f32", "data": "synthetic",
        "config": {"workload": f"int4 group-quantized decode GEMV M={m} N={N_OUT} K={K_IN} g={GROUP} (config 2)",
                   "per_gpu_shard": [N_OUT, K_IN], "parallelism": f"column-parallel x{world}" + (" + peer-store all-gather over NVLink on a side stream" if world > 1 else ""),
                   "l2_policy": f"inputs larger than L2: {COPIES} rotating weight copies = {COPIES * (N_OUT * K_IN // 2) / 1e6:.0f} MB",
                   "launch": f"CUDA graph of {COPIES} launches, programmatic dependent launch (constant weights)"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(m), "peak_kind": f"of {peak_kind}", "kernel": "int4_gemv_kernel",
                     "us_per_launch": round(kernel_us, 3), "algorithmic_bytes_per_launch": bytes_per_step,
                     "frac_of_nominal_8tbs": achieved / 8000.0},
        "cpu_baseline": {"value": cpu_gbs, "unit": "GB/s", "cores": cpu_threads, "kind": "port", "sample": cpu_sample,
                         "ms_per_gemv": round(cpu_dt * 1e3, 2)},
        "e2e": e2e, "gpu_launches": steps * (2 if world > 1 else 1) + (steps // COPIES if world > 1 else 0), "clocks": clocks, "other_batches": extra, "secondary": secondary,
    }
    print(json.dumps(line))


def run_moe_ep(args) -> None:
    """Config 4 across the ranks: 4096 tokens in total (strong scaling), 8 experts top-2 split expert-parallel, two
    all-to-all exchanges per layer. A step is one layer over every rank's tokens; value = tokens / s over all ranks.
    The timed region holds everything a caller of the layer pays: routing, the host-side exchange plan (one
    device-to-host read of the routing indices), both exchanges, grouped GEMMs and the combine."""
    import torch

    from vyre_b200 import sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    import torch.distributed as dist

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    tokens_total, inter, hidden = args.shape
    experts, topk = 8, 2
    local = experts // world
    tokens = tokens_total // world
    torch.manual_seed(1234 + rank)
    x = torch.randn((tokens, hidden), device="cuda").to(torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(7)  # the router is replicated: same values on every rank
    wr = (torch.randn((experts, hidden), device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    w13 = torch.randint(0, 256, (local, 2, inter, hidden // 2), dtype=torch.uint8, device="cuda")
    s13 = (torch.rand((local, 2, inter, hidden // GROUP), device="cuda") * 0.019 + 0.001).to(torch.bfloat16)
    w2 = torch.randint(0, 256, (local, hidden, inter // 2), dtype=torch.uint8, device="cuda")
    s2 = (torch.rand((local, hidden, inter // GROUP), device="cuda") * 0.019 + 0.001).to(torch.bfloat16)
    if args.ep == "host":
        # exchange planned on the host (one read-back of the routing), rows moved by NCCL all-to-all
        ops = sharding.KernelOps(w13, s13, w2, s2, hidden, inter, local, GROUP)
        max_rows = ((tokens_total * topk + 255) // 256) * 256 + local * 256  # worst case: every pair lands on this rank

        def step():
            return sharding.expert_parallel_moe_ffn(x, wr, ops, experts, topk, max_rows=max_rows)
    else:
        # dispatch and combine by the library's own kernels over peer memory, nothing read back by the host
        ops = sharding.DeviceExpertParallel(wr, w13, s13, w2, s2, hidden, inter, experts, topk, tokens_local_max=tokens,
                                            tokens_total=tokens_total, group_size=GROUP)

        def step():
            return ops.forward(x)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    steps = max(1, args.steps)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    assert ops.status.cpu().tolist() == [0, 0, 0, 0]
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        flops = 2.0 * tokens_total * topk * 3 * inter * hidden
        print(json.dumps({
            "metric": "moe_ffn_tokens_per_s", "value": tokens_total / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16xint4->f32", "data": "synthetic",
            "config": {"workload": f"int4 MoE FFN layer, {tokens_total} tokens, hidden {hidden}, inter {inter}, {experts} experts "
                                   f"top-{topk} (config 4)", "parallelism": f"expert-parallel x{world}, " + ("host-planned NCCL all-to-all" if args.ep == "host" else "device-side dispatch/combine over peer memory (NVLink)"),
                       "tokens_per_rank": tokens, "experts_per_rank": local},
            "expert_tflops": flops / (ms * 1e-3) / 1e12}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100000)
    ap.add_argument("--warmup", type=int, default=2000)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--m", type=int, default=1, help="decode batch (1, 4 or 8)")
    ap.add_argument("--case", default="gemv", choices=["gemv", "prefill", "int8gemm", "moe"],
                    help="kernel exercised by --quick")
    ap.add_argument("--shape", type=int, nargs=3, default=[2048, 14336, 4096], metavar=("M", "N", "K"),
                    help="GEMM shape for --quick --case prefill|int8gemm")
    ap.add_argument("--copies", type=int, default=COPIES,
                    help="weight copies rotated in --quick mode (1 keeps the weights L2-resident: compute-bound check)")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "moe"],
                    help="gemv: the headline decode GEMV; moe: the expert-parallel MoE FFN layer (--shape TOKENS INTER HIDDEN)")
    ap.add_argument("--ep", default="device", choices=["device", "host"],
                    help="--workload moe: device-side dispatch/combine over peer memory, or host-planned NCCL all-to-all")
    ap.add_argument("--quick", action="store_true",
                    help="kernel-only run without graphs, end-to-end leg or CPU baseline (the case profiled under ncu)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.quick:
        run_quick(args)
    elif args.workload == "moe":
        if args.shape == [2048, 14336, 4096]:
            args.shape = [4096, 14336, 4096]
        if args.steps == 100000:
            args.steps, args.warmup = 20, 3
        run_moe_ep(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
