#!/usr/bin/env python
"""Benchmark of the quantization-simulation hot path on B200.

Headline workload (benchmark configuration 3): TF-Enhanced encoding calibration of one quantizer -- per batch a
512-bucket histogram of fp32 activations [64, 256, 28, 28] (ReLU(N(0,1)) with 0.1 % outliers x20), then the
running-PDF replay and the SQNR grid search for an 8-bit asymmetric encoding.  A step is one batch.  With N GPUs
every rank calibrates its own K batches (batch b of the job belongs to rank b % N) and the ranks exchange the
per-batch histogram table once (NCCL all-reduce) before the search: weak scaling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Prints ONE JSON line.  `value` is whole-job samples/s with the batches resident in HBM; `e2e` is the same job fed
from pinned host memory through AimetTensorQuantizer.updateStats / getEncoding; `roofline` is the histogram kernel
against the measured HBM copy bandwidth; `cpu_baseline` is the reference's own CPU code on one host core.
`--impl reference` times that CPU code alone.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH_SHAPE = (64, 256, 28, 28)
SAMPLES_PER_BATCH = BATCH_SHAPE[0]
N_EL = 64 * 256 * 28 * 28
BATCH_BYTES = 4 * N_EL
MAX_DISTINCT = 256            # distinct device batches kept per GPU (13.2 GB); more steps cycle through them
METRIC = "TF-Enhanced calibration throughput (512-bin histogram + SQNR search)"
WORKLOAD = ("configuration 3: TF-Enhanced calibration, fp32 activations [64,256,28,28] = ReLU(N(0,1)) with 0.1% "
            "outliers x20, 8-bit asymmetric, 512 buckets")
# dram__bytes_read+write per algorithmic byte of the histogram kernel, from the ncu capture summarised in
# profiles/tfe_hist_lane_kernel_relu_256MB.md (captured on a 256 MB input; traffic grows in proportion)
HIST_TRAFFIC_RATIO = 1.024


def peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def host_batch(b: int):
    """Batch b of the calibration set on the host (numpy; used by the CPU arms)."""
    import numpy as np
    rng = np.random.default_rng(1000 + b)
    a = np.maximum(rng.standard_normal(N_EL, dtype=np.float32), 0)
    a[rng.random(N_EL, dtype=np.float32) < 1e-3] *= 20
    return a


def device_batch(b: int, device):
    """Batch b of the calibration set generated on the device (same distribution; own seed per batch)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(1000 + b)
    a = torch.relu(torch.randn(N_EL, device=device, generator=g))
    m = torch.rand(N_EL, device=device, generator=g) < 1e-3
    return torch.where(m, a * 20, a).view(BATCH_SHAPE)


# ---------------------------------------------------------------------------------------------------------------------
# CPU arms (reference code on the host cores)
# ---------------------------------------------------------------------------------------------------------------------
def cpu_calibration(num_batches: int, distinct: int = 4):
    """Times the reference's TF-Enhanced updateStats/computeEncoding on `num_batches` batches (single thread: the
    reference's loops are scalar and serial).  Returns (seconds, kind)."""
    from oracle import Oracle, OracleTfeAnalyzer, RefAnalyzer, Reference
    data = [host_batch(b) for b in range(min(distinct, num_batches))]
    if Reference.available():
        an, kind = RefAnalyzer(Reference(), "tfe"), "reference"
    else:
        an, kind = OracleTfeAnalyzer(Oracle()), "port"
    an.update(data[0][:4096])            # warm-up (page in the library), then a fresh analyzer
    an = RefAnalyzer(Reference(), "tfe") if kind == "reference" else OracleTfeAnalyzer(Oracle())
    t0 = time.perf_counter()
    for b in range(num_batches):
        an.update(data[b % len(data)])
    an.compute(8, False, False, False)
    return time.perf_counter() - t0, kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # warm-up steps, then K timed steps; one step = one full batch through the reference's CPU code
    cpu_calibration(min(args.warmup, 1), 1)
    secs, kind = cpu_calibration(args.steps)
    value = args.steps * SAMPLES_PER_BATCH / secs
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_shape": list(BATCH_SHAPE), "batches": args.steps,
                   "note": "reference DlQuantization TfEnhancedEncodingAnalyzer on the host, rank 0 only"},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": 1, "kind": kind,
                         "sample": f"{args.steps} batches of [64,256,28,28] (4 distinct, cycled) + computeEncoding"},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the benchmark runs (read-only)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self.ok = index, [], set(), None, False
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        while self.ok and not self._stop_evt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        s = sorted(self.samples)
        # samples under load: the upper half (idle samples between phases sit at the idle clock)
        busy = s[len(s) // 2:] if s else []
        return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
def run_b200(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from aimet_b200 import _lib, libpymo
    from aimet_b200._lib import lib
    from aimet_b200.calibration import TfEnhancedCalibrator

    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(local)
    sampler.start()

    # ---- data: this rank's batches (global batch index k * world + rank), resident in HBM -----------------------
    distinct = min(max(K, 4), MAX_DISTINCT)   # at least 4 x 51 MB, so that the rotating inputs exceed the 126 MB L2
    batches = [device_batch(k * world + rank, device) for k in range(distinct)]
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def calibrate(steps):
        cal = TfEnhancedCalibrator(device)
        for k in range(steps):
            cal.update(batches[k % distinct])
        return cal.compute_encoding(8, False, False, False)

    # ---- warm-up, then the timed job ------------------------------------------------------------------------------
    calibrate(W)
    barrier()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    enc = calibrate(K)
    e1.record()
    barrier()
    launches = _lib.launch_count() - launches0
    secs = e0.elapsed_time(e1) * 1e-3
    if world > 1:
        t = torch.tensor([secs], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t)
    value = world * K * SAMPLES_PER_BATCH / secs

    # ---- roofline of the dominant kernel: K back-to-back histogram launches through the raw C ABI ------------------
    from aimet_b200 import ops
    st = ops.TfeDeviceState(device, capacity=distinct)
    st.init_grid_from(ops.minmax(batches[0]).reshape(-1))
    stream = torch.cuda.current_stream().cuda_stream
    ptrs = [b.data_ptr() for b in batches]
    hp, cp, sp = st.hists.data_ptr(), st.counts.data_ptr(), st.state.data_ptr()
    reps = max(K, 64)
    for i in range(3):
        lib.aq_tfe_histogram(ptrs[i % distinct], N_EL, sp, hp + 2048 * (i % distinct), cp + 8 * (i % distinct), stream)
    torch.cuda.synchronize()
    e0.record()
    for i in range(reps):
        j = i % distinct
        lib.aq_tfe_histogram(ptrs[j], N_EL, sp, hp + 2048 * j, cp + 8 * j, stream)
    e1.record()
    torch.cuda.synchronize()
    kernel_s = e0.elapsed_time(e1) * 1e-3 / reps
    peak, peak_kind = peak_hbm()
    achieved = BATCH_BYTES / kernel_s / 1e9

    # ---- end to end: batches start in pinned host memory; H2D copy, updateStats, and a D2H read every step ---------
    ring = [torch.empty(BATCH_SHAPE, dtype=torch.float32).pin_memory() for _ in range(4)]
    for i, r in enumerate(ring):
        r.copy_(batches[i % distinct])
    dev_buf = [torch.empty(BATCH_SHAPE, dtype=torch.float32, device=device) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    host_counts = torch.zeros(2, dtype=torch.int64).pin_memory()

    def e2e_job(steps):
        q = libpymo.AimetTensorQuantizer(libpymo.QUANTIZATION_TF_ENHANCED)
        main = torch.cuda.current_stream()
        for k in range(steps):
            s = k % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[s])
                dev_buf[s].copy_(ring[k % len(ring)], non_blocking=True)
                copied[s].record(copy_stream)
            main.wait_event(copied[s])
            q.updateStats(dev_buf[s], True)
            consumed[s].record(main)
            # per-step device->host read of the step's result (the batch's sample count)
            host_counts[s:s + 1].copy_(q._stats.dev.counts[k:k + 1], non_blocking=True)
        return q.getEncoding(8, False, False, False)

    for ev in consumed:
        ev.record(torch.cuda.current_stream())
    e2e_job(W)
    barrier()
    e0.record()
    e2e_job(K)
    e1.record()
    barrier()
    e2e_secs = e0.elapsed_time(e1) * 1e-3
    if world > 1:
        t = torch.tensor([e2e_secs], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs = float(t)
    e2e_value = world * K * SAMPLES_PER_BATCH / e2e_secs

    # ---- secondary numbers: fake-quant forward / backward kernels (reported, not the headline) ---------------------
    qdq = qdq_numbers(torch, lib, device, peak) if (rank == 0 and not args.skip_qdq) else None
    clocks = sampler.stop()

    # ---- CPU baseline: the reference's own code on one host core, bounded sample (rank 0, N = 1 only) -------------
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        nb = 200
        cs, kind = cpu_calibration(nb)
        cpu = {"value": nb * SAMPLES_PER_BATCH / cs, "unit": "samples/s", "cores": 1, "kind": kind,
               "sample": f"{nb} batches of [64,256,28,28] (4 distinct, cycled) + computeEncoding, {cs:.1f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_shape": list(BATCH_SHAPE), "batches_per_gpu": K,
                       "batches_total": K * world, "parallelism": f"batch-sharded x{world}, histogram-table all-reduce",
                       "l2": f"inputs larger than L2: {distinct} distinct batches x 51.4 MB per GPU",
                       "timed_region": "K x update (histogram kernel; first batch also min/max + grid) + exchange + "
                                       "PDF replay + SQNR search + encoding read-back",
                       "encoding": [enc.min, enc.max, enc.delta, enc.offset, enc.bw]},
            "roofline": {"bound": "hbm", "kernel": "tfe_hist_lane_kernel", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": HIST_TRAFFIC_RATIO * BATCH_BYTES, "bytes_per_launch": BATCH_BYTES,
                         "us_per_launch": kernel_s * 1e6},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": BATCH_BYTES, "d2h_bytes_per_step": 8,
                    "ms_per_step": e2e_secs / K * 1e3, "api": "AimetTensorQuantizer.updateStats / getEncoding"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if qdq is not None:
            line["qdq"] = qdq
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def qdq_numbers(torch, lib, device, peak):
    """Fake-quant kernels at the shapes of benchmark configurations 1, 2 and 5, raw C-ABI launches over rotating buffers
    larger than L2, CUDA-event timed."""
    stream = torch.cuda.current_stream().cuda_stream
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(calls, reps):
        for c in calls[:3]:
            c()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            for c in calls:
                c()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / (reps * len(calls))

    out = {}
    # config 1: [32,64,56,56] fp32 per-tensor 8-bit asymmetric
    n1, nb = 32 * 64 * 56 * 56, 12
    xs = [torch.randn(n1, device=device) for _ in range(nb)]
    ys = [torch.empty(n1, device=device) for _ in range(nb)]
    ms = [torch.empty(n1, dtype=torch.uint8, device=device) for _ in range(nb)]
    sc, of = torch.tensor([0.0353], device=device), torch.tensor([-128.0], device=device)
    P = lambda t: t.data_ptr()

    def rec(name, bytes_, secs):
        out[name] = {"us": secs * 1e6, "GBps": bytes_ / secs / 1e9, "frac": bytes_ / secs / 1e9 / peak}

    rec("c1_v2_qdq_fwd_8B", 8 * n1, timed([lambda i=i: lib.aq_v2_quantize(P(xs[i]), P(ys[i]), None, 0, n1, 1, n1, P(sc), P(of), 0.0, 255.0, 0, 0, stream) for i in range(nb)], 4))
    rec("c1_v2_qdq_fwd_mask_9B", 9 * n1, timed([lambda i=i: lib.aq_v2_quantize(P(xs[i]), P(ys[i]), P(ms[i]), 0, n1, 1, n1, P(sc), P(of), 0.0, 255.0, 0, 0, stream) for i in range(nb)], 4))
    rec("c1_v2_qdq_bwd_9B", 9 * n1, timed([lambda i=i: lib.aq_v2_qdq_backward(P(xs[i]), P(ms[i]), P(ys[i]), 0, n1, stream) for i in range(nb)], 4))
    rec("c1_libpymo_qdq_fwd_8B", 8 * n1, timed([lambda i=i: lib.aq_qdq_per_tensor(P(xs[i]), P(ys[i]), n1, -4.4, 4.6, 8, 0, stream) for i in range(nb)], 4))
    emn, emx = torch.tensor([-4.4], device=device), torch.tensor([4.6], device=device)
    rec("c1_v1_ste_bwd_12B", 12 * n1, timed([lambda i=i: lib.aq_ste_backward_v1(P(xs[i]), P(xs[(i + 1) % nb]), P(ys[i]), n1, 1, n1, P(emn), P(emx), stream) for i in range(nb)], 4))
    mm = torch.empty(2, device=device)
    ws = torch.zeros(int(lib.aq_minmax_workspace_bytes(n1, 1, n1)), dtype=torch.uint8, device=device)
    rec("c1_minmax_4B", 4 * n1, timed([lambda i=i: lib.aq_minmax(P(xs[i]), 0, n1, 1, n1, P(mm[0:1]), P(mm[1:2]), 0, 0, P(ws), ws.numel(), stream) for i in range(nb)], 4))
    del xs, ys, ms
    # config 2: [512,256,3,3] fp32 per-output-channel 8-bit symmetric (launch-latency bound: 9.4 MB per launch);
    # timed launch by launch and, without the per-launch CPU cost, as one CUDA graph of all the launches
    n2, kb = 512 * 2304, 64
    w = [torch.randn(n2, device=device) * 0.03 for _ in range(kb)]
    wo = [torch.empty(n2, device=device) for _ in range(kb)]
    s2, o2 = torch.full((512,), 1e-3, device=device), torch.zeros(512, device=device)
    c2 = lambda st: [lambda i=i: lib.aq_v2_quantize(P(w[i]), P(wo[i]), None, 0, n2, 512, 2304, P(s2), P(o2), -128.0, 127.0, 0, 0, st) for i in range(kb)]
    rec("c2_v2_qdq_fwd_per_channel_8B", 8 * n2, timed(c2(stream), 3))
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for c in c2(side.cuda_stream):
            c()
    torch.cuda.current_stream().wait_stream(side)
    rec("c2_v2_qdq_fwd_per_channel_8B_graph", 8 * n2, timed([graph.replay], 6) / kb)
    del w, wo, graph
    # config 5: bf16 weight [4096,11008], W4 symmetric, block 64 on the input dim
    n5 = 4096 * 11008
    wh = [(torch.randn(n5, device=device) * 0.02).to(torch.bfloat16) for _ in range(4)]
    wq = [torch.empty_like(t) for t in wh]
    nch = n5 // 64
    s5, o5 = torch.full((nch,), 0.004, device=device), torch.zeros(nch, device=device)
    rec("c5_v2_qdq_fwd_bf16_block64_4B", 4 * n5 + 8 * nch, timed([lambda i=i: lib.aq_v2_quantize(P(wh[i]), P(wq[i]), None, 2, n5, nch, 64, P(s5), P(o5), -8.0, 7.0, 0, 0, stream) for i in range(4)], 4))
    s1, o1 = torch.full((1,), 4e-4, device=device), torch.zeros(1, device=device)
    rec("c5_v2_qdq_fwd_bf16_per_tensor_4B", 4 * n5, timed([lambda i=i: lib.aq_v2_quantize(P(wh[i]), P(wq[i]), None, 2, n5, 1, n5, P(s1), P(o1), -32768.0, 32767.0, 0, 0, stream) for i in range(4)], 4))
    bm = torch.empty((2, nch), device=device)
    rec("c5_minmax_bf16_block64_2B", 2 * n5 + 8 * nch, timed([lambda i=i: lib.aq_minmax(P(wh[i]), 2, n5, nch, 64, P(bm[0]), P(bm[1]), 0, 0, P(ws), ws.numel(), stream) for i in range(4)], 4))
    return out


# ---------------------------------------------------------------------------------------------------------------------
# single-kernel cases (micro-benchmarks; also the small commands the ncu captures under profiles/ were taken with)
# ---------------------------------------------------------------------------------------------------------------------
KERNEL_CASES = ("tfe_hist", "minmax_f32", "minmax_f32_rows", "minmax_bf16_block64", "v2_qdq_f32", "v2_qdq_f32_mask",
                "v2_qdq_f32_per_channel", "v2_qdq_bf16", "v2_qdq_bf16_block64", "v2_bwd_f32", "v2_bwd_bf16",
                "pymo_qdq_f32", "pymo_qdq_f32_per_channel", "ste_v1_f32", "tfe_replay", "tfe_search")


def build_kernel_case(name, mb, torch, lib, device):
    """Returns (calls, algorithmic bytes per launch): `calls` launch the named kernel through the C ABI on rotating
    inputs of `mb` MB each whose total exceeds the L2 capacity."""
    from aimet_b200 import ops
    stream = torch.cuda.current_stream().cuda_stream
    half = "bf16" in name
    esz = 2 if half else 4
    n = (mb << 20) // esz // 2304 * 2304          # multiple of 2304 = 36 * 64: rows of 2304 and blocks of 64 both fit
    nbuf = max(2, -(-320 // mb))                  # rotating set larger than L2 (126 MB)
    dt = 2 if half else 0
    P = lambda t: t.data_ptr()

    def data(kind="normal"):
        g = torch.Generator(device=device)
        out = []
        for b in range(nbuf):
            g.manual_seed(77 + b)
            a = torch.randn(n, device=device, generator=g)
            if kind == "relu_outliers":
                a = torch.relu(a)
                a = torch.where(torch.rand(n, device=device, generator=g) < 1e-3, a * 20, a)
            out.append((a * (0.02 if half else 1.0)).to(torch.bfloat16 if half else torch.float32))
        return out

    if name in ("tfe_replay", "tfe_search"):
        # the tail of a calibration: running-mean replay over `mb` x 8 per-batch rows (2048 at the default), SQNR search
        rows = mb * 8
        g = torch.Generator(device=device)
        g.manual_seed(5)
        x = torch.relu(torch.randn(1 << 22, device=device, generator=g))
        st = ops.TfeDeviceState(device, capacity=rows)
        st.init_grid_from(ops.minmax(x).reshape(-1))
        for r in range(rows):
            st.add_batch(x[(r % 8) * 4096:(r % 8) * 4096 + (1 << 19)], r)
        st.replay()
        ws = ops.workspace(st.state, int(lib.aq_tfe_search_workspace_bytes()))
        if name == "tfe_replay":
            calls = [lambda: lib.aq_tfe_pdf_replay(P(st.hists), P(st.counts), rows, P(st.pdf), P(st.iterations), stream)]
            return calls, rows * (2048 + 8) + 4096, [st, x]
        calls = [lambda: lib.aq_tfe_search(P(st.state), P(st.pdf), 1, 8, 0, 0, 0, P(st.encoding), P(ws), ws.numel(), stream)]
        return calls, 2 * 512 * 8, [st, x, ws]
    xs = data("relu_outliers" if name == "tfe_hist" else "normal")
    if name == "tfe_hist":
        st = ops.TfeDeviceState(device, capacity=nbuf)
        st.init_grid_from(ops.minmax(xs[0]).reshape(-1))
        hp, cp, sp = P(st.hists), P(st.counts), P(st.state)
        keep = [st]
        calls = [lambda i=i: lib.aq_tfe_histogram(P(xs[i]), n, sp, hp + 2048 * i, cp + 8 * i, stream) for i in range(nbuf)]
        return calls, 4 * n, keep + xs
    if name.startswith("minmax"):
        num_ch, inner = {"minmax_f32": (1, n), "minmax_f32_rows": (n // 2304, 2304), "minmax_bf16_block64": (n // 64, 64)}[name]
        need = int(lib.aq_minmax_workspace_bytes(n, num_ch, inner))
        ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=device)
        o = torch.empty((2, num_ch), dtype=torch.float32, device=device)
        calls = [lambda i=i: lib.aq_minmax(P(xs[i]), dt, n, num_ch, inner, P(o[0]), P(o[1]), 0, 0, P(ws), ws.numel(), stream)
                 for i in range(nbuf)]
        return calls, esz * n + 8 * num_ch, [ws, o] + xs
    ys = [torch.empty_like(x) for x in xs]
    if name.startswith("v2_bwd"):
        ms = [(torch.rand(n, device=device) < 0.97).to(torch.uint8) for _ in range(nbuf)]
        calls = [lambda i=i: lib.aq_v2_qdq_backward(P(xs[i]), P(ms[i]), P(ys[i]), dt, n, stream) for i in range(nbuf)]
        return calls, (2 * esz + 1) * n, [ms, ys] + xs
    if name.startswith("v2_qdq"):
        if name.endswith("block64"):
            num_ch, inner, qmin, qmax, sc = n // 64, 64, -8.0, 7.0, 0.004
        elif name.endswith("per_channel"):
            num_ch, inner, qmin, qmax, sc = n // 2304, 2304, -128.0, 127.0, 0.03
        else:
            num_ch, inner, qmin, qmax, sc = 1, n, (-128.0 if half else 0.0), (127.0 if half else 255.0), (4e-4 if half else 0.0353)
        s = torch.full((num_ch,), sc, device=device)
        o = torch.full((num_ch,), 0.0 if qmin < 0 else -128.0, device=device)
        ms = [torch.empty(n, dtype=torch.uint8, device=device) for _ in range(nbuf)] if name.endswith("mask") else None
        calls = [lambda i=i: lib.aq_v2_quantize(P(xs[i]), P(ys[i]), P(ms[i]) if ms else None, dt, n, num_ch, inner, P(s), P(o),
                                                qmin, qmax, 0, 0, stream) for i in range(nbuf)]
        return calls, (2 * esz + (1 if ms else 0)) * n + (8 * num_ch if num_ch > 1 else 0), [s, o, ms, ys] + xs
    if name == "pymo_qdq_f32":
        calls = [lambda i=i: lib.aq_qdq_per_tensor(P(xs[i]), P(ys[i]), n, -4.4, 4.6, 8, 0, stream) for i in range(nbuf)]
        return calls, 8 * n, [ys] + xs
    num_ch, inner = n // 2304, 2304
    # encodings as a calibration produces them: min and max are multiples of the step, so clamped values land on a
    # grid point (with arbitrary bounds every clamped value sits on a rounding boundary and takes the exact path)
    step = 4.0 / 255.0
    emn, emx = torch.full((num_ch,), -128 * step, device=device), torch.full((num_ch,), 127 * step, device=device)
    if name == "pymo_qdq_f32_per_channel":
        calls = [lambda i=i: lib.aq_qdq_per_channel(P(xs[i]), P(ys[i]), n, num_ch, inner, P(emn), P(emx), 255.0, 0, stream)
                 for i in range(nbuf)]
        return calls, 8 * n + 8 * num_ch, [emn, emx, ys] + xs
    if name == "ste_v1_f32":
        gs = [torch.randn(n, device=device) for _ in range(nbuf)]
        calls = [lambda i=i: lib.aq_ste_backward_v1(P(xs[i]), P(gs[i]), P(ys[i]), n, 1, n, P(emn), P(emx), stream)
                 for i in range(nbuf)]
        return calls, 12 * n, [emn, emx, gs, ys] + xs
    raise SystemExit(f"unknown kernel case {name}")


def run_kernel_case(args):
    """`--kernel-case NAME --mb M --steps K --warmup W`: W + K launches of one kernel, one JSON line."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
    from aimet_b200._lib import lib
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    calls, nbytes, keep = build_kernel_case(args.kernel_case, args.mb, torch, lib, device)
    W, K = max(args.warmup, 3), args.steps
    for i in range(W):
        rc = calls[i % len(calls)]()
        assert rc == 0, rc
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        calls[i % len(calls)]()
    e1.record()
    torch.cuda.synchronize()
    secs = e0.elapsed_time(e1) * 1e-3 / K
    peak, peak_kind = peak_hbm()
    print(json.dumps({"kernel_case": args.kernel_case, "mb_per_input": args.mb, "inputs_rotated": len(calls), "steps": K,
                      "warmup": W, "us_per_launch": secs * 1e6, "bytes_per_launch": nbytes,
                      "achieved_GBps": nbytes / secs / 1e9, "peak_GBps": peak, "peak_kind": peak_kind,
                      "frac": nbytes / secs / 1e9 / peak}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg")
    ap.add_argument("--skip-qdq", action="store_true", help="omit the secondary fake-quant kernel numbers")
    ap.add_argument("--kernel-case", choices=KERNEL_CASES, help="time one kernel alone instead of the calibration job")
    ap.add_argument("--mb", type=int, default=256, help="input size in MB for --kernel-case")
    ap.add_argument("--model-case", choices=("resnet50", "llama_layer"),
                    help="whole-model calibration / fake-quant measurement instead of the calibration job")
    ap.add_argument("--batches", type=int, default=32, help="calibration batches for --model-case resnet50")
    ap.add_argument("--batch-size", type=int, default=128, help="batch size for --model-case resnet50")
    args = ap.parse_args()
    if args.model_case:
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
        from aimet_b200.v2 import model_cases
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        kw = {"batches": args.batches, "batch_size": args.batch_size} if args.model_case == "resnet50" else {}
        print(json.dumps(model_cases.CASES[args.model_case](dev, **kw)), flush=True)
    elif args.kernel_case:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
