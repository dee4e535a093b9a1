#!/usr/bin/env python
"""Benchmark of the quantization-simulation hot path on B200.

Headline workload (benchmark configuration 3): TF-Enhanced encoding calibration of one quantizer over 256 batches of
fp32 activations [64, 256, 28, 28] (ReLU(N(0,1)) with 0.1 % outliers x20): per batch a 512-bucket histogram, then the
running-PDF replay and the SQNR grid search for an 8-bit asymmetric encoding.

A STEP is one whole calibration job.  `--steps K` times K jobs back to back; the K-job block is repeated until at
least half a second has been timed and the median block is reported.  With N GPUs every rank calibrates 256 batches
of its own per job (batch b of the N x 256 belongs to rank b % N) and the ranks exchange the per-batch histogram
table once per job (one NCCL all-reduce) before the search: weak scaling, `value`.  The same run also times
configuration 3 itself split over the N ranks (256 batches in total, 256 / N per rank: strong scaling, key `strong`)
and checks, outside the timed regions, that the N-rank result equals a single-process run over the same batches bit
for bit (`parity_multi_gpu`).

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
JOB_BATCHES = 256             # batches of one calibration job per GPU (configuration 3; 13.2 GB resident)
METRIC = "TF-Enhanced calibration throughput (512-bin histogram + SQNR search)"
WORKLOAD = ("configuration 3: TF-Enhanced calibration, 256 batches of fp32 activations [64,256,28,28] = ReLU(N(0,1)) "
            "with 0.1% outliers x20, 8-bit asymmetric, 512 buckets")
# dram__bytes_read+write per algorithmic byte of the histogram kernel, from an ncu capture of a 16-batch launch on
# 49 MB batches (846.3 MB of traffic for 822.1 MB of input; traffic grows in proportion to the input)
HIST_TRAFFIC_RATIO = 1.030
MIN_TIMED_S = 0.5


def peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def job_config(n_gpus: int):
    """`config` of the JSON line; both arms print exactly this."""
    return {"workload": WORKLOAD, "batch_shape": list(BATCH_SHAPE), "step": "one calibration job",
            "batches_per_job_per_gpu": JOB_BATCHES, "batches_per_job": JOB_BATCHES * n_gpus,
            "samples_per_step": JOB_BATCHES * n_gpus * SAMPLES_PER_BATCH,
            "parallelism": f"batch-sharded x{n_gpus}, one histogram-table all-reduce per job" if n_gpus > 1
            else "single GPU",
            "l2": f"inputs larger than L2: {JOB_BATCHES} distinct batches x 51.4 MB per GPU"}


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


def median_spread(xs):
    s = sorted(xs)
    return s[len(s) // 2], s[0], s[-1]


# ---------------------------------------------------------------------------------------------------------------------
# CPU arms (reference code on the host cores)
# ---------------------------------------------------------------------------------------------------------------------
def cpu_calibration(num_batches: int, data):
    """Times the reference's TF-Enhanced updateStats/computeEncoding on `num_batches` batches cycled from `data`
    (single thread: the reference's loops are scalar and serial).  Returns (seconds, kind)."""
    from oracle import Oracle, OracleTfeAnalyzer, RefAnalyzer, Reference
    kind = "reference" if Reference.available() else "port"
    an = RefAnalyzer(Reference(), "tfe") if kind == "reference" else OracleTfeAnalyzer(Oracle())
    t0 = time.perf_counter()
    for b in range(num_batches):
        an.update(data[b % len(data)])
    an.compute(8, False, False, False)
    return time.perf_counter() - t0, kind


CPU_SAMPLE_BATCHES = 8   # batches of the job that one CPU step really runs (about a quarter of a second)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # A step is a bounded sample of the job: the first CPU_SAMPLE_BATCHES batches through updateStats, then
    # computeEncoding.  The reference's per-batch cost does not depend on how many batches came before, so
    # samples/s of the sample is samples/s of the whole job.
    data = [host_batch(b) for b in range(4)]
    for _ in range(max(args.warmup, 1)):
        cpu_calibration(1, data)
    times = []
    kind = "port"
    for _ in range(args.steps):
        secs, kind = cpu_calibration(CPU_SAMPLE_BATCHES, data)
        times.append(secs)
    total = sum(times)
    value = args.steps * CPU_SAMPLE_BATCHES * SAMPLES_PER_BATCH / total
    sample = (f"each step = the first {CPU_SAMPLE_BATCHES} of the job's {JOB_BATCHES} batches [64,256,28,28] (4 distinct, "
              f"cycled) + computeEncoding; {args.steps} steps, {total:.1f} s")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3 * (JOB_BATCHES * args.gpus / CPU_SAMPLE_BATCHES),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": job_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": 1, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "notes": "reference DlQuantization TfEnhancedEncodingAnalyzer on one host core (its loops are scalar and "
                 "serial), rank 0 only; ms_per_step is the sampled rate scaled to a whole job",
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
        self.loaded = []          # samples taken while `busy` was set (inside a timed region)
        self.busy = False
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
                mhz = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                self.samples.append(mhz)
                if self.busy:
                    self.loaded.append(mhz)
                    r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                    for bit, name in self.REASONS.items():
                        if r & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        s = sorted(self.loaded)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples), "samples_under_load": len(s)}


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
def gpu_numa_setup(local: int):
    """Best effort: run this rank on the CPUs of its GPU's NUMA node, so that the pinned staging buffers it
    allocates afterwards are local to the GPU's PCIe root.  Returns a short description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        path = f"/sys/bus/pci/devices/{bus[-12:].lower()}/numa_node"
        node = int(open(path).read()) if os.path.exists(path) else -1
        if node < 0:
            return {"gpu_numa_node": node, "affinity": "unchanged"}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        want = cpus & allowed
        if want:
            os.sched_setaffinity(0, want)
            return {"gpu_numa_node": node, "affinity": f"{len(want)} CPUs of node {node}"}
        return {"gpu_numa_node": node, "affinity": f"unchanged (node {node} CPUs not in this process's cpuset)"}
    except Exception as e:   # sysfs / NVML not available: nothing to do
        return {"gpu_numa_node": None, "affinity": f"unchanged ({type(e).__name__})"}


def _cpu_sets_by_node():
    """CPU ids of every host NUMA node that sysfs lists (empty when it lists none)."""
    sets = []
    base = "/sys/devices/system/node"
    try:
        for name in sorted(os.listdir(base)):
            if name.startswith("node") and name[4:].isdigit():
                cpus = set()
                for part in open(f"{base}/{name}/cpulist").read().strip().split(","):
                    if part:
                        lo, _, hi = part.partition("-")
                        cpus.update(range(int(lo), int(hi or lo) + 1))
                sets.append((name, cpus))
    except OSError:
        pass
    return sets


def pick_host_node_by_measurement(torch, device, info):
    """When sysfs does not say which NUMA node a GPU hangs off (containers often hide it), find out by measurement:
    pin this process to the CPUs of each host node in turn, allocate a pinned buffer there (pinned pages are placed on
    the node of the allocating thread) and time host-to-device copies from it; stay on the fastest node, so that the
    staging ring allocated afterwards is local to the GPU.  Before any timed region; changes only this process's CPU
    affinity."""
    if info.get("gpu_numa_node") not in (-1, None):
        return info
    try:
        allowed = os.sched_getaffinity(0)
        nodes = [(n, c & allowed) for n, c in _cpu_sets_by_node()]
        nodes = [(n, c) for n, c in nodes if c]
        if len(nodes) < 2:
            return dict(info, affinity=f"unchanged ({len(nodes)} host NUMA node(s) visible)")
        rates = {}
        dst = torch.empty(64 << 20, dtype=torch.uint8, device=device)
        for name, cpus in nodes:
            os.sched_setaffinity(0, cpus)
            src = torch.empty(64 << 20, dtype=torch.uint8).pin_memory()
            src.fill_(1)
            dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize(device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(8):
                dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize(device)
            rates[name] = 8 * src.numel() / (a.elapsed_time(b) * 1e-3) / 1e9
            del src
        best = max(rates, key=rates.get)
        os.sched_setaffinity(0, dict(nodes)[best])
        return dict(info, affinity=f"CPUs of {best}, chosen by measured H2D rate",
                    probed_h2d_GBps={k: round(v, 1) for k, v in rates.items()})
    except Exception as e:   # affinity calls not permitted, no sysfs ...: leave everything as it is
        try:
            os.sched_setaffinity(0, allowed)
        except Exception:
            pass
        return dict(info, affinity=f"unchanged ({type(e).__name__})")


def run_b200(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
    numa = gpu_numa_setup(local)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = pick_host_node_by_measurement(torch, device, numa)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from aimet_b200 import _lib, libpymo, ops
    from aimet_b200._lib import lib
    from aimet_b200.calibration import TfEnhancedCalibrator

    K, W = max(args.steps, 1), max(args.warmup, 3)
    sampler = ClockSampler(local)
    sampler.start()

    # ---- data: this rank's batches (global batch index k * world + rank), resident in HBM -----------------------
    batches = [device_batch(k * world + rank, device) for k in range(JOB_BATCHES)]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(secs):
        if world > 1:
            t = torch.tensor([secs], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        return secs

    def calibrate(rounds):
        """One job: `rounds` batches of this rank (all resident), exchange, replay, search, encoding on the host."""
        cal = TfEnhancedCalibrator(device, num_batches=rounds * world)
        cal.update_many(batches[:rounds])
        return cal, cal.compute_encoding(8, False, False, False)

    def timed_jobs(rounds, steps):
        """`steps` jobs back to back, device-timed, max over ranks."""
        barrier()
        sampler.busy = True
        e0.record()
        for _ in range(steps):
            out = calibrate(rounds)
        e1.record()
        barrier()
        sampler.busy = False
        return max_over_ranks(e0.elapsed_time(e1) * 1e-3), out

    def measure(rounds):
        """W warm-up jobs, then blocks of exactly K jobs until MIN_TIMED_S has been timed (at least 3 blocks)."""
        for _ in range(W):
            calibrate(rounds)
        launches0 = _lib.launch_count()
        first, out = timed_jobs(rounds, K)
        launches = _lib.launch_count() - launches0
        reps = max(3, min(200, int(MIN_TIMED_S / max(first, 1e-6)) + 1))
        if world > 1:   # every rank must run the same number of blocks
            t = torch.tensor([reps], dtype=torch.int64, device=device)
            dist.broadcast(t, 0)
            reps = int(t)
        times = [first] + [timed_jobs(rounds, K)[0] for _ in range(reps - 1)]
        med, lo, hi = median_spread(times)
        return {"secs": med, "min": lo, "max": hi, "blocks": len(times), "total_s": sum(times),
                "launches": launches, "out": out}

    # ---- the timed job: 256 batches per GPU (weak scaling) -----------------------------------------------------------
    weak = measure(JOB_BATCHES)
    value = world * K * JOB_BATCHES * SAMPLES_PER_BATCH / weak["secs"]
    cal, enc = weak["out"]

    # ---- configuration 3 itself split over the ranks (strong scaling): 256 batches in total --------------------------
    strong = None
    if world > 1 and JOB_BATCHES % world == 0:
        strong = measure(JOB_BATCHES // world)

    # ---- parity of the N-rank result with a single-process run over the same batches (outside the timed regions) ----
    parity = None
    if world > 1:
        parity = multi_gpu_parity(torch, dist, device, rank, world, batches,
                                  [("weak", weak["out"]), ("strong", strong["out"])] if strong else [("weak", weak["out"])])

    # ---- the v2 flavour of the analyzer on the same batches, sharded the same way (secondary) --------------------------
    v2 = None if args.skip_v2 else v2_sqnr_leg(torch, dist, device, rank, world, batches, barrier, max_over_ranks, e0, e1)

    # ---- roofline of the dominant kernel: back-to-back launches through the raw C ABI, CUDA events ---------------------
    roof = hist_roofline(torch, lib, ops, device, batches, e0, e1, sampler)

    # ---- end to end: batches start in pinned host memory; H2D copy + updateStats per batch, getEncoding per job ------
    e2e = e2e_leg(torch, libpymo, device, batches, K, W, barrier, max_over_ranks, e0, e1, sampler)
    e2e_value = world * K * JOB_BATCHES * SAMPLES_PER_BATCH / e2e["secs"]
    h2d_rates = [e2e["h2d_gbps"]]
    if world > 1:
        t = torch.zeros(world, dtype=torch.float64, device=device)
        t[rank] = e2e["h2d_gbps"]
        dist.all_reduce(t)
        h2d_rates = [round(v, 2) for v in t.tolist()]

    # ---- secondary numbers (rank 0): fake-quant kernels, model-level configurations 4 and 5 ----------------------------
    del batches
    torch.cuda.empty_cache()
    qdq = qdq_numbers(torch, lib, device, roof["peak"]) if (rank == 0 and not args.skip_qdq) else None
    models = None
    if rank == 0 and world == 1 and not args.skip_models:
        from aimet_b200.v2 import model_cases
        models = {}
        for name, case, kw in (("resnet50", "resnet50", {"batches": 32, "batch_size": 128}),
                               ("resnet50_v2_sqnr", "resnet50", {"batches": 32, "batch_size": 128,
                                                                 "scheme": "post_training_tf_enhanced"}),
                               ("llama_layer", "llama_layer", {})):
            try:
                models[name] = model_cases.CASES[case](device, **kw)
            except Exception as e:   # a model case must not take the headline down with it
                models[name] = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.empty_cache()
    clocks = sampler.stop()

    # ---- CPU baseline: the reference's own code on one host core, bounded sample (rank 0, N = 1 only) -------------
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        nb = 400
        data = [host_batch(b) for b in range(4)]
        cpu_calibration(1, data)
        cs, kind = cpu_calibration(nb, data)
        cpu = {"value": nb * SAMPLES_PER_BATCH / cs, "unit": "samples/s", "cores": 1, "kind": kind,
               "sample": f"{nb} batches of [64,256,28,28] (4 distinct, cycled) + computeEncoding, {cs:.1f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": weak["secs"] / K * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": job_config(world),
            "timing": {"blocks_of_K_steps": weak["blocks"], "timed_region_s": weak["total_s"],
                       "block_s_median": weak["secs"], "block_s_min": weak["min"], "block_s_max": weak["max"],
                       "us_per_batch": weak["secs"] / (K * JOB_BATCHES) * 1e6,
                       "timed_region": "per job: update_many over the rank's resident batches (first batch: fused "
                                       "min/max + grid setup, then histogram launches of up to 16 batches), "
                                       "table all-reduce (N > 1), PDF replay + SQNR search, encoding read-back"},
            "encoding": [enc.min, enc.max, enc.delta, enc.offset, enc.bw],
            "roofline": roof,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": JOB_BATCHES * BATCH_BYTES,
                    "d2h_bytes_per_step": 40, "ms_per_step": e2e["secs"] / K * 1e3,
                    "ms_per_batch": e2e["secs"] / (K * JOB_BATCHES) * 1e3, "h2d_GBps_per_rank": h2d_rates,
                    "api": "AimetTensorQuantizer.updateStats per batch (pinned host buffer -> device copy inside the "
                           "timed region) / getEncoding per job (the 5-double encoding comes back to the host)",
                    "numa": numa},
            "gpu_launches": weak["launches"],
            "clocks": clocks,
        }
        if strong is not None:
            sv = K * JOB_BATCHES * SAMPLES_PER_BATCH / strong["secs"]
            line["strong"] = {"value": sv, "unit": "samples/s", "scaling": "strong", "batches_per_job": JOB_BATCHES,
                              "batches_per_job_per_gpu": JOB_BATCHES // world,
                              "ms_per_step": strong["secs"] / K * 1e3, "blocks_of_K_steps": strong["blocks"],
                              "block_s_min": strong["min"], "block_s_max": strong["max"]}
        if parity is not None:
            line["parity_multi_gpu"] = parity["ok"]
            line["parity_multi_gpu_detail"] = parity
        if v2 is not None:
            line["v2_sqnr_sharded"] = v2
        if qdq is not None:
            line["qdq"] = qdq
        if models is not None:
            line["model_cases"] = models
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def multi_gpu_parity(torch, dist, device, rank, world, batches, jobs):
    """Bit-for-bit check of the N-rank result against a single-process run over the same global batches.

    Every rank contributes its encoding (all ranks must hold the same bits: nothing is broadcast); rank 0 regenerates
    the batches of the other ranks one at a time (batches are seeded by global index), runs the single-process
    calibrator over all of them in global order and compares the encoding, the merged [n, 512] row table and the
    counts as raw bits.  Returns {"ok": bool, "<job>": {...mismatch counts...}}."""
    from aimet_b200.calibration import TfEnhancedCalibrator
    result = {"ok": True}
    for name, (cal, enc) in jobs:
        n_total = cal.round * world
        mine = torch.tensor([enc.min, enc.max, enc.delta, enc.offset, float(enc.bw)], dtype=torch.float64, device=device)
        everyone = torch.empty(world * 5, dtype=torch.float64, device=device)
        dist.all_gather_into_tensor(everyone, mine)
        detail = {"batches": n_total}
        if rank == 0:
            ranks_differ = int((everyone.view(world, 5).view(torch.int64) != mine.view(torch.int64)).any(dim=1).sum())
            single = TfEnhancedCalibrator(device, num_batches=n_total)
            single.distributed, single.world, single.rank = False, 1, 0
            for g in range(n_total):
                x = batches[g // world] if g % world == 0 else device_batch(g, device)
                single.update(x)
            ref = single.compute_encoding(8, False, False, False)
            st_n, st_1 = cal.engine.state, single.engine.state
            rows_bad = int((st_n.hists[:n_total] != st_1.hists[:n_total]).any(dim=1).sum())
            counts_bad = int((st_n.counts[:n_total] != st_1.counts[:n_total]).sum())
            enc_same = [ref.min, ref.max, ref.delta, ref.offset, ref.bw] == [enc.min, enc.max, enc.delta, enc.offset, enc.bw]
            pdf_bad = int((st_n.pdf.view(torch.int64) != st_1.pdf.view(torch.int64)).sum())
            detail.update({"ranks_with_other_encoding": ranks_differ, "rows_mismatched": rows_bad,
                           "counts_mismatched": counts_bad, "pdf_buckets_mismatched": pdf_bad,
                           "encoding_equal": bool(enc_same)})
            ok = ranks_differ == 0 and rows_bad == 0 and counts_bad == 0 and pdf_bad == 0 and enc_same
            result["ok"] = bool(result["ok"] and ok)
        result[name] = detail
    flag = torch.tensor([1 if result["ok"] else 0], dtype=torch.int32, device=device)
    dist.broadcast(flag, 0)
    result["ok"] = bool(int(flag))
    return result


def v2_sqnr_leg(torch, dist, device, rank, world, batches, barrier, max_over_ranks, e0, e1):
    """The same batches through the aimet_torch v2 flavour of the analyzer (SqnrEncodingAnalyzer, 512 bins), sharded
    like the headline job: per job two passes over the rank's resident batches, two integer all-reduces (N > 1), the
    merges replayed in global batch order, the search, (min, max) read back.  Checked bit for bit against the
    sequential observer fed all batches in global order by rank 0.  A secondary number, not the headline."""
    from aimet_b200.calibration import SqnrCalibrator
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    rounds, bins, jobs = 32, 512, 5
    mine = batches[:rounds]

    def job():
        cal = SqnrCalibrator(SqnrEncodingAnalyzer((1,), bins), device)
        cal.calibrate(mine)
        mn, mx = cal.compute_encodings(255, False)
        return cal, [float(mn), float(mx)]

    for _ in range(3):
        job()
    barrier()
    e0.record()
    for _ in range(jobs):
        cal, enc = job()
    e1.record()
    barrier()
    secs = max_over_ranks(e0.elapsed_time(e1) * 1e-3)
    # parity, outside the timed region
    mine_enc = torch.tensor(enc, dtype=torch.float64, device=device)
    ok = True
    if world > 1:
        everyone = torch.empty(world * 2, dtype=torch.float64, device=device)
        dist.all_gather_into_tensor(everyone, mine_enc)
        ok = bool((everyone.view(world, 2) == mine_enc).all())
    if rank == 0:
        seq = SqnrEncodingAnalyzer((1,), bins)
        for g in range(rounds * world):
            seq.update_stats(batches[g // world] if g % world == 0 else device_batch(g, device))
        want, got = seq.observer.get_stats()[0], cal.analyzer.observer.get_stats()[0]
        mn, mx = seq.compute_encodings(255, False)
        ok = ok and bool(torch.equal(want.histogram.view(torch.int32), got.histogram.view(torch.int32))) \
            and bool(torch.equal(want.bin_edges.view(torch.int32), got.bin_edges.view(torch.int32))) \
            and [float(mn), float(mx)] == enc
    if world > 1:
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.broadcast(flag, 0)
        ok = bool(int(flag))
    return {"value": world * jobs * rounds * SAMPLES_PER_BATCH / secs, "unit": "samples/s", "ms_per_job": secs / jobs * 1e3,
            "batches_per_gpu": rounds, "bins": bins, "passes_over_data": 2, "encoding": enc,
            "parity_with_sequential_observer": ok,
            "algorithmic_GBps_per_gpu": jobs * rounds * 2 * BATCH_BYTES / secs / 1e9}


def hist_roofline(torch, lib, ops, device, batches, e0, e1, sampler):
    """The dominant kernel alone, as the job launches it (16 resident batches per launch) and one batch per launch."""
    import ctypes as C
    M = 16
    n = len(batches)
    st = ops.TfeDeviceState(device, capacity=n)
    st.offer_grid(batches[0])
    stream = torch.cuda.current_stream().cuda_stream
    hp, cp, sp = st.hists.data_ptr(), st.counts.data_ptr(), st.state.data_ptr()
    groups = []
    for i in range(0, n, M):
        part = batches[i:i + M]
        groups.append(((C.c_void_p * len(part))(*[b.data_ptr() for b in part]),
                       (C.c_int64 * len(part))(*[b.numel() for b in part]), len(part), i))

    def many_pass():
        for ptrs, ns, m, row in groups:
            lib.aq_tfe_histogram_many(ptrs, ns, m, 1, sp, hp + 2048 * row, cp + 8 * row, None, stream)

    def single_pass():
        for i, b in enumerate(batches):
            lib.aq_tfe_histogram(b.data_ptr(), N_EL, sp, hp + 2048 * i, cp + 8 * i, stream)

    out = {}
    for name, fn, launches in (("many", many_pass, len(groups)), ("single", single_pass, n)):
        fn()
        torch.cuda.synchronize()
        sampler.busy = True
        times = []
        for _ in range(5):
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e-3)
        sampler.busy = False
        out[name] = median_spread(times)[0] / launches
    peak, peak_kind = peak_hbm()
    per_launch = M * BATCH_BYTES
    achieved = per_launch / out["many"] / 1e9
    single = BATCH_BYTES / out["single"] / 1e9
    return {"bound": "hbm", "kernel": "tfe_hist_lane_kernel", "achieved": achieved, "peak": peak,
            "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
            "traffic": HIST_TRAFFIC_RATIO * per_launch, "bytes_per_launch": per_launch,
            "batches_per_launch": M, "us_per_launch": out["many"] * 1e6,
            "one_batch_per_launch": {"bytes_per_launch": BATCH_BYTES, "us_per_launch": out["single"] * 1e6,
                                     "achieved": single, "frac": single / peak}}


def e2e_leg(torch, libpymo, device, batches, K, W, barrier, max_over_ranks, e0, e1, sampler):
    """K jobs through the reference-facing API with HOST buffers: every batch is copied from pinned host memory to the
    device inside the timed region (double-buffered on a copy stream), and every job ends with getEncoding."""
    ring = [torch.empty(BATCH_SHAPE, dtype=torch.float32).pin_memory() for _ in range(4)]
    for i, r in enumerate(ring):
        r.copy_(batches[i])
    dev_buf = [torch.empty(BATCH_SHAPE, dtype=torch.float32, device=device) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def job(num):
        q = libpymo.AimetTensorQuantizer(libpymo.QUANTIZATION_TF_ENHANCED)
        main = torch.cuda.current_stream()
        for k in range(num):
            s = k % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[s])
                dev_buf[s].copy_(ring[k % len(ring)], non_blocking=True)
                copied[s].record(copy_stream)
            main.wait_event(copied[s])
            q.updateStats(dev_buf[s], True)
            consumed[s].record(main)
        return q.getEncoding(8, False, False, False)

    for ev in consumed:
        ev.record(torch.cuda.current_stream())
    job(8)   # warm-up: a short job is enough to page everything in
    # e2e steps are long (a quarter of a second each): a few of them already give a stable number
    steps = K if K * JOB_BATCHES * 1e-3 < 6.0 else max(1, int(6.0 / (JOB_BATCHES * 1e-3)))
    barrier()
    sampler.busy = True
    e0.record()
    for _ in range(steps):
        job(JOB_BATCHES)
    e1.record()
    barrier()
    sampler.busy = False
    local = e0.elapsed_time(e1) * 1e-3
    secs = max_over_ranks(local) * K / steps    # scaled to K steps when fewer were run
    return {"secs": secs, "steps_run": steps, "h2d_gbps": steps * JOB_BATCHES * BATCH_BYTES / local / 1e9}


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
    # the same launches without the per-launch CPU cost (a ctypes call costs about as much as this kernel runs)
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(nb):
            lib.aq_minmax(P(xs[i]), 0, n1, 1, n1, P(mm[0:1]), P(mm[1:2]), 0, 0, P(ws), ws.numel(), side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    rec("c1_minmax_4B_graph", 4 * n1, timed([graph.replay], 6) / nb)
    del xs, ys, ms, graph
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
# single-kernel cases (micro-benchmarks; small enough to capture under a profiler: one kernel, a few launches)
# ---------------------------------------------------------------------------------------------------------------------
KERNEL_CASES = ("tfe_hist", "tfe_hist_many", "tfe_offer_grid", "minmax_f32", "minmax_f32_rows", "minmax_bf16_block64", "v2_qdq_f32", "v2_qdq_f32_mask",
                "v2_qdq_f32_per_channel", "v2_qdq_bf16", "v2_qdq_bf16_block64", "v2_bwd_f32", "v2_bwd_bf16",
                "pymo_qdq_f32", "pymo_qdq_f32_per_channel", "ste_v1_f32", "tfe_replay", "tfe_search",
                "v2_param_grad_f32_per_channel", "pymo_broadcast_f32", "v2hist_update_f32", "quantize_packed_f32",
                "qdq_fp16_f32", "tfe_mse")


def build_kernel_case(name, mb, torch, lib, device):
    """Returns (calls, algorithmic bytes per launch): `calls` launch the named kernel through the C ABI on rotating
    inputs of `mb` MB each whose total exceeds the L2 capacity."""
    from aimet_b200 import ops, _lib
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

    if name == "tfe_mse":
        # the MSE analyzer's candidate search on the statistics of 8 post-ReLU batches (replay included)
        g = torch.Generator(device=device)
        g.manual_seed(5)
        x = torch.relu(torch.randn(1 << 22, device=device, generator=g))
        st = ops.TfeDeviceState(device, capacity=8)
        st.init_grid_from(ops.minmax(x).reshape(-1))
        for r in range(8):
            st.add_batch(x[r * 4096:r * 4096 + (1 << 19)], r)
        calls = [lambda: (st.mse_encoding(True, 8, False, False, False), 0)[1]]
        return calls, 8 * 2056 + 2 * 512 * 8, [st, x]
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
    if name == "tfe_hist_many":
        # 16 resident batches of `mb` MB per launch, each into its own row; two such groups are rotated
        import ctypes as C
        nbuf = 32
        xs = data("relu_outliers")
        st = ops.TfeDeviceState(device, capacity=nbuf)
        st.offer_grid(xs[0])
        hp, cp, sp = P(st.hists), P(st.counts), P(st.state)
        groups = [((C.c_void_p * 16)(*[P(x) for x in xs[i:i + 16]]), (C.c_int64 * 16)(*([n] * 16)), i) for i in (0, 16)]
        calls = [lambda g=g: lib.aq_tfe_histogram_many(g[0], g[1], 16, 1, sp, hp + 2048 * g[2], cp + 8 * g[2], None, stream)
                 for g in groups]
        return calls, 16 * 4 * n, [st, groups] + xs
    xs = data("relu_outliers" if name.startswith("tfe_") else "normal")
    if name == "tfe_offer_grid":
        # fused min/max pass + grid setup on a state that is reset before every launch (otherwise the launch is a no-op)
        st = ops.TfeDeviceState(device, capacity=1)
        ws = ops.workspace(st.state, int(lib.aq_tfe_offer_grid_workspace_bytes()))
        sp = P(st.state)
        flag = st.state[_lib.AqTfeState.initialized.offset:_lib.AqTfeState.initialized.offset + 4]
        def call(i):
            flag.zero_()
            return lib.aq_tfe_offer_grid(P(xs[i]), n, sp, None, 1, P(ws), ws.numel(), stream)
        return [lambda i=i: call(i) for i in range(nbuf)], 4 * n, [st, ws] + xs
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
    if name == "v2hist_update_f32":
        # one calibration step of the v2 histogram observer on a post-ReLU activation: finite min/max pass, then one
        # counting pass for the batch's own range and the widened range (2048 bins), merge into the running histogram
        from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
        xr = data("relu_outliers")
        an = SqnrEncodingAnalyzer(())
        an.update_stats(xr[0])
        calls = [lambda i=i: (an.update_stats(xr[i]), 0)[1] for i in range(nbuf)]
        return calls, 8 * n, [an] + xr
    if name == "quantize_packed_f32":
        outs = [torch.empty(n, dtype=torch.uint8, device=device) for _ in range(nbuf)]
        calls = [lambda i=i: lib.aq_quantize_packed(P(xs[i]), P(outs[i]), n, -4.4, 4.6, 8, 0, 0, stream) for i in range(nbuf)]
        return calls, 5 * n, [outs] + xs
    if name == "qdq_fp16_f32":
        calls = [lambda i=i: lib.aq_qdq_fp16(P(xs[i]), P(ys[i]), n, stream) for i in range(nbuf)]
        return calls, 8 * n, [ys] + xs
    if name == "v2_param_grad_f32_per_channel":
        # scale / offset gradients summed per channel inside the kernel: rows of 2304 elements, 8-bit signed grid
        num_ch, inner = n // 2304, 2304
        s, o = torch.full((num_ch,), 0.03, device=device), torch.zeros(num_ch, device=device)
        gs = [torch.randn(n, device=device) for _ in range(nbuf)]
        ms = [(torch.rand(n, device=device) < 0.97).to(torch.uint8) for _ in range(nbuf)]
        ds, do = torch.empty(num_ch, device=device), torch.empty(num_ch, device=device)
        calls = [lambda i=i: lib.aq_v2_qdq_backward_params_reduced(P(xs[i]), P(gs[i]), P(ms[i]), P(ds), P(do), 0, n, num_ch,
                                                                   inner, P(s), P(o), -128.0, 127.0, stream)
                 for i in range(nbuf)]
        return calls, 9 * n + 16 * num_ch, [s, o, gs, ms, ds, do] + xs
    if name == "pymo_broadcast_f32":
        # encodings interleaved with broadcast dimensions ([R, 1, 3] against a [R, 768, 3] tensor): the only shape that
        # does not reduce to channel = (i / inner) % num_ch and therefore takes the general strided kernel
        import ctypes as C
        R = n // 2304
        enc = [torch.full((R * 3,), v, device=device) for v in (-4.0, 4.0, 8.0 / 255.0, -128.0)]
        in_strides = (C.c_int64 * 3)(2304, 3, 1)
        enc_strides = (C.c_int64 * 3)(3, 0, 1)
        calls = [lambda i=i: lib.aq_qdq_broadcast(P(xs[i]), P(ys[i]), n, 3, in_strides, enc_strides, P(enc[0]), P(enc[1]),
                                                  P(enc[2]), P(enc[3]), stream) for i in range(nbuf)]
        return calls, 8 * n + 16 * R * 3, [enc, in_strides, enc_strides, ys] + xs
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
    ap.add_argument("--steps", type=int, default=20, help="calibration jobs per timed block")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg")
    ap.add_argument("--skip-qdq", action="store_true", help="omit the secondary fake-quant kernel numbers")
    ap.add_argument("--skip-v2", action="store_true", help="omit the sharded v2 SQNR calibration leg")
    ap.add_argument("--skip-models", action="store_true", help="omit the model-level cases (configurations 4 and 5)")
    ap.add_argument("--kernel-case", choices=KERNEL_CASES, help="time one kernel alone instead of the calibration job")
    ap.add_argument("--mb", type=int, default=256, help="input size in MB for --kernel-case")
    ap.add_argument("--model-case", choices=("resnet50", "llama_layer"),
                    help="whole-model calibration / fake-quant measurement instead of the calibration job")
    ap.add_argument("--batches", type=int, default=32, help="calibration batches for --model-case resnet50")
    ap.add_argument("--batch-size", type=int, default=128, help="batch size for --model-case resnet50")
    ap.add_argument("--scheme", default=None, help="quant scheme for --model-case resnet50 (default: the case's own)")
    args = ap.parse_args()
    if args.model_case:
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
        from aimet_b200.v2 import model_cases
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        kw = {"batches": args.batches, "batch_size": args.batch_size} if args.model_case == "resnet50" else {}
        if args.scheme and args.model_case == "resnet50":
            kw["scheme"] = args.scheme
        print(json.dumps(model_cases.CASES[args.model_case](dev, **kw)), flush=True)
    elif args.kernel_case:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
