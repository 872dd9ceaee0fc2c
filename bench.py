#!/usr/bin/env python
"""Benchmark of the B200 batched token sampler on the headline configuration (B = 64 rows, V = 262144 fp32 logits).

    python bench.py --gpus 1 --steps 400 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      (the reference's CPU sampler on the host cores, same workload)

A step is one pass of the sampler over one batch: Student-t(3) * 4 logits soft-capped at 30, temperature 1,
top-k 64, top-p 0.95, repetition penalty 1.0 / 1.1 on alternating rows over 512-id histories.  Data is synthetic
and seeded (ferro_b200.synth.config3; the logits rotate through several buffers of the same distribution, the first
of which holds the configuration's own array).  With N GPUs every rank samples its own batch of 64 rows (rows are
independent streams: row sharding, no data-path collective), so scaling is weak and `value` is the rows of all
ranks per second.

Timing: CUDA events on the launching stream around exactly K back-to-back launches after W warm-up launches, a
barrier and a device synchronisation on both sides, the maximum over ranks.  The launches do not overlap: every
launch starts after the one before has finished, as the steps of a decode loop do.  The logits rotate through a set
of buffers larger than L2, so every step reads its logits from HBM.  `e2e` is the same batch through the public
call `fsb_sample_batch` with the logits in pinned host memory (host-to-device copy and token read-back inside the
timed region).  PyTorch is used for device memory, streams and the process group only; the sampler is the C-ABI
library.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, VOCAB, TOP_K, HIST = 64, 262144, 64, 512
METRIC, UNIT = "sampled_rows_per_s", "rows/s"
WORKLOAD = "cfg3: B=64 x V=262144 fp32, Student-t(3)*4 softcap 30, T=1 top_k=64 top_p=0.95, penalty 1.0/1.1 alternating, 512-id histories"
# DRAM traffic of one launch of the streaming kernel on this workload, from the committed ncu summary
# (profiles/stream_select_kernel_cfg3.md: dram__bytes_read.sum + dram__bytes_write.sum)
NCU_TRAFFIC_BYTES = 68.57e6   # dram__bytes_read.sum + dram__bytes_write.sum per launch, mean of two captured launches (profiles/stream_select_kernel_cfg3.md)


def algorithmic_bytes(rows=ROWS, vocab=VOCAB, hist=HIST):
    """Bytes one launch must move: the logits once, the penalty-window ids, one engine word and one token per row."""
    return rows * (4 * vocab + 4 * hist + 8 + 4)


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    except Exception:
        return 6650.0, "fallback (earlier measurement on this pool)"


def c_softcap():
    """In-place float32 softcap built on the C library's tanhf (the function the reference calls): oracle.softcap."""
    from oracle import Oracle
    orc = Oracle()
    return orc.softcap


def workload(rank, tanhf=None):
    """The configuration's parameters, histories and (rank 0's buffer 0) logits."""
    from ferro_b200 import synth
    cfg = synth.config3(rows=ROWS, tanhf=tanhf)
    p = cfg["params"].copy()
    p["seed"] = 7 + 1000 * rank + np.arange(ROWS)
    if rank == 0:
        return cfg["logits"], p, cfg["hists"], cfg["raw_logits"]
    rng = np.random.default_rng(700 + rank)
    return cfg["logits"], p, [rng.integers(0, VOCAB, size=HIST).astype(np.int32) for _ in range(ROWS)], cfg["raw_logits"]


def device_logits(torch, gen, device, rows=ROWS, vocab=VOCAB):
    """Student-t(3) * 4, then 30 * tanh(x / 30): the Gemma-4-style large-vocabulary row."""
    z = torch.randn(rows, vocab, device=device, generator=gen)
    den = torch.zeros(rows, vocab, device=device)
    for _ in range(3):
        den += torch.randn(rows, vocab, device=device, generator=gen) ** 2
    x = 4.0 * z / torch.sqrt(den / 3.0)
    return (30.0 * torch.tanh(x / 30.0)).float().contiguous()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = "index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ the CPU side
def cpu_rows_per_s(params, logits, hists, seconds_budget, threads=None):
    """Times the reference's own CPU sampler (compiled unmodified into oracle/_ref; else the C port of it) on the
    host cores on the given rows.  Returns (all-threads rows/s, single-thread rows/s, threads, kind, passes)."""
    from oracle import Oracle, RefLib
    rows = len(params)
    n_threads = min(threads or (os.cpu_count() or 1), rows)
    if RefLib.available():
        ref = RefLib()
        kind = "reference"

        def one_pass(nt):
            secs, _ = ref.time_rows(params, logits.copy(), hists, nt)
            return secs
    else:
        orc = Oracle()
        kind = "port"

        def one_pass(nt):
            x = logits.copy()
            rngs = orc.new_rngs(params["seed"])
            t0 = time.perf_counter()
            if nt == 1:
                orc.sample_rows(params, rngs, x, hists)
            else:   # ctypes releases the GIL: row blocks run on Python threads
                bounds = [rows * t // nt for t in range(nt + 1)]
                ths = [threading.Thread(target=orc.sample_rows, args=(params[a:b], rngs[a:b], x[a:b], hists[a:b])) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
                [t.start() for t in ths]
                [t.join() for t in ths]
            return time.perf_counter() - t0
    one_pass(1)
    single, multi, passes = [], [], 0
    t_end = time.perf_counter() + seconds_budget
    while (passes < 3 or time.perf_counter() < t_end) and passes < 200:
        single.append(one_pass(1))
        multi.append(one_pass(n_threads))
        passes += 1
    return rows / float(np.median(multi)), rows / float(np.median(single)), n_threads, kind, passes


def cpu_baseline_cfg3(seconds_budget):
    from ferro_b200 import synth
    cfg = synth.config3(rows=ROWS, tanhf=c_softcap())
    val, single, threads, kind, passes = cpu_rows_per_s(cfg["params"], cfg["logits"], cfg["hists"], seconds_budget)
    sample = f"{passes} passes over {ROWS} rows x {VOCAB} (median), fresh logits copy per pass, sample() calls only"
    return val, single, threads, kind, sample


def run_reference_arm(args, rank):
    """The reference's CPU sampler on the host cores; touches neither a GPU nor this repository's CUDA library."""
    if rank != 0:
        return
    steps_budget = max(4.0, min(60.0, 0.15 * (args.steps + args.warmup)))
    val, single, threads, kind, sample = cpu_baseline_cfg3(steps_budget)
    out = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * ROWS / val, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "global_rows": ROWS, "vocab": VOCAB, "parallelism": "host threads"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample, "single_thread_value": single},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------ helpers of the GPU side
def bind_to_gpu_numa_node(local_rank):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off (read-only topology query), so that the pinned
    buffers allocated afterwards and the copies out of them stay on that node.  Returns a short description."""
    try:
        bus = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(local_rank)], capture_output=True, text=True,
                             timeout=10).stdout.strip().lower()
        if bus.startswith("0000"):
            bus = bus[4:]   # sysfs uses a four-digit domain
        node_file = f"/sys/bus/pci/devices/{bus}/numa_node"
        node = int(open(node_file).read().strip())
        if node < 0:   # sysfs does not say (virtual machines): ask NVML for the GPU's ideal CPUs (a read-only query)
            try:
                import pynvml
                pynvml.nvmlInit()
                words = pynvml.nvmlDeviceGetCpuAffinity(pynvml.nvmlDeviceGetHandleByIndex(local_rank), 16)
                ideal = {64 * w + b for w, x in enumerate(words) for b in range(64) if (int(x) >> b) & 1}
            except Exception:
                return "numa node unknown"
            here = os.sched_getaffinity(0)
            allowed = sorted(ideal & here)
            if not allowed or len(allowed) == len(here):
                return f"one numa node visible ({len(here)} cpus): nothing to bind"
            os.sched_setaffinity(0, allowed)
            return f"nvml cpu affinity, {len(allowed)} of {len(here)} cpus"
        cpus = open(f"/sys/devices/system/node/node{node}/cpulist").read().strip()
        ids = []
        for part in cpus.split(","):
            a, _, b = part.partition("-")
            ids += list(range(int(a), int(b or a) + 1))
        allowed = sorted(set(ids) & os.sched_getaffinity(0))
        if not allowed:
            return f"numa node {node}: none of its cpus is allowed here"
        os.sched_setaffinity(0, allowed)
        return f"numa node {node}, {len(allowed)} cpus"
    except Exception as ex:   # no sysfs, no nvidia-smi, a container without the files: carry on unbound
        return f"unbound ({type(ex).__name__})"


def time_launches(torch, launch, n, warm=3):
    """Microseconds per call of `launch(i)` over n back-to-back calls, CUDA events on the current stream."""
    for i in range(warm):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / n


def time_calls(call, n, warm=3):
    """Wall-clock microseconds per synchronous call."""
    for i in range(warm):
        call(i)
    t0 = time.perf_counter()
    for i in range(n):
        call(i)
    return 1e6 * (time.perf_counter() - t0) / n


def config_figures(torch, fb, device, peak, tanhf, budget_s=3.0, only=None):
    """The other four configurations through the call a server would make, each with the reference's CPU time on the
    same rows beside it: device time per step (CUDA events, logits resident, buffers rotating past L2 where they are
    large enough to matter), wall time of the public call, algorithmic bytes and the fraction of the HBM peak."""
    from ferro_b200 import synth
    out = {}
    stream = torch.cuda.current_stream().cuda_stream

    def engine_for(rows, vocab, hist_ids):
        e = fb.Engine(device=device.index, max_rows=rows, max_vocab=vocab, max_hist_ids=hist_ids)
        e.set_cuda_stream(stream)
        return e

    def entry(name, rows, vocab, hist, step_us, call_us, cpu, extra=None):
        b = algorithmic_bytes(rows, vocab, hist)
        d = {"rows": rows, "vocab": vocab, "device_step_us": step_us, "public_call_us": call_us, "algorithmic_bytes": b,
             "achieved_gb_s": b / step_us / 1e3, "frac_of_measured_peak": b / step_us / 1e3 / peak, "rows_per_s": rows / step_us * 1e6,
             "cpu_reference": {"rows_per_s_all_threads": cpu[0], "rows_per_s_one_thread": cpu[1], "threads": cpu[2], "kind": cpu[3],
                               "sample": f"{cpu[4]} passes over {cpu[5]} rows"}}
        if extra:
            d.update(extra)
        out[name] = d

    def resident_call_us(e, sids, hists, devs, vocab, n):
        for s_, h_ in zip(sids, hists):
            e.history_set(int(s_), h_)
        return time_calls(lambda i: e.sample_batch_resident(sids, devs[i % len(devs)].data_ptr(), n_vocab=vocab), n)

    if only not in (None, "cfg1"):
        return config_figures_rest(torch, fb, device, peak, tanhf, budget_s, only, out, engine_for, entry, resident_call_us)
    # ---- cfg 1: one row, the latency of a single stream's step
    c1 = synth.config1()
    e = engine_for(1, 65536, 1 << 12)
    sid = e.open_streams(c1["params"])
    devs = [torch.from_numpy(c1["logits"]).to(device) for _ in range(4)]
    batch = e.prepare_batch(sid, c1["hists"], 65536)
    step = time_launches(torch, lambda i: batch.launch(devs[i % 4].data_ptr()), 200)
    batch.free()
    call = time_calls(lambda i: e.sample_batch(sid, devs[i % 4], c1["hists"], n_vocab=65536), 200)
    cpu = cpu_rows_per_s(c1["params"], c1["logits"], c1["hists"], budget_s / 2, threads=1)
    entry("cfg1_1x65536_k40", 1, 65536, 64, step, call, cpu + (1,), {"public_call_resident_us": resident_call_us(e, sid, c1["hists"], devs, 65536, 200)})
    e.close()
    return config_figures_rest(torch, fb, device, peak, tanhf, budget_s, only, out, engine_for, entry, resident_call_us)


def config_figures_rest(torch, fb, device, peak, tanhf, budget_s, only, out, engine_for, entry, resident_call_us):
    from ferro_b200 import synth
    if only in (None, "cfg2"):
        config2_figures(torch, fb, device, synth, budget_s, engine_for, entry, resident_call_us)
    if only in (None, "cfg4"):
        config4_figures(torch, fb, device, synth, budget_s, engine_for, entry)
    if only in (None, "cfg5"):
        config5_figures(torch, fb, device, synth, budget_s, tanhf, engine_for, entry, resident_call_us)
    return out


def config2_figures(torch, fb, device, synth, budget_s, engine_for, entry, resident_call_us):
    # ---- cfg 2: the mixed decode batch, four of its eight rows take the full-vocabulary kernel
    c2 = synth.config2()
    e = engine_for(8, 65536, 1 << 14)
    sids = e.open_streams(c2["params"])
    devs = [torch.from_numpy(c2["logits"]).to(device) for _ in range(4)]
    batch = e.prepare_batch(sids, c2["hists"], 65536)
    step = time_launches(torch, lambda i: batch.launch(devs[i % 4].data_ptr()), 100)
    kernels = batch.kernels_per_launch
    batch.free()
    call = time_calls(lambda i: e.sample_batch(sids, devs[i % 4], c2["hists"], n_vocab=65536), 100)
    cpu = cpu_rows_per_s(c2["params"], c2["logits"], c2["hists"], budget_s)
    entry("cfg2_8x65536_mixed", 8, 65536, 256, step, call, cpu + (8,),
          {"kernels_per_step": kernels, "full_vocabulary_rows": 4, "public_call_resident_us": resident_call_us(e, sids, c2["hists"], devs, 65536, 100)})
    e.close()


def config4_figures(torch, fb, device, synth, budget_s, engine_for, entry):
    # ---- cfg 4: 8 verification windows of 17 rows through fsb_verify_windows
    c4 = synth.config4()
    e = engine_for(136, 65536, 1 << 14)
    sids = e.open_streams(c4["params"])
    devs = [torch.from_numpy(c4["logits"]).to(device) for _ in range(4)]
    p_rows = np.repeat(c4["params"], 17)
    row_sids = e.open_streams(p_rows)
    batch = e.prepare_batch(row_sids, [[]] * 136, 65536)
    step = time_launches(torch, lambda i: batch.launch(devs[i % 4].data_ptr()), 100)
    batch.free()
    call = time_calls(lambda i: e.verify_windows(sids, c4["rows"], devs[i % 4], c4["hists"], n_vocab=65536), 100)
    cpu = cpu_rows_per_s(p_rows, c4["logits"], [np.zeros(0, np.int32)] * 136, budget_s)
    entry("cfg4_8x17_windows_65536_greedy", 136, 65536, 0, step, call, cpu + (136,), {"public_call": "fsb_verify_windows"})
    e.close()


def config5_figures(torch, fb, device, synth, budget_s, tanhf, engine_for, entry, resident_call_us):
    # ---- cfg 5 on one GPU: 512 rows; the first 64 are the configuration's own rows (the CPU sample), the rest are
    # drawn on the device from the same distribution
    n_own = 64
    c5 = synth.config5(rows=n_own, tanhf=tanhf)
    gen = torch.Generator(device=device)
    gen.manual_seed(99)
    devs = []
    for _ in range(2):
        d = device_logits(torch, gen, device, 512, 262144)
        d[:n_own].copy_(torch.from_numpy(c5["logits"]))
        devs.append(d)
    p = np.concatenate([c5["params"]] * (512 // n_own))
    p["seed"] = 99 + np.arange(512)
    rng = np.random.default_rng(99)
    hists = list(c5["hists"]) + [c5["hists"][int(i)] for i in rng.integers(0, n_own, size=512 - n_own)]
    e = engine_for(512, 262144, 512 * 1024 + 64)
    sids = e.open_streams(p)
    batch = e.prepare_batch(sids, hists, 262144)
    step = time_launches(torch, lambda i: batch.launch(devs[i % 2].data_ptr()), 30)
    batch.free()
    call = time_calls(lambda i: e.sample_batch(sids, devs[i % 2], hists, n_vocab=262144), 20)
    cpu = cpu_rows_per_s(c5["params"], c5["logits"], c5["hists"], budget_s)
    entry("cfg5_512x262144_k40", 512, 262144, 1024, step, call, cpu + (n_own,),
          {"public_call_resident_us": resident_call_us(e, sids, hists, devs, 262144, 20)})
    e.close()
    del devs


def softcap_mismatches(fb, eng, sids, raw, ref_tokens, hists):
    """The fused device softcap on the raw logits against the host-capped oracle tokens: mismatching rows of 64."""
    eng.set_softcap(30.0)
    try:
        tok = eng.sample_batch(sids, raw, hists)
    finally:
        eng.set_softcap(0.0)
    return int((tok != ref_tokens).sum())


def c_call_latency(fb):
    """The public calls timed from C++ (tests/call_latency.cpp, built here with g++): medians in microseconds for the
    headline shape.  None when the machine has no compiler or no CUDA toolkit headers."""
    import shutil
    import subprocess
    import tempfile
    gxx, cuda = shutil.which("g++"), os.environ.get("CUDA_HOME", "/usr/local/cuda")
    src = os.path.join(ROOT, "tests", "call_latency.cpp")
    if not gxx or not os.path.exists(src) or not os.path.exists(os.path.join(cuda, "include", "cuda_runtime.h")):
        return None
    lib = fb.library_path()
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "call_latency")
        cmd = [gxx, "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"), src, "-L", os.path.dirname(lib),
               "-lferro_sampler_b200", "-Wl,-rpath," + os.path.dirname(lib), "-L", os.path.join(cuda, "lib64"), "-lcudart", "-o", exe]
        if subprocess.run(cmd, capture_output=True).returncode != 0:
            return None
        r = subprocess.run([exe, str(ROWS), str(VOCAB), str(HIST), "200"], capture_output=True, text=True, timeout=300)
        if r.returncode != 0:
            return {"error": (r.stderr or r.stdout)[-200:]}
        return json.loads(r.stdout.strip().splitlines()[-1])


def vocab_sharded_leg(torch, dist, fb, device, rank, world, barrier):
    """The serving batch split by vocabulary: every rank holds V / world columns of all 512 rows, selects its
    candidates, NCCL exchange, merge (ferro_b200.sharded).  Timed, and its tokens compared: across ranks, and on
    rank 0 with the unsharded launch over the gathered columns."""
    from ferro_b200 import sharded
    rows, vocab = 512, 262144
    lo, hi = sharded.vocab_partition(vocab, world)[rank]
    out = {}
    ready, eng, samp = 1, None, None
    try:
        gen = torch.Generator(device=device)
        gen.manual_seed(4321)                                    # the same full matrix on every rank; each keeps its columns
        full = [torch.randn(rows, vocab, device=device, generator=gen) * 3.0 for _ in range(2)]
        shard = [f[:, lo:hi].contiguous() for f in full]
        p = fb.make_params(rows, temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1)
        p["seed"] = 99 + np.arange(rows)                       # the same streams on every rank
        hh = [np.random.default_rng(1000 + r).integers(0, vocab, size=1024).astype(np.int32) for r in range(rows)]
        eng = fb.Engine(device=device.index, max_rows=rows, max_vocab=hi - lo, max_hist_ids=rows * 1024 + 16)
        eng.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
    except Exception as ex:
        ready = 0
        out["error"] = f"{type(ex).__name__}: {ex}"
    flag = torch.tensor([ready], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)                # every rank takes part in the collectives below, or none
    if int(flag.item()) == 1:
        want = None
        if rank == 0:                                            # the unsharded launch over the whole rows: first draw of every stream
            e0 = fb.Engine(device=device.index, max_rows=rows, max_vocab=vocab, max_hist_ids=rows * 1024 + 16)
            e0.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
            want = e0.sample_batch(e0.open_streams(p), full[0], hh, n_vocab=vocab)
            e0.close()
        for mode in ("all_to_all", "all_gather"):
            samp = sharded.VocabShardedSampler(eng, vocab, rank, world, exchange=mode)
            samp.prepare(eng.open_streams(p), hh, rows)
            for i in range(5):
                samp.step(shard[i % 2])
            barrier()
            us = time_launches(torch, lambda i: samp.step(shard[i % 2]), 30)
            t = torch.tensor([us], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            samp.prepare(eng.open_streams(p), hh, rows)      # fresh streams: their first draw, as in the unsharded launch
            samp.step(shard[0])
            tok = samp.tokens()
            mine = torch.from_numpy(tok.astype(np.int64)).to(device)
            allt = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allt, mine)
            across = int(sum(int((a != allt[0]).sum().item()) for a in allt[1:]))
            out[mode] = {"step_us": float(t.item()), "rows_per_s": rows / float(t.item()) * 1e6, "exchange": samp.exchange_description(),
                         "parity_mismatches_across_ranks": across,
                         "parity_mismatches_vs_unsharded": int((want != tok).sum()) if want is not None else None}
            samp.release()
        out["columns_per_gpu"] = hi - lo
    if eng is not None:
        eng.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the side figures (other configurations, staging, vocabulary sharding)")
    ap.add_argument("--only", choices=["cfg1", "cfg2", "cfg4", "cfg5"], help="run one side configuration alone and print its figures (a small "
                    "command to profile: cfg2 launches the full-vocabulary kernel); not a benchmark line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    numa = bind_to_gpu_numa_node(local_rank)   # before anything is pinned
    import torch
    import torch.distributed as dist
    import ferro_b200 as fb

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.only:
        peak, _ = measured_hbm_peak()
        print(json.dumps({"only": args.only, "figures": config_figures(torch, fb, device, peak, c_softcap(), budget_s=0.5, only=args.only)}), flush=True)
        return

    # ---- workload, resident in HBM before anything is timed
    tanhf = c_softcap()
    own_logits, params, hists, raw_logits = workload(rank, tanhf)
    gen = torch.Generator(device=device)
    gen.manual_seed(7 + rank)
    n_buf = 8   # 8 x 67 MB = 537 MB, more than four times the 126 MB L2: every step streams from HBM
    bufs = [torch.from_numpy(own_logits).to(device)] + [device_logits(torch, gen, device) for _ in range(n_buf - 1)]
    eng = fb.Engine(device=local_rank, max_rows=ROWS, max_vocab=VOCAB, max_hist_ids=2 * ROWS * HIST + 16)
    eng.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
    sids = eng.open_streams(params)
    batch = eng.prepare_batch(sids, hists, VOCAB)
    kernels_per_step = batch.kernels_per_launch

    # ---- the timed steps: a train of launches on one stream, no overlap between them
    eng.set_launch_overlap(0)
    for i in range(args.warmup):
        batch.launch(bufs[i % n_buf].data_ptr())
    barrier()
    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        batch.launch(bufs[i % n_buf].data_ptr())
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    # parity of a timed batch: the launch on buffer 0 (the configuration's own logits), outside the timed region
    batch.launch(bufs[0].data_ptr())
    tokens = batch.tokens()
    # the same train with the launches chained by programmatic stream serialization.  Mode 2: every CTA waits for the
    # previous launch to be complete before it touches memory - plain stream order, only the launch latency is hidden.
    # Mode 1: a launch may read logits while the previous one is in its tail - a figure for independent batches.
    def chained_train(mode):
        eng.set_launch_overlap(mode)
        for i in range(3):
            batch.launch(bufs[i % n_buf].data_ptr())
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for i in range(args.steps):
            batch.launch(bufs[i % n_buf].data_ptr())
        s1.record()
        barrier()
        eng.set_launch_overlap(0)
        return s0.elapsed_time(s1) / args.steps
    ms_hidden = chained_train(2)
    ms_overlap = chained_train(1)
    # the timed region is short: keep the device busy a little longer so that the clock record has samples under load
    if rank == 0:
        t_busy = time.perf_counter()
        while time.perf_counter() - t_busy < 0.6:
            for i in range(50):
                batch.launch(bufs[i % n_buf].data_ptr())
            torch.cuda.synchronize()
    clock_rec = clocks.stop() if rank == 0 else None
    t = torch.tensor([ms_total, ms_overlap, ms_hidden], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_overlap, ms_hidden = float(t[0].item()), float(t[1].item()), float(t[2].item())
    ms_step = ms_total / args.steps

    # ---- end to end through the public call: pinned host logits in, tokens out, every step
    host = [torch.empty(ROWS, VOCAB, dtype=torch.float32, pin_memory=True) for _ in range(2)]
    for h, b in zip(host, bufs):
        h.copy_(b)
    torch.cuda.synchronize()
    host_np = [h.numpy() for h in host]
    e2e_steps = max(5, min(40, args.steps // 10))
    for i in range(3):
        eng.sample_batch(sids, host_np[i % 2], hists)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        eng.sample_batch(sids, host_np[i % 2], hists)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    h2d = ROWS * VOCAB * 4 + ROWS * 64 + ROWS * HIST * 4
    d2h = ROWS * 4 + 4

    # ---- parity of the timed batch and of the fused-softcap variant (rank 0, outside the timed region)
    parity, softcap_mism = None, None
    if rank == 0:
        try:
            from oracle import Oracle
            orc = Oracle()
            # the batch's engine words were drawn when it was prepared: the first output of every stream
            ref = orc.sample_rows(params, orc.new_rngs(params["seed"]), own_logits.copy(), hists)
            parity = int((ref["tokens"] != tokens).sum())
            s2 = eng.open_streams(params)
            softcap_mism = softcap_mismatches(fb, eng, s2, raw_logits, ref["tokens"], hists)
        except Exception as ex:   # the checker is optional here; tests/ are the gate
            parity = f"not checked: {ex}"

    # ---- side figures, outside the headline.  Skipped with --no-extras.
    peak, peak_src = measured_hbm_peak()
    extras = None
    if not args.no_extras:
        extras = {}
        try:
            eng.set_launch_overlap(0)
            for resident in (False, True):   # the whole public call on device-resident logits, as a server makes it every step
                if resident:
                    for s_, hh_ in zip(sids, hists):
                        eng.history_set(int(s_), hh_)
                call = (lambda i: eng.sample_batch_resident(sids, bufs[i % n_buf].data_ptr(), n_vocab=VOCAB)) if resident else \
                       (lambda i: eng.sample_batch(sids, bufs[i % n_buf], hists, n_vocab=VOCAB))
                extras["device_logits_call_us_resident_histories" if resident else "device_logits_call_us"] = time_calls(call, 100)
            extras["staging_h2d_bytes"] = ROWS * 64 + ROWS * HIST * 4
            extras["warm_launch_us"] = time_launches(torch, lambda i: batch.launch(bufs[0].data_ptr()), 100)   # the same 67 MB every launch: mostly L2
            if rank == 0:
                extras["configs"] = config_figures(torch, fb, device, peak, tanhf)
                extras["c_call_latency"] = c_call_latency(fb)
        except Exception as ex:   # side figures must never cost the headline line
            extras["error"] = f"{type(ex).__name__}: {ex}"
        if world > 1:   # (every rank reaches this point: the figures above involve no collective and are guarded per rank)
            try:
                extras["cfg5_vocab_sharded"] = vocab_sharded_leg(torch, dist, fb, device, rank, world, barrier)
            except Exception as ex:
                extras["cfg5_vocab_sharded"] = {"error": f"{type(ex).__name__}: {ex}"}
    batch.free()

    if rank == 0:
        bytes_launch = algorithmic_bytes()
        achieved = bytes_launch / (ms_step * 1e-3) / 1e9
        overlapped = bytes_launch / (ms_overlap * 1e-3) / 1e9
        out = {
            "metric": METRIC, "value": world * ROWS / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/f64", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "global_rows": world * ROWS, "vocab": VOCAB, "parallelism": f"rows{world}",
                       "cache": f"logits rotate through {n_buf} buffers of {ROWS * VOCAB * 4 / 1e6:.0f} MB (> L2), inputs larger than L2",
                       "launches": "one stream, no overlap: a launch starts when the one before has finished", "host_binding": numa},
            "logits_gb_s": world * ROWS * VOCAB * 4 / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": bytes_launch, "frac_of_nominal_8000": achieved / 8000.0,
                         "kernel": "stream_select_kernel", "launch_us": ms_step * 1e3,
                         "note": "achieved = algorithmic bytes / duration of one launch in the timed train (no overlap between launches)"},
            "hidden_launch_latency_train": {"step_us": ms_hidden * 1e3, "rows_per_s": world * ROWS / (ms_hidden * 1e-3),
                                            "achieved_gb_s": bytes_launch / (ms_hidden * 1e-3) / 1e9, "frac": bytes_launch / (ms_hidden * 1e-3) / 1e9 / peak,
                                            "note": "fsb_set_launch_overlap(2): every CTA waits for the previous launch to complete before its first "
                                                    "access; same results and ordering as the plain train"},
            "overlapped_train": {"step_us": ms_overlap * 1e3, "rows_per_s": world * ROWS / (ms_overlap * 1e-3), "achieved_gb_s": overlapped, "frac": overlapped / peak,
                                 "note": "programmatic stream serialization on: independent batches only"},
            "e2e": {"value": world * ROWS * e2e_steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1e3 * e2e_s / e2e_steps, "steps": e2e_steps, "h2d_gb_s_per_rank": h2d / (e2e_s / e2e_steps) / 1e9,
                    "call": "fsb_sample_batch(FSB_LOGITS_ON_HOST), pinned host logits"},
            "gpu_launches": args.steps * kernels_per_step,
            "clocks": clock_rec,
            "parity_mismatches_timed_batch": parity,
            "fused_softcap_mismatches_of_64_rows": softcap_mism,
        }
        if extras is not None:
            out["extras"] = extras
        if world == 1 and not args.no_cpu_baseline:
            val, single, threads, kind, sample = cpu_baseline_cfg3(10.0)
            out["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample, "single_thread_value": single}
        print(json.dumps(out), flush=True)
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
