#!/usr/bin/env python
"""Benchmark of the B200 batched token sampler on the headline configuration (B = 64 rows, V = 262144 fp32 logits).

    python bench.py --gpus 1 --steps 400 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      (the reference's CPU sampler on the host cores, same workload)

A step is one pass of the sampler over one batch: Student-t(3) * 4 logits soft-capped at 30, temperature 1,
top-k 64, top-p 0.95, repetition penalty 1.0 / 1.1 on alternating rows over 512-id histories.  Data is synthetic
and seeded.  With N GPUs every rank samples its own batch of 64 rows (rows are independent streams: row
sharding, no data-path collective), so scaling is weak and `value` is the rows of all ranks per second.

Timing: CUDA events on the launching stream around exactly K back-to-back launches after W warm-up launches, a
barrier and a device synchronisation on both sides, the maximum over ranks.  The logits rotate through a set of
buffers larger than L2, so every step reads its logits from HBM.  `e2e` is the same batch through the public call
`fsb_sample_batch` with the logits in pinned host memory (host-to-device copy and token read-back inside the timed
region).  PyTorch is used for device memory, streams and the process group only; the sampler is the C-ABI library.
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
NCU_TRAFFIC_BYTES = 67.27e6 + 1.27e6


def algorithmic_bytes(rows=ROWS, vocab=VOCAB, hist=HIST):
    """Bytes one launch must move: the logits once, the penalty-window ids, one engine word and one token per row."""
    return rows * (4 * vocab + 4 * hist + 8 + 4)


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    except Exception:
        return 6650.0, "fallback (earlier measurement on this pool)"


def make_params(rank):
    import ferro_b200 as fb
    p = fb.make_params(ROWS, temperature=1.0, top_k=TOP_K, top_p=0.95, min_p=0.0, repetition_penalty=1.0, repeat_last_n=-1, penalty_from=0)
    p["repetition_penalty"][1::2] = 1.1
    p["seed"] = 7 + 1000 * rank + np.arange(ROWS)
    return p


def make_histories(rank):
    rng = np.random.default_rng(700 + rank)
    return [rng.integers(0, VOCAB, size=HIST).astype(np.int32) for _ in range(ROWS)]


def device_logits(torch, gen, device):
    """Student-t(3) * 4, then 30 * tanh(x / 30): the Gemma-4-style large-vocabulary row."""
    z = torch.randn(ROWS, VOCAB, device=device, generator=gen)
    den = torch.zeros(ROWS, VOCAB, device=device)
    for _ in range(3):
        den += torch.randn(ROWS, VOCAB, device=device, generator=gen) ** 2
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


def cpu_reference_rows_per_s(seconds_budget=12.0, threads=None, rows=ROWS):
    """Times the reference's own CPU sampler (compiled unmodified into oracle/_ref; else the C port of it) on the
    host cores on this workload.  Returns (all-threads rows/s, single-thread rows/s, threads, kind, sample text)."""
    from oracle import Oracle, RefLib
    from ferro_b200 import synth
    cfg = synth.config3(rows=rows)
    lg, hists = cfg["logits"], cfg["hists"]
    p = make_params(0)[:rows]
    n_threads = threads or (os.cpu_count() or 1)
    if RefLib.available():
        ref = RefLib()
        kind = "reference"

        def one_pass(nt):
            secs, _ = ref.time_rows(p, lg.copy(), hists, nt)
            return secs
    else:
        orc = Oracle()
        kind = "port"

        def one_pass(nt):
            x = lg.copy()
            rngs = orc.new_rngs(p["seed"])
            t0 = time.perf_counter()
            if nt == 1:
                orc.sample_rows(p, rngs, x, hists)
            else:   # ctypes releases the GIL: row blocks run on Python threads
                bounds = [rows * t // nt for t in range(nt + 1)]
                ths = [threading.Thread(target=orc.sample_rows, args=(p[a:b], rngs[a:b], x[a:b], hists[a:b])) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]
                [t.start() for t in ths]
                [t.join() for t in ths]
            return time.perf_counter() - t0
    one_pass(1)
    single, multi, passes = [], [], 0
    t_end = time.perf_counter() + seconds_budget
    while (passes < 3 or time.perf_counter() < t_end) and passes < 200:
        single.append(one_pass(1))
        multi.append(one_pass(min(n_threads, rows)))
        passes += 1
    s1, sm = float(np.median(single)), float(np.median(multi))
    sample = f"{passes} passes over {rows} rows x {VOCAB} (median), fresh logits copy per pass, sample() calls only"
    return rows / sm, rows / s1, min(n_threads, rows), kind, sample


def run_reference_arm(args, rank):
    if rank != 0:
        return
    steps_budget = max(4.0, min(60.0, 0.15 * (args.steps + args.warmup)))
    val, single, threads, kind, sample = cpu_reference_rows_per_s(seconds_budget=steps_budget)
    out = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * ROWS / val, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "vocab": VOCAB},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample, "single_thread_value": single},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def _time_launches(torch, launch, n):
    """Microseconds per call of `launch(i)` over n back-to-back calls, CUDA events on the current stream."""
    for i in range(3):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / n


def side_figures(torch, dist, fb, eng, device, rank, world, sids, hists, bufs, barrier):
    """Figures that explain the headline but are not it.  All device-timed, launch overlap off."""
    from ferro_b200 import sharded
    out = {}
    eng.set_launch_overlap(False)
    gen = torch.Generator(device=device)
    gen.manual_seed(99 + rank)
    try:   # nothing in here is collective: a rank that fails still reaches the collective part below
        # the whole public call with device-resident logits, as a server makes it every step: stage descriptors and the
        # 512-id windows (one host-to-device copy), launch, read the tokens back, synchronise; and the same with the
        # histories resident on the device (only descriptors go up)
        for resident in (False, True):
            if resident:
                for s_, hh_ in zip(sids, hists):
                    eng.history_set(int(s_), hh_)
            call = (lambda i: eng.sample_batch_resident(sids, bufs[i % len(bufs)].data_ptr(), n_vocab=VOCAB)) if resident else \
                   (lambda i: eng.sample_batch(sids, bufs[i % len(bufs)], hists, n_vocab=VOCAB))
            for i in range(3):
                call(i)
            t0 = time.perf_counter()
            n_call = 100
            for i in range(n_call):
                call(i)
            out["device_logits_call_us_resident_histories" if resident else "device_logits_call_us"] = 1e6 * (time.perf_counter() - t0) / n_call
        out["staging_h2d_bytes"] = ROWS * 64 + ROWS * HIST * 4
        # warm: the same 67 MB buffer every launch (mostly L2-resident)
        batch = eng.prepare_batch(sids, hists, VOCAB)
        out["warm_launch_us"] = _time_launches(torch, lambda i: batch.launch(bufs[0].data_ptr()), 100)
        batch.free()
        # other shapes through the same kernel (seeded normal logits; the value distribution does not matter for time)
        gen = torch.Generator(device=device)
        gen.manual_seed(99 + rank)
        rng = np.random.default_rng(5)
        for name, rows, vocab, k, hl, temp in (("cfg5_512x262144_k40", 512, 262144, 40, 1024, 0.8), ("cfg4_136x65536_greedy", 136, 65536, 1, 0, 0.0),
                                               ("cfg2_like_8x65536_k50", 8, 65536, 50, 256, 0.8)):
            big = [torch.randn(rows, vocab, device=device, generator=gen) * 3.0 for _ in range(2 if rows * vocab > 5e7 else 8)]
            p = fb.make_params(rows, temperature=temp, top_k=max(k, 1), top_p=0.9, repetition_penalty=1.1 if hl else 1.0)
            p["seed"] = 99 + np.arange(rows)
            hh = [rng.integers(0, vocab, size=hl).astype(np.int32) for _ in range(rows)]
            e2 = fb.Engine(device=device.index, max_rows=rows, max_vocab=vocab, max_hist_ids=rows * max(hl, 1) + 16)
            e2.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
            s2 = e2.open_streams(p)
            b2 = e2.prepare_batch(s2, hh, vocab)
            us = _time_launches(torch, lambda i: b2.launch(big[i % len(big)].data_ptr()), 40)
            out[name] = {"launch_us": us, "logits_gb_s": rows * vocab * 4 / us / 1e3, "rows_per_s": rows / us * 1e6}
            b2.free()
            e2.close()
            del big
    except Exception as ex:
        out["error"] = f"{type(ex).__name__}: {ex}"
    if world > 1:
        # (every rank reaches this point: the figures above involve no collective and are guarded per rank)
        # the serving batch split by vocabulary: every rank holds V / world columns of all 512 rows, selects its
        # candidates, one NCCL all-gather, merge on every rank (ferro_b200.sharded.VocabShardedSampler)
        rows, vocab = 512, 262144
        lo, hi = sharded.vocab_partition(vocab, world)[rank]
        ready, e3, b3 = 1, None, None
        try:
            shard = [torch.randn(rows, hi - lo, device=device, generator=gen) * 3.0 for _ in range(2)]
            p = fb.make_params(rows, temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1)
            p["seed"] = 99 + np.arange(rows)                       # the same streams on every rank
            hh = [np.random.default_rng(1000 + r).integers(0, vocab, size=1024).astype(np.int32) for r in range(rows)]
            e3 = fb.Engine(device=device.index, max_rows=rows, max_vocab=hi - lo, max_hist_ids=rows * 1024 + 16)
            e3.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
            e3.set_vocab_offset(lo)
            s3 = e3.open_streams(p)
            b3 = e3.prepare_batch(s3, hh, hi - lo)
            lists = torch.zeros((rows, sharded.MAX_K), dtype=torch.int64, device=device)
            counts = torch.zeros((rows,), dtype=torch.int32, device=device)
        except Exception:
            ready = 0
        flag = torch.tensor([ready], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)            # every rank takes part in the collectives below, or none
        if int(flag.item()) == 1:
            def step(i):
                b3.shard_launch(shard[i % 2].data_ptr(), lists.data_ptr(), counts.data_ptr())
                al, ac = sharded.gather_candidate_lists(lists, counts)
                b3.merge_launch(al.data_ptr(), ac.data_ptr(), world)
            barrier()
            us = _time_launches(torch, step, 30)
            t = torch.tensor([us], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out["cfg5_vocab_sharded"] = {"step_us": float(t.item()), "rows_per_s": rows / float(t.item()) * 1e6, "columns_per_gpu": hi - lo,
                                         "exchange": "NCCL all-gather of 512 x 256 x 8 B + 512 x 4 B per rank"}
        if b3 is not None:
            b3.free()
        if e3 is not None:
            e3.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the side figures (staging, warm launch, other shapes, vocabulary sharding)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

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

    # ---- workload, resident in HBM before anything is timed
    gen = torch.Generator(device=device)
    gen.manual_seed(7 + rank)
    n_buf = 8   # 8 x 67 MB = 537 MB, more than four times the 126 MB L2: every step streams from HBM
    bufs = [device_logits(torch, gen, device) for _ in range(n_buf)]
    params, hists = make_params(rank), make_histories(rank)
    eng = fb.Engine(device=local_rank, max_rows=ROWS, max_vocab=VOCAB, max_hist_ids=2 * ROWS * HIST + 16)
    eng.set_cuda_stream(torch.cuda.current_stream().cuda_stream)
    sids = eng.open_streams(params)
    batch = eng.prepare_batch(sids, hists, VOCAB)
    kernels_per_step = batch.kernels_per_launch

    # The timed steps are a train of launches on one stream with launch overlap on: a launch may begin to read its
    # logits while the previous one is finishing, its writes wait for it (the buffers were all filled beforehand).
    # The same train with overlap off, timed right after, gives the duration of one launch on its own.
    eng.set_launch_overlap(True)
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
    tokens = batch.tokens()
    eng.set_launch_overlap(False)
    for i in range(3):
        batch.launch(bufs[i % n_buf].data_ptr())
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for i in range(args.steps):
        batch.launch(bufs[i % n_buf].data_ptr())
    s1.record()
    barrier()
    ms_serial = s0.elapsed_time(s1) / args.steps
    # the timed region is short: keep the device busy a little longer so that the clock record has samples under load
    if rank == 0:
        t_busy = time.perf_counter()
        while time.perf_counter() - t_busy < 0.6:
            for i in range(50):
                batch.launch(bufs[i % n_buf].data_ptr())
            torch.cuda.synchronize()
    clock_rec = clocks.stop() if rank == 0 else None
    t = torch.tensor([ms_total, ms_serial], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_serial = float(t[0].item()), float(t[1].item())
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

    # ---- side figures, outside the headline: staging cost, a warm (L2-resident) launch, two other shapes, and with
    # several GPUs the vocabulary-sharded variant of the serving batch.  Skipped with --no-extras.
    extras = None
    if not args.no_extras:
        try:
            extras = side_figures(torch, dist, fb, eng, device, rank, world, sids, hists, bufs, barrier)
        except Exception as ex:   # side figures must never cost the headline line
            extras = {"error": f"{type(ex).__name__}: {ex}"}

    # ---- parity of the last timed batch (outside the timed region; rank 0)
    parity = None
    if rank == 0:
        try:
            from oracle import Oracle
            orc = Oracle()
            # the batch's engine words were drawn when it was prepared: the first output of every stream
            ref = orc.sample_rows(params, orc.new_rngs(params["seed"]), bufs[(args.steps - 1) % n_buf].cpu().numpy(), hists)
            parity = int((ref["tokens"] != tokens).sum())
        except Exception as ex:   # the checker is optional here; tests/ are the gate
            parity = f"not checked: {ex}"

    if rank == 0:
        peak, peak_src = measured_hbm_peak()
        bytes_launch = algorithmic_bytes()
        achieved = bytes_launch / (ms_serial * 1e-3) / 1e9          # one launch on its own: the kernel's figure
        pipelined = bytes_launch / (ms_step * 1e-3) / 1e9           # the timed train of overlapping launches
        out = {
            "metric": METRIC, "value": world * ROWS / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/f64", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "global_rows": world * ROWS, "vocab": VOCAB, "parallelism": f"rows{world}",
                       "cache": f"logits rotate through {n_buf} buffers of {ROWS * VOCAB * 4 / 1e6:.0f} MB (> L2), inputs larger than L2",
                       "launches": "one stream, launch overlap on (programmatic stream serialization): a launch's reads may overlap the previous launch's tail"},
            "logits_gb_s": world * ROWS * VOCAB * 4 / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": bytes_launch, "frac_of_nominal_8000": achieved / 8000.0,
                         "kernel": "stream_select_kernel", "launch_us": ms_serial * 1e3,
                         "note": "achieved = algorithmic bytes / duration of one launch in a train without overlap; pipelined_* = the same per step of the timed train with overlap",
                         "pipelined_achieved": pipelined, "pipelined_frac": pipelined / peak, "pipelined_step_us": ms_step * 1e3},
            "e2e": {"value": world * ROWS * e2e_steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1e3 * e2e_s / e2e_steps, "steps": e2e_steps, "call": "fsb_sample_batch(FSB_LOGITS_ON_HOST), pinned host logits"},
            "gpu_launches": args.steps * kernels_per_step,
            "clocks": clock_rec,
            "parity_mismatches_last_batch": parity,
        }
        if extras is not None:
            out["extras"] = extras
        if world == 1 and not args.no_cpu_baseline:
            val, single, threads, kind, sample = cpu_reference_rows_per_s(seconds_budget=10.0)
            out["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample, "single_thread_value": single}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
