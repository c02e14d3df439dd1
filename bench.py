#!/usr/bin/env python
"""Benchmark of the tensor-op hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--no-ops]

Headline workload (one "step" = one launch of the fused residual-add + RMSNorm
kernel over one batch): configuration 2 of the baseline at its largest shape,
rows = 65536, hidden = 4096, fp16 in/out with fp32 accumulation, per GPU (weak
scaling: token rows are independent, so ranks share nothing and no collective is
on the data path).  The working set (2.1 GB per GPU) is far larger than L2.

One JSON line is printed by rank 0.  Beside the contract keys it carries
  roofline      achieved algorithmic GB/s of the kernel vs the measured HBM copy peak
  cpu_baseline  the reference's own CPU operators timed on this box's host cores
  e2e           the same metric with host buffers: pinned H2D of both inputs, the kernel,
                D2H of both outputs, every step
  ops           per-operator GB/s (and rows/s) of the other benchmark configurations
Inputs are synthetic (seeded normal / uniform draws of the named shapes); no dataset is involved.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, HIDDEN = 65536, 4096
METRIC = "fused_add_rmsnorm_hbm_gbs"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the headline kernel, from an ncu capture
# at 16384 rows scaled to 65536 (None until a capture of this build exists).
HEADLINE_TRAFFIC_BYTES = 1944171520  # 4 x (268.458 + 217.584) MB


def algorithmic_bytes(rows: int, hidden: int, elem: int = 2) -> int:
    """Two inputs read, two outputs written, one weight vector read."""
    return 4 * rows * hidden * elem + hidden * elem


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def config_block(n_gpus: int):
    return {"workload": f"config2 fused residual-add + RMSNorm, rows={ROWS} x hidden={HIDDEN} per GPU, fp16 in/out, "
                        f"fp32 accumulation, eps=1e-6",
            "rows_per_gpu": ROWS, "hidden": HIDDEN, "parallelism": f"row-sharded x{n_gpus}, no collective",
            "l2": "inputs (2.1 GB per GPU) larger than L2, no flush needed"}


# ------------------------------------------------------------------------------------------
# clocks: NVML reads only (never sets anything)
# ------------------------------------------------------------------------------------------

class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------
# CPU baseline: the reference's own operators (oracle/_ref) or, without them, the C port
# ------------------------------------------------------------------------------------------

def cpu_baseline(target_seconds: float, steps: int = 1, warmup: int = 0):
    """Times add + rms_norm as the reference's CPU layer runs them, rows split over all host
    threads.  Returns (equivalent GB/s of the fp16 workload's algorithmic bytes, description dict)."""
    import numpy as np
    import oracle
    ref = oracle.ref()
    rng = np.random.default_rng(2000)
    w = (rng.random(HIDDEN, dtype=np.float32) + np.float32(0.5))

    def make(rows):
        return rng.standard_normal((rows, HIDDEN), dtype=np.float32), rng.standard_normal((rows, HIDDEN), dtype=np.float32)

    if ref is not None:
        kind, cores = "reference", max(1, ref.hardware_threads())
        run = lambda x, r: ref.time_add_rms_norm(x, r, w, 1e-6, cores)
    else:
        kind, cores = "port", 1
        port = oracle.port()

        def run(x, r):
            t0 = time.perf_counter()
            port.add_rms_norm(x, r, w, 1e-6)
            return time.perf_counter() - t0
    probe_rows = 64 * cores
    x, r = make(probe_rows)
    run(x, r)
    rate = probe_rows / run(x, r)
    rows = int(min(ROWS, max(probe_rows, rate * target_seconds)))
    x, r = make(rows)
    for _ in range(warmup):
        run(x, r)
    times = [run(x, r) for _ in range(max(1, steps))]
    per_step = sum(times) / len(times)
    gbs = algorithmic_bytes(rows, HIDDEN) / per_step / 1e9
    return gbs, per_step, {"value": round(gbs, 4), "unit": UNIT, "cores": cores, "kind": kind,
                           "rows_per_s": round(rows / per_step, 1),
                           "sample": f"{rows} of {ROWS} rows x hidden {HIDDEN}, fp16 inputs de-quantised to the fp32 the "
                                     f"CPU operators take; GB/s counts the fp16 workload's algorithmic bytes per row"}


def cpu_operator_table():
    """The reference's unmodified CPU operators (oracle/_ref; the C port where the reference has no CPU form) on
    bounded samples of the configurations' shapes: single thread as the reference runs them, and rows split over all
    host threads.  A reported baseline: rows/s and the GB/s those rows are worth in the fp16/fp32 GPU workload."""
    import concurrent.futures as cf
    import numpy as np
    import oracle
    ref, port = oracle.ref(), oracle.port()
    if ref is None:
        return {"unavailable": "oracle/_ref/liboracle_ref.so was not built (reference tree absent at build time)"}
    threads = max(1, ref.hardware_threads())
    rng = np.random.default_rng(7)
    f = np.float32
    table = []

    def timed(fn):
        fn()
        t0 = time.perf_counter()
        fn()
        return time.perf_counter() - t0

    def entry(op, shape, rows, gpu_bytes_per_row, single, chunked, kind="reference"):
        t1 = timed(single)
        tn = timed(chunked) if chunked is not None else None
        e = {"op": op, "sample": shape, "kind": kind, "single_thread_rows_per_s": round(rows / t1, 1),
             "single_thread_gbs_equivalent": round(rows * gpu_bytes_per_row / t1 / 1e9, 4)}
        if tn is not None:
            e.update({"threads": threads, "all_threads_rows_per_s": round(rows / tn, 1),
                      "all_threads_gbs_equivalent": round(rows * gpu_bytes_per_row / tn / 1e9, 4)})
        table.append(e)

    def split(fn, *arrays):
        """fn over disjoint row slices of the arrays, one slice per host thread (ctypes releases the GIL)."""
        n = arrays[0].shape[0]
        bounds = [(n * i // threads, n * (i + 1) // threads) for i in range(threads)]

        def run():
            with cf.ThreadPoolExecutor(threads) as pool:
                list(pool.map(lambda b: fn(*[a[b[0]:b[1]] for a in arrays]) if b[1] > b[0] else None, bounds))
        return run

    w4096 = (rng.random(4096, dtype=f) + f(0.5))
    x = rng.standard_normal((2048, 4096), dtype=f)
    entry("rms_norm", "2048 x 4096 f32", 2048, 2 * 4096 * 2, lambda: ref.rms_norm(x, w4096, 1e-6),
          split(lambda a: ref.rms_norm(a, w4096, 1e-6), x))
    g, u = rng.standard_normal((1024, 3072), dtype=f) * 2, rng.standard_normal((1024, 3072), dtype=f) * 2
    entry("swiglu", "1024 x 3072 f32", 1024, 3 * 3072 * 2, lambda: ref.swiglu(g, u), split(lambda a, b: ref.swiglu(a, b), g, u))
    q = rng.standard_normal((1024, 24, 128), dtype=f)
    pos = rng.integers(0, 512, 1024).astype(np.int32)
    w128 = (rng.random(128, dtype=f) + f(0.5))
    qk = lambda a, p: ref.rope(ref.rms_norm(a.reshape(-1, 128), w128, 1e-6).reshape(a.shape), p, 1e6)
    entry("qk rms_norm + rope", "1024 tokens x 24 heads x 128 f32", 1024, 2 * 24 * 128 * 2 + 4, lambda: qk(q, pos), split(qk, q, pos))
    emb = rng.standard_normal((8192, 4096), dtype=f) * f(0.02)
    ids = rng.integers(0, 8192, 4096).astype(np.int32)
    entry("embedding_lookup", "4096 ids, table 8192 x 4096 f32", 4096, 2 * 4096 * 2 + 4, lambda: ref.embedding_lookup(emb, ids),
          split(lambda i: ref.embedding_lookup(emb, i), ids))
    logits = rng.standard_normal((16, 151936), dtype=f) * 4
    entry("softmax_last_dim", "16 x 151936 f32", 16, 2 * 151936 * 4, lambda: ref.softmax(logits), split(lambda a: ref.softmax(a), logits))
    entry("argmax (C restatement of the device rule: the reference has no CPU argmax)", "16 x 151936 f32", 16, 151936 * 4,
          lambda: port.argmax_rows(logits), None, kind="port")
    entry("sample top_k=50 top_p=0.95 (C restatement of the device rule)", "4 x 151936 f32", 4, 151936 * 4,
          lambda: [port.sample_row(logits[r], 0.8, 50, 0.95, 7, r) for r in range(4)], None, kind="port")
    lm_table = rng.standard_normal((16384, 1024), dtype=f) * f(0.02)
    lm_hidden = rng.standard_normal((1, 1024), dtype=f)
    entry("lm_head, one hidden row (unit: table rows; 16384 of the vocabulary's 151936, cost is linear in them)",
          "1 x 1024 by 16384 x 1024 f32", 16384, 1024 * 2, lambda: ref.lm_head(lm_hidden, lm_table),
          split(lambda t: ref.lm_head(lm_hidden, t), lm_table))
    return {"threads_available": threads, "entries": table}


def reference_gpu_kernels(L, lib, dev, stream):
    """The reference's own CUDA operators (src/ops_cuda.cu recompiled for sm_100a, oracle/_ref/libref_cuda.so)
    timed on this GPU beside ours, same shapes, device-resident tensors, CUDA events.  A reported baseline."""
    import torch
    import oracle
    from cuda_llm_b200 import ops
    ref = oracle.ref_cuda()
    if ref is None:
        return {"unavailable": "oracle/_ref/libref_cuda.so was not built (reference tree absent at build time)"}
    s = stream.cuda_stream
    half = torch.float16

    def ours(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    out = {}

    def row(name, ref_ms, our_ms, note=None):
        out[name] = {"reference_ms": round(ref_ms, 4), "ours_ms": round(our_ms, 4), "speedup": round(ref_ms / our_ms, 1)}
        if note:
            out[name]["note"] = note

    rows, hidden = ROWS, HIDDEN
    x, y = torch.randn(rows, hidden, device=dev).to(half), torch.randn(rows, hidden, device=dev).to(half)
    g = (torch.rand(hidden, device=dev) + 0.5).to(half)
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    row(f"add_rms_norm {rows}x{hidden} f16", ref.time_add_rms_norm(x, y, g, rows, hidden, 1e-6, 1, 2),
        ours(lambda: lib.check(L.b2_add_rms_norm(x.data_ptr(), y.data_ptr(), g.data_ptr(), o1.data_ptr(), o2.data_ptr(), rows,
                                                 hidden, 1e-6, lib.F16, lib.FAST, s))))
    row(f"rms_norm {rows}x{hidden} f16", ref.time_rms_norm(x, g, rows, hidden, 1e-6, 1, 2),
        ours(lambda: lib.check(L.b2_rms_norm(x.data_ptr(), g.data_ptr(), o1.data_ptr(), rows, hidden, 1e-6, lib.F16, lib.FAST, s))))
    n = rows * hidden
    row(f"add {rows}x{hidden} f16", ref.time_binary(x, y, n, 1, False, 3),
        ours(lambda: lib.check(L.b2_add(x.data_ptr(), y.data_ptr(), o1.data_ptr(), n, lib.F16, s))))
    row(f"swiglu {rows}x{hidden} f16", ref.time_binary(x, y, n, 1, True, 3),
        ours(lambda: lib.check(L.b2_swiglu(x.data_ptr(), y.data_ptr(), o1.data_ptr(), n, lib.F16, lib.FAST, s))))
    del x, y, o1, o2
    T = 16384
    q, k = torch.randn(T, 16, 128, device=dev).to(half), torch.randn(T, 8, 128, device=dev).to(half)
    g128 = (torch.rand(128, device=dev) + 0.5).to(half)
    pos = torch.randint(0, 512, (T,), device=dev, dtype=torch.int32)
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    ref_ms = (ref.time_rms_norm(q, g128, T * 16, 128, 1e-6, 1, 3) + ref.time_rms_norm(k, g128, T * 8, 128, 1e-6, 1, 3) +
              ref.time_rope_token_positions(q, pos, T, 16, 1e6, 3) + ref.time_rope_token_positions(k, pos, T, 8, 1e6, 3))
    row("qk_norm + rope, T=16384, 16+8 heads x 128 f16", ref_ms,
        ours(lambda: lib.check(L.b2_qk_norm_rope(q.data_ptr(), k.data_ptr(), g128.data_ptr(), g128.data_ptr(), pos.data_ptr(),
                                                 qo.data_ptr(), ko.data_ptr(), T, 16, 8, 128, 1e-6, 1e6, lib.F16, None, s))),
        note="reference: its four launches (rms_norm x2, rope_token_positions x2); ours: one fused launch")
    del q, k, qo, ko
    vocab, tokens = 151936, 262144
    table = (torch.randn(vocab, 4096, device=dev) * 0.02).to(half)
    ids = torch.randint(0, vocab, (tokens,), device=dev, dtype=torch.int32)
    gout = torch.empty(tokens, 4096, device=dev, dtype=half)
    row(f"embedding gather {tokens} rows x 4096 f16", ref.time_embedding(table, ids, tokens, 4096, vocab, 1, 3),
        ours(lambda: lib.check(L.b2_embedding_gather(table.data_ptr(), ids.data_ptr(), gout.data_ptr(), tokens, 4096, vocab,
                                                     lib.F16, None, s))))
    del table, gout
    R = 256
    logits = torch.randn(R, vocab, device=dev) * 4
    ids_out = torch.empty(R, dtype=torch.int32, device=dev)
    ws = ops.argmax_workspace(dev, R)
    row(f"argmax of {R} rows x {vocab} f32", R * ref.time_argmax_last_row(logits, R, vocab, 0, 5),
        ours(lambda: lib.check(L.b2_argmax_rows(logits.data_ptr(), R, vocab, vocab, lib.F32, ids_out.data_ptr(), ws.data_ptr(), s))),
        note="reference: one blocking call per row (2 cudaMalloc + 2 cudaFree + a D2H copy each), timed on one row x 256")
    sws, sout = ops.softmax_workspace(dev, R), torch.empty_like(logits)
    row(f"softmax {R}x{vocab} f32", ref.time_softmax(logits, R, vocab, 0, 1),
        ours(lambda: lib.check(L.b2_softmax_rows(logits.data_ptr(), sout.data_ptr(), R, vocab, lib.F32, lib.FAST, sws.data_ptr(), s))))
    # decode tail: the reference's cuda_lm_head (library GEMM into a fresh logits tensor) + cuda_argmax_last_row
    for R in (1, 4, 64):
        hid = torch.randn(R, 1024, device=dev).to(half)
        emb = (torch.randn(vocab, 1024, device=dev) * 0.02).to(half)
        lm_ids = torch.empty(R, dtype=torch.int32, device=dev)
        ref_ms = ref.time_lm_head_argmax(hid, emb, R, 1024, vocab, 1, 5)
        if ref_ms > 0:
            row(f"lm_head + argmax, {R} x 1024 by {vocab} x 1024 f16", ref_ms,
                ours(lambda: lib.check(L.b2_lm_head_argmax(hid.data_ptr(), emb.data_ptr(), R, 1024, vocab, lib.F16, lib.FAST, 0,
                                                           None, vocab, lm_ids.data_ptr(), None, ws.data_ptr(), s))),
                note="reference: cuda_lm_head (cuBLASLt GEMM, allocates the logits) + cuda_argmax_last_row (last row only, "
                     "blocking, 2 cudaMalloc + 2 cudaFree); ours: one launch, every row, ids stay on the device")
        del hid, emb
    # the launch-paced regime: one decoder layer's in-scope operators back to back (the reference's eight launches)
    if hasattr(ref.lib, "refcu_time_decode_chain"):
        for tokens in (1, 4, 64):
            out[f"decode layer chain, {tokens} tokens (reference: 8 launches)"] = {
                "reference_us_eager": round(ref.time_decode_chain(tokens, 1e-6, 1e6, 0, 200) * 1e3, 2),
                "reference_us_graph_replay": round(ref.time_decode_chain(tokens, 1e-6, 1e6, 1, 200) * 1e3, 2),
                "note": "ours: the `decode layer chain` entries of `ops` (5 launches)"}
    # sampling: the reference draws one token per blocking call; ours draws all rows in one call
    sampler_ws = torch.empty(L.b2_sampler_workspace_bytes(R, vocab), dtype=torch.uint8, device=dev)
    offs = torch.arange(R, dtype=torch.int64, device=dev)
    for label, temp, top_k, top_p, ref_reps in (("top_k=50 top_p=0.95", 0.8, 50, 0.95, 3), ("top_k=0 top_p=0.9", 1.0, 0, 0.9, 2)):
        per_row = ref.time_sample_row(logits, R, vocab, 0, temp, top_k, top_p, ref_reps)
        if per_row < 0:
            continue
        row(f"sample {R} rows x {vocab} f32, {label}", R * per_row,
            ours(lambda: lib.check(L.b2_sample_rows(logits.data_ptr(), R, vocab, vocab, lib.F32, temp, top_k, top_p, 7,
                                                    offs.data_ptr(), ids_out.data_ptr(), sampler_ws.data_ptr(), s)), reps=3),
            note="reference: one blocking CudaSampler::sample_row call per row (full-vocabulary sort + single-thread scans), "
                 "timed per row x 256")
    return out


def sharded_parity(dev, world, rank, calls=3):
    """Result check of every vocabulary-sharded form on the seeded configuration 5 (planted maxima), run by
    bench.py with N > 1 ranks outside all timed regions: ids bit-exact against the CPU oracle's argmax, this
    rank's columns of the softmax against the oracle's exact (fp64) softmax and its fp32 CPU operator under the
    rule of the GPU tests, over `calls` consecutive calls (both parities of the exchange buffers).  The oracle is
    only the checker here.  Returns {form: "ok" | "<what differed>"}, identical on every rank."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import oracle
    from cuda_llm_b200 import sharded, workloads as wl
    port = oracle.port()
    rows = 256
    c5 = wl.config5(rows=rows)
    x = c5["logits"]
    want_ids = port.argmax_rows(x)
    assert np.array_equal(want_ids, c5["planted"])
    lo, hi = sharded.column_range(wl.VOCAB, world, rank)
    exact = port.softmax_f64(x)
    floor = exact.max(axis=-1, keepdims=True)
    cpu = port.softmax(x).astype(np.float64)
    drift = float((np.abs(cpu - exact) / np.maximum(exact, floor)).max())
    exact, cpu = exact[:, lo:hi], cpu[:, lo:hi]
    shard = torch.from_numpy(np.ascontiguousarray(x[:, lo:hi])).to(dev)
    lm = wl.lm_head_case(4, 1024, wl.VOCAB, seed=6800, dtype=np.float16)
    planted = np.array([11, wl.VOCAB // 2 - 1, wl.VOCAB // 2, wl.VOCAB - 1], np.int32)
    for r in range(4):
        lm["table"][planted[r]] = (lm["hidden"][r].astype(np.float32) * np.float32(0.02)).astype(np.float16)
    hidden = torch.from_numpy(lm["hidden"]).to(dev)
    table_shard = torch.from_numpy(np.ascontiguousarray(lm["table"][lo:hi])).to(dev)
    del lm
    result = {}

    def ids_check(name, fn, want):
        bad = ""
        for call in range(calls):
            got = fn().cpu().numpy()
            if not np.array_equal(got, want):
                bad = bad or f"rank {rank} call {call}: {int((got != want).sum())} of {want.size} ids differ"
        result[name] = bad

    def softmax_check(name, fn):
        bad = ""
        for call in range(calls):
            got = fn().cpu().numpy().astype(np.float64)
            e_exact = float((np.abs(got - exact) / np.maximum(exact, floor)).max())
            e_cpu = float((np.abs(got - cpu) / np.maximum(exact, floor)).max())
            if not (e_exact <= 1e-5 and e_cpu <= 1e-5 + drift):
                bad = bad or f"rank {rank} call {call}: {e_exact:.2e} vs exact, {e_cpu:.2e} vs ops_cpu (its drift {drift:.2e})"
        result[name] = bad

    ex = sharded.PeerExchange(max_rows=rows)
    try:
        ids_check("argmax_nccl", lambda: sharded.sharded_argmax(shard, lo), want_ids)
        ids_check("argmax_fused", lambda: sharded.sharded_argmax_fused(shard, lo, ex), want_ids)
        softmax_check("softmax_nccl", lambda: sharded.sharded_softmax(shard))
        softmax_check("softmax_fused", lambda: sharded.sharded_softmax_fused(shard, ex))
        ids_check("lm_head_nccl", lambda: sharded.sharded_lm_head_argmax(hidden, table_shard, lo), planted)
        ids_check("lm_head_fused", lambda: sharded.sharded_lm_head_argmax_fused(hidden, table_shard, lo, ex), planted)
        if ex.timed_out():
            result["argmax_fused"] = result["argmax_fused"] or f"rank {rank}: a bounded wait for a peer ran out"
    finally:
        ex.close()
    # every rank reports the same verdict: the first complaint of any rank, or "ok"
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    return {k: next((g[k] for g in gathered if g[k]), "ok") for k in result}


_REAL_STDOUT = None


def emit(text: str) -> None:
    """The one JSON line, to the process's original stdout."""
    sys.stdout.flush()
    if _REAL_STDOUT is None:
        print(text)
    else:
        os.write(_REAL_STDOUT, (text + "\n").encode())


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    total = args.steps + args.warmup
    per_step = min(1.0, 120.0 / max(1, total))
    gbs, sec, desc = cpu_baseline(per_step, steps=args.steps, warmup=args.warmup)
    desc["value"] = round(gbs, 4)
    emit(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(gbs, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_block(args.gpus),
        "cpu_baseline": desc,
        "e2e": {"value": round(gbs, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------
# the B200 arm
# ------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-operator table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--rows", type=int, default=ROWS, help=argparse.SUPPRESS)   # smaller cases for profiler captures
    args = ap.parse_args()
    # stdout carries exactly one JSON line: anything a library prints there meanwhile (NCCL's version banner, for
    # one) goes to stderr instead; emit() writes to the real stdout
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from cuda_llm_b200 import build, lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    L = lib.load()
    warmup = max(args.warmup, 3)
    rows = args.rows

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    stream = torch.cuda.Stream(device=dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(2000 + rank)
    with torch.cuda.stream(stream):
        x = torch.randn(rows, HIDDEN, device=dev, dtype=torch.float32, generator=gen).half()
        res = torch.randn(rows, HIDDEN, device=dev, dtype=torch.float32, generator=gen).half()
        gamma = (torch.rand(HIDDEN, device=dev, generator=gen) + 0.5).half()
        out_res, out_nrm = torch.empty_like(x), torch.empty_like(x)

        def step():
            lib.check(L.b2_add_rms_norm(x.data_ptr(), res.data_ptr(), gamma.data_ptr(), out_res.data_ptr(),
                                        out_nrm.data_ptr(), rows, HIDDEN, 1e-6, lib.F16, lib.FAST, stream.cuda_stream))

        for _ in range(warmup):
            step()
        sampler = ClockSampler(local)
        barrier()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        local_ms = e0.elapsed_time(e1)
        total_ms = max_over_ranks(local_ms)
        ms_per_step = total_ms / args.steps
        alg = algorithmic_bytes(rows, HIDDEN)
        value = world * alg / (ms_per_step * 1e-3) / 1e9
        kernel_gbs = alg / (local_ms / args.steps * 1e-3) / 1e9

        # ---- end to end: host buffers in, host buffers out, every step (the public host-buffer call:
        # row chunks, copies in both directions overlapped with the kernel on three streams)
        from cuda_llm_b200 import hostio
        e2e_steps = max(1, min(args.steps, 10))
        hx = torch.empty(rows, HIDDEN, dtype=torch.float16).pin_memory()
        hr = torch.empty(rows, HIDDEN, dtype=torch.float16).pin_memory()
        hx.copy_(x, non_blocking=False)
        hr.copy_(res, non_blocking=False)
        h_res, h_nrm = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
        del x, res, out_res, out_nrm
        pipe = hostio.AddRmsNormHostPipeline(rows, HIDDEN, dev, chunks=8)
        pipe(hx, hr, gamma, h_res, h_nrm).synchronize()
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t0.record(pipe.s_in)
        for _ in range(e2e_steps):
            done = pipe(hx, hr, gamma, h_res, h_nrm)
        t1 = torch.cuda.Event(enable_timing=True)
        pipe.s_out.wait_event(done)
        t1.record(pipe.s_out)
        barrier()
        clocks = sampler.stop()
        e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / e2e_steps
        e2e_value = world * alg / (e2e_ms * 1e-3) / 1e9
        # the ceiling of that number on this box with this many ranks: the same pinned copies, no kernel
        pipe(hx, hr, gamma, h_res, h_nrm, copies_only=True).synchronize()
        barrier()
        c0 = torch.cuda.Event(enable_timing=True)
        c0.record(pipe.s_in)
        for _ in range(e2e_steps):
            done = pipe(hx, hr, gamma, h_res, h_nrm, copies_only=True)
        c1 = torch.cuda.Event(enable_timing=True)
        pipe.s_out.wait_event(done)
        c1.record(pipe.s_out)
        barrier()
        copy_ms = max_over_ranks(c0.elapsed_time(c1)) / e2e_steps
        del hx, hr, h_res, h_nrm, pipe

        op_table, parity_n, sharded_block = None, None, None
        if world > 1:
            torch.cuda.empty_cache()
            parity_n = sharded_parity(dev, world, rank)     # outside every timed region
        if not args.no_ops:
            import opbench
            torch.cuda.empty_cache()
            op_table = opbench.run(L, lib, dev, stream, world, rank, barrier, max_over_ranks)
            sharded_block = opbench.sharded_summary(op_table, world)
        ref_gpu = None
        if world == 1 and not args.no_ops and not args.no_cpu:
            torch.cuda.empty_cache()
            try:
                ref_gpu = reference_gpu_kernels(L, lib, dev, stream)
            except Exception as exc:      # a reported baseline, never required for our numbers
                ref_gpu = {"error": str(exc)}

    failed = parity_n is not None and any(v != "ok" for v in parity_n.values())
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if failed:
            raise SystemExit(3)
        return
    peak, peak_kind = measured_peak()
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 storage, f32 arithmetic", "data": "synthetic", "config": config_block(world),
        "rows_per_s": round(world * rows / (ms_per_step * 1e-3), 1),
        "frac_of_nominal_8TBs": round(value / world / NOMINAL_HBM_GBS, 4),
        "roofline": {"bound": "hbm", "achieved": round(kernel_gbs, 2), "peak": peak, "unit": UNIT,
                     "frac": round(kernel_gbs / peak, 4), "traffic": HEADLINE_TRAFFIC_BYTES, "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": alg, "kernel": "rms_norm_rows_kernel<__half, 2, true>"},
        "e2e": {"value": round(e2e_value, 3), "unit": UNIT, "h2d_bytes_per_step": 2 * rows * HIDDEN * 2,
                "d2h_bytes_per_step": 2 * rows * HIDDEN * 2, "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps,
                "how": "pinned host buffers; 8 row chunks; H2D, kernel and D2H overlapped on three streams",
                "host_copies_only_ms_per_step": round(copy_ms, 3),
                "frac_of_host_copy_ceiling": round(copy_ms / e2e_ms, 4)},
        "gpu_launches": args.steps, "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        try:
            _, _, line["cpu_baseline"] = cpu_baseline(10.0)
        except Exception as exc:  # the baseline is reported, never required for the GPU number
            line["cpu_baseline"] = {"error": str(exc)}
    if world == 1 and not args.no_cpu and not args.no_ops:
        try:
            line["cpu_ops"] = cpu_operator_table()
        except Exception as exc:
            line["cpu_ops"] = {"error": str(exc)}
    if op_table is not None:
        line["ops"] = op_table
    if ref_gpu is not None:
        line["reference_cuda_kernels_on_this_gpu"] = ref_gpu
    # last, so that they are what the end of the line shows: the multi-GPU numbers and result checks
    if sharded_block is not None:
        line["sharded"] = sharded_block
    if parity_n is not None:
        line["parity_n"] = parity_n
    emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit("bench.py: a multi-GPU result differs from the CPU oracle: " + json.dumps(parity_n))


if __name__ == "__main__":
    main()
