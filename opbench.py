"""Per-operator throughput table of the benchmark configurations (used by bench.py; also runs alone).

Every entry is timed with CUDA events on the launching stream after warm-up, over
`reps` back-to-back launches.  Working sets smaller than a few times L2 are rotated
through enough distinct buffer sets to exceed 512 MB, so the bytes really come from
HBM.  GB/s = algorithmic bytes / time: the bytes an ideal kernel must move (inputs
read once, outputs written once).

With several ranks the row-independent operators split configuration 4's T tokens
over the ranks (no collective) and the vocabulary reductions split V over the ranks
with the NCCL exchange inside the timed region; times are the maximum over ranks.
"""
from __future__ import annotations

import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

VOCAB = 151936
NOMINAL = 8000.0


def _peak():
    try:
        root = os.path.dirname(os.path.abspath(__file__))
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


def run(L, lib, dev, stream, world, rank, barrier, max_over_ranks, quick=False, only=None, reps_scale=1.0, sampler_rows=256):
    """only: substring selecting one group of entries ("add_rms_norm", "headline_shape", "qk_norm_rope",
    "swiglu", "gather", "argmax", "softmax", "sampler", "kvmove", "lm_head", "decode_chain"); reps_scale shortens the runs for profiler captures."""
    from cuda_llm_b200 import sharded

    def want(group):
        return only is None or only in group

    def nreps(n):
        return max(1, int(n * reps_scale))
    peak = _peak()
    s = stream.cuda_stream
    F16, F32, FAST = lib.F16, lib.F32, lib.FAST
    table = []
    half = torch.float16

    def randn(*shape, sigma=1.0, dtype=half):
        return (torch.randn(*shape, device=dev, dtype=torch.float32) * sigma).to(dtype)

    def timed(calls, reps, warm=3):
        """calls: list of zero-argument launchers (one per buffer set); returns ms per launch (max over ranks)."""
        n = len(calls)
        for i in range(warm):
            calls[i % n]()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(reps):
            calls[i % n]()
        e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / reps

    def sets_for(bytes_per_set):
        return max(1, min(8, -(-512 * 1024 * 1024 // max(1, bytes_per_set))))

    def record(op, shape, alg_bytes_local, ms, rows_local=None, note=None, sharded_over=1):
        gbs = sharded_over * alg_bytes_local / (ms * 1e-3) / 1e9
        e = {"op": op, "shape": shape, "us": round(ms * 1e3, 2), "gbs": round(gbs, 1),
             "frac_measured_copy": round(gbs / sharded_over / peak, 4), "frac_nominal": round(gbs / sharded_over / NOMINAL, 4)}
        if rows_local is not None:
            e["rows_per_s"] = round(sharded_over * rows_local / (ms * 1e-3), 1)
        if note:
            e["note"] = note
        table.append(e)

    # ---- configuration 2: fused add + RMSNorm sweep (single-GPU shapes; every rank runs them alike)
    for rows in ((1, 64, 4096, 65536) if want("add_rms_norm") else ()):
        for hidden in (1024, 2048, 4096):
            per_set = 4 * rows * hidden * 2
            n = sets_for(per_set) if rows >= 4096 else 1
            bufs = [(randn(rows, hidden), randn(rows, hidden), torch.empty(rows, hidden, device=dev, dtype=half),
                     torch.empty(rows, hidden, device=dev, dtype=half)) for _ in range(n)]
            g = (torch.rand(hidden, device=dev) + 0.5).half()
            calls = [(lambda b=b: lib.check(L.b2_add_rms_norm(b[0].data_ptr(), b[1].data_ptr(), g.data_ptr(),
                                                               b[2].data_ptr(), b[3].data_ptr(), rows, hidden, 1e-6, F16,
                                                               FAST, s))) for b in bufs]
            ms = timed(calls, nreps(20 if rows >= 4096 else 100))
            record("add_rms_norm", f"{rows}x{hidden} f16", per_set + 2 * hidden, ms, rows,
                   note=None if rows >= 4096 else "latency-bound: cannot fill the GPU")
            if rows <= 4096:
                # launches this short are paced by the host's launch path: the same launches recorded once into a CUDA
                # graph (24 in a row over the rotating buffer sets) and replayed give the device-side time per launch
                try:
                    K = 24
                    replayed = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(replayed, stream=stream):
                        for i in range(K):
                            calls[i % n]()
                    ms_g = timed([replayed.replay], nreps(10)) / K
                    gbs_g = (per_set + 2 * hidden) / (ms_g * 1e-3) / 1e9
                    table[-1].update({"us_graph_replay": round(ms_g * 1e3, 2), "gbs_graph_replay": round(gbs_g, 1),
                                      "frac_measured_copy_graph_replay": round(gbs_g / peak, 4)})
                    del replayed
                except Exception as exc:   # a measurement aid, not a requirement
                    table[-1]["graph_replay_error"] = str(exc)[:120]
            del bufs, calls
    if quick:
        return table

    if want("headline_shape"):
        _headline_shape_ops(L, lib, dev, s, timed, record, randn, nreps)
    if want("qk_norm_rope"):
        _config3(L, lib, dev, s, timed, record, randn, sets_for, nreps)
    if want("swiglu") or want("gather"):
        _config4(L, lib, dev, s, timed, record, randn, sharded, world, rank, want, nreps)
    if want("argmax") or want("softmax"):
        _config5(L, lib, dev, s, timed, record, randn, sets_for, sharded, world, rank, want, nreps, table, barrier)
    if world == 1 and want("copy"):
        # a yardstick measured in the same run with the same harness: plain device-to-device copies (torch's kernel, not
        # ours) of 1 GiB and of the byte counts of the two small configurations
        for label, nbytes in (("1 GiB each way", 1 << 30), ("100.7 MB each way (configuration 3's bytes)", 100_663_296),
                              ("155.6 MB each way (configuration 5's softmax bytes)", 155_582_464)):
            n = max(2, min(4, -(-512 * 1024 * 1024 // nbytes)))
            bufs = [(torch.empty(nbytes, dtype=torch.uint8, device=dev), torch.empty(nbytes, dtype=torch.uint8, device=dev))
                    for _ in range(n)]
            for a, _ in bufs:
                a.fill_(1)
            ms = timed([(lambda b=b: b[1].copy_(b[0])) for b in bufs], nreps(20))
            record("device copy (library kernel, yardstick only)", label, 2 * nbytes, ms)
            del bufs
    if world == 1 and (want("sampler") or want("kvmove")):
        _next_rows(L, lib, dev, s, timed, record, randn, want, nreps, sampler_rows, stream)
    if world == 1 and want("decode_chain"):
        _decode_chain(L, lib, dev, stream, timed, table)
    if world == 1 and want("lm_head"):
        _lm_head(L, lib, dev, s, timed, record, randn, nreps)
        _lm_head_other_hidden_sizes(L, lib, dev, s, timed, record, randn, nreps)
    if world > 1 and want("lm_head"):
        _lm_head_sharded(lib, dev, timed, record, randn, nreps, sharded, world, rank, table)
    return table


def _lm_head_sharded(lib, dev, timed, record, randn, nreps, sharded, world, rank, table):
    """Vocabulary-parallel LM head + greedy pick: every GPU reads its rows of the 151936 x 1024 fp16 table once; the
    packed keys are combined by an NCCL all-reduce (MAX) or by this library's own exchange kernel (peer stores)."""
    H, R = 1024, 4
    lo, hi = sharded.column_range(VOCAB, world, rank)
    shards = [randn(hi - lo, H, sigma=0.02) for _ in range(2)]
    hidden = randn(R, H)
    keys = torch.empty(R, dtype=torch.int64, device=dev)
    ids = torch.empty(R, dtype=torch.int32, device=dev)
    local_bytes = (hi - lo) * H * 2 + R * H * 2 + 4 * R
    shape = f"{R} x {H} by {VOCAB}/{world} x {H} f16"
    ms = timed([(lambda t=t: sharded.sharded_lm_head_argmax(hidden, t, lo, keys=keys, out=ids)) for t in shards], nreps(40))
    record("lm_head_argmax (vocab-parallel + all-reduce MAX of packed keys), eager launches", shape, local_bytes, ms, R,
           sharded_over=world)
    ex = sharded.PeerExchange(max_rows=R)
    try:
        ms = timed([(lambda t=t: sharded.sharded_lm_head_argmax_fused(hidden, t, lo, ex, keys=keys, out=ids)) for t in shards],
                   nreps(40))
        record("lm_head_argmax (vocab-parallel + keys exchange kernel, peer stores over NVLink), eager launches", shape,
               local_bytes, ms, R, sharded_over=world, note="two launches per GPU, no collective library call")
        if ex.timed_out():
            table.append({"op": "vocab-parallel lm_head, keys exchange", "error": "a bounded wait for a peer ran out"})
    except Exception as exc:
        table.append({"op": "vocab-parallel lm_head, keys exchange", "error": str(exc)[:200]})
    finally:
        ex.close()


def _lm_head(L, lib, dev, s, timed, record, randn, nreps):
    """Decode-size LM head fused with the greedy pick, Qwen3-0.6B's shape (151936 x 1024): bytes = the table read once
    (+ hidden rows and ids; + the logits when they are written).  Two tables alternate (622 MB > L2).  Beside it the
    two-step form it replaces, with a library GEMM standing in for the reference's cuBLAS call: matmul into a logits
    tensor, then this library's argmax over it."""
    F16, F32, FAST, DET = lib.F16, lib.F32, lib.FAST, lib.DETERMINISTIC
    H = 1024
    ws = torch.zeros(4096, dtype=torch.uint8, device=dev)
    for dtype, code, e in ((torch.float16, F16, 2), (torch.float32, F32, 4)):
        tables = [randn(VOCAB, H, sigma=0.02, dtype=dtype) for _ in range(2)]
        for R in ((1, 4, 8, 16, 64) if e == 2 else (1, 4)):
            hidden = randn(R, H, dtype=dtype)
            ids = torch.empty(R, dtype=torch.int32, device=dev)
            logits = torch.empty(R, VOCAB, dtype=dtype, device=dev)
            name = "f16" if e == 2 else "f32"
            for label, lp, mode in (("ids only", 0, FAST), ("ids + logits written", logits.data_ptr(), FAST),
                                    ("ids only, deterministic (k-ordered sums)", 0, DET)):
                if mode == DET and (R != 1 or e != 2):
                    continue
                if R > 4 and lp:
                    continue
                calls = [(lambda t=t: lib.check(L.b2_lm_head_argmax(hidden.data_ptr(), t.data_ptr(), R, H, VOCAB, code, mode, 0,
                                                                    lp, VOCAB, ids.data_ptr(), None, ws.data_ptr(), s)))
                         for t in tables]
                ms = timed(calls, nreps(20))
                record(f"lm_head_argmax ({label})", f"{R} x {H} by {VOCAB} x {H} {name}",
                       VOCAB * H * e + R * H * e + 4 * R + (R * VOCAB * e if lp else 0), ms, R)

            def two_step(t):
                torch.matmul(hidden, t.t(), out=logits)
                lib.check(L.b2_argmax_rows(logits.data_ptr(), R, VOCAB, VOCAB, code, ids.data_ptr(), ws.data_ptr(), s))
            ms = timed([(lambda t=t: two_step(t)) for t in tables], nreps(20))
            record("library GEMM into logits + argmax_rows (two launches, yardstick)", f"{R} x {H} by {VOCAB} x {H} {name}",
                   VOCAB * H * e + R * H * e + 4 * R + 2 * R * VOCAB * e, ms, R)
        del tables


def _decode_chain(L, lib, dev, stream, timed, table):
    """The launch-paced regime: the in-scope operators of ONE decoder layer of a decode step, back to back on one
    stream, Qwen3-0.6B shapes, fp16 -- residual add + norm, QK-norm + RoPE (one launch for the reference's four),
    residual add + norm, SwiGLU, residual add: five launches where the reference's layer makes eight
    (src/qwen3_layer_cuda.cu:285-292,319-325).  The projections and the attention between them are not on this path.
    Microseconds per chain, launched call by call or replayed from a CUDA graph, with and without programmatic
    dependent launch (b2_set_programmatic_launch)."""
    s = stream.cuda_stream
    half = torch.float16
    F16, FAST = lib.F16, lib.FAST
    for tokens in (1, 4, 64):
        z = lambda *shape: torch.zeros(*shape, device=dev, dtype=half)
        x, r, g, res, nrm, out = z(tokens, 1024), z(tokens, 1024), torch.ones(1024, device=dev, dtype=half), z(tokens, 1024), z(tokens, 1024), z(tokens, 1024)
        q, k, g128, qo, ko = z(tokens, 16, 128), z(tokens, 8, 128), torch.ones(128, device=dev, dtype=half), z(tokens, 16, 128), z(tokens, 8, 128)
        gate, up, act = z(tokens, 3072), z(tokens, 3072), z(tokens, 3072)
        pos = torch.zeros(tokens, dtype=torch.int32, device=dev)
        p = lambda t: t.data_ptr()

        def chain():
            lib.check(L.b2_add_rms_norm(p(x), p(r), p(g), p(res), p(nrm), tokens, 1024, 1e-6, F16, FAST, s))
            lib.check(L.b2_qk_norm_rope(p(q), p(k), p(g128), p(g128), p(pos), p(qo), p(ko), tokens, 16, 8, 128, 1e-6, 1e6, F16, None, s))
            lib.check(L.b2_add_rms_norm(p(res), p(nrm), p(g), p(x), p(r), tokens, 1024, 1e-6, F16, FAST, s))
            lib.check(L.b2_swiglu(p(gate), p(up), p(act), tokens * 3072, F16, FAST, s))
            lib.check(L.b2_add(p(x), p(r), p(out), tokens * 1024, F16, s))
        entry = {"op": "decode layer chain of the in-scope operators (5 launches)", "shape": f"{tokens} tokens, hidden 1024, 16+8 heads x 128, I=3072 f16"}
        for pdl in (0, 1):
            L.b2_set_programmatic_launch(pdl)
            try:
                tag = "_pdl" if pdl else ""
                entry["us_eager" + tag] = round(timed([chain], 200, warm=10) * 1e3, 2)
                K = 20
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(K):
                        chain()
                entry["us_graph_replay" + tag] = round(timed([graph.replay], 20) / K * 1e3, 2)
                del graph
            except Exception as exc:
                entry["error" + ("_pdl" if pdl else "")] = str(exc)[:160]
            finally:
                L.b2_set_programmatic_launch(0)
        table.append(entry)


def _lm_head_other_hidden_sizes(L, lib, dev, s, timed, record, randn, nreps):
    """The LM head at the other hidden sizes of the configurations (2048, 4096), fp16: one table each (622 MB / 1.24 GB > L2)."""
    ws = torch.zeros(4096, dtype=torch.uint8, device=dev)
    for H in (2048, 4096):
        table = randn(VOCAB, H, sigma=0.02)
        for R in (1, 4, 16, 64):
            hidden = randn(R, H)
            ids = torch.empty(R, dtype=torch.int32, device=dev)
            call = lambda: lib.check(L.b2_lm_head_argmax(hidden.data_ptr(), table.data_ptr(), R, H, VOCAB, lib.F16, lib.FAST, 0,
                                                         None, VOCAB, ids.data_ptr(), None, ws.data_ptr(), s))
            ms = timed([call], nreps(10))
            record("lm_head_argmax (ids only)", f"{R} x {H} by {VOCAB} x {H} f16", VOCAB * H * 2 + R * H * 2 + 4 * R, ms, R)
        del table


def _next_rows(L, lib, dev, s, timed, record, randn, want, nreps, sampler_rows=256, stream=None):
    """The callers either side of the path: sampling over the LM-head logits, paged-KV row writes, last-valid-row gather."""
    F16, F32 = lib.F16, lib.F32
    if want("sampler"):
        R = sampler_rows
        logits = [randn(R, VOCAB, sigma=4.0, dtype=torch.float32) for _ in range(2)]
        ids = torch.empty(R, dtype=torch.int32, device=dev)
        offs = torch.arange(R, dtype=torch.int64, device=dev)
        ws = torch.empty(L.b2_sampler_workspace_bytes(R, VOCAB), dtype=torch.uint8, device=dev)
        for label, temp, top_k, top_p in (("top_k=50 top_p=0.95 (sampled threshold, one pass)", 0.8, 50, 0.95),
                                          ("top_k=0 top_p=0.9 (top-p over the whole vocabulary, head sorted, tail summed)", 1.0, 0, 0.9)):
            calls = [(lambda x=x: lib.check(L.b2_sample_rows(x.data_ptr(), R, VOCAB, VOCAB, F32, temp, top_k, top_p, 7,
                                                             offs.data_ptr(), ids.data_ptr(), ws.data_ptr(), s))) for x in logits]
            ms = timed(calls, nreps(6), warm=2)
            record(f"sample_rows {label}", f"{R}x{VOCAB} f32", R * VOCAB * 4 + 12 * R, ms, R,
                   note="bytes = the logits read once; launches and the ordered fp32 sums set the time, not HBM")
        if stream is not None and R >= 2:
            # the same batch as two half-batches on two streams (each call has its own workspace): the kernels that
            # are one thread block per row and latency-bound (threshold search, head, finish) of one half run under
            # the passes over the logits of the other
            halves = ((0, R // 2), (R // 2, R))
            sides = [torch.cuda.Stream(device=dev) for _ in halves]
            wss = [torch.empty(L.b2_sampler_workspace_bytes(hi - lo, VOCAB), dtype=torch.uint8, device=dev) for lo, hi in halves]

            def split_call(x, temp, top_k, top_p):
                fork = torch.cuda.Event()
                fork.record(stream)
                for h, (lo, hi) in enumerate(halves):
                    sides[h].wait_event(fork)
                    lib.check(L.b2_sample_rows(x[lo:hi].data_ptr(), hi - lo, VOCAB, VOCAB, F32, temp, top_k, top_p, 7,
                                               offs[lo:hi].data_ptr(), ids[lo:hi].data_ptr(), wss[h].data_ptr(), sides[h].cuda_stream))
                    done = torch.cuda.Event()
                    done.record(sides[h])
                    stream.wait_event(done)
            for label, temp, top_k, top_p in (("top_k=50 top_p=0.95", 0.8, 50, 0.95), ("top_k=0 top_p=0.9", 1.0, 0, 0.9)):
                ms = timed([(lambda x=x: split_call(x, temp, top_k, top_p)) for x in logits], nreps(6), warm=2)
                record(f"sample_rows {label}, the batch as two half-batches on two streams", f"{R}x{VOCAB} f32", R * VOCAB * 4 + 12 * R,
                       ms, R, note="two calls, one workspace each; fork and join by events on the caller's stream")
            del wss
        del logits, ws
    if want("kvmove"):
        half = torch.float16
        layers, block_size, kv_heads, head_dim = 2, 16, 8, 128
        row_bytes = kv_heads * head_dim * 2
        T = 16384
        total_blocks = T // block_size + 8
        storage = torch.zeros(layers, total_blocks, 2, block_size, kv_heads, head_dim, device=dev, dtype=half)
        table = torch.randperm(total_blocks, device=dev)[: T // block_size].to(torch.int32)
        sets = [(randn(T, kv_heads, head_dim), randn(T, kv_heads, head_dim)) for _ in range(4)]
        calls = [(lambda b=b: lib.check(L.b2_paged_kv_prefill_copy(b[0].data_ptr(), b[1].data_ptr(), storage.data_ptr(),
                                                                   table.data_ptr(), T, table.numel(), 1, layers, total_blocks,
                                                                   block_size, kv_heads, head_dim, F16, None, s))) for b in sets]
        ms = timed(calls, nreps(40))
        record("paged_kv_prefill_copy", f"T={T}, {kv_heads} heads x {head_dim} f16", 4 * T * row_bytes + 4 * table.numel(), ms, T)
        B = 256
        tables = torch.randperm(total_blocks, device=dev)[:B * 4].reshape(B, 4).to(torch.int32).contiguous()
        pos = torch.randint(0, 4 * block_size, (B,), device=dev, dtype=torch.int32)
        k1, v1 = randn(B, kv_heads, head_dim), randn(B, kv_heads, head_dim)
        calls = [lambda: lib.check(L.b2_paged_kv_write_decode_batch(k1.data_ptr(), v1.data_ptr(), storage.data_ptr(),
                                                                    tables.data_ptr(), pos.data_ptr(), B, 4, 0, layers,
                                                                    total_blocks, block_size, kv_heads, head_dim, F16, None, s))]
        ms = timed(calls, nreps(100))
        record("paged_kv_write_decode_batch", f"B={B}, {kv_heads} heads x {head_dim} f16", 4 * B * row_bytes + 20 * B, ms, B,
               note="latency-bound: 2 MB moved")
        # the attention prologue in one launch: QK-norm + RoPE with K and V landing in the paged cache
        Tq = 16384
        q, kk, vv = randn(Tq, 16, head_dim), randn(Tq, kv_heads, head_dim), randn(Tq, kv_heads, head_dim)
        qo, ko = torch.empty_like(q), torch.empty_like(kk)
        g = (torch.rand(head_dim, device=dev) + 0.5).half()
        rpos = torch.randint(0, 512, (Tq,), device=dev, dtype=torch.int32)
        fused = [lambda: lib.check(L.b2_qk_norm_rope_paged(q.data_ptr(), kk.data_ptr(), vv.data_ptr(), g.data_ptr(), g.data_ptr(),
                                                           rpos.data_ptr(), qo.data_ptr(), storage.data_ptr(), table.data_ptr(),
                                                           None, Tq, 16, kv_heads, head_dim, 1e-6, 1e6, Tq, table.numel(), 1,
                                                           layers, total_blocks, block_size, F16, None, s))]
        ms = timed(fused, nreps(40))
        fused_bytes = 2 * Tq * 16 * head_dim * 2 + 4 * Tq * row_bytes + 8 * Tq      # q in/out, k in, v in, K and V rows out
        record("qk_norm_rope_paged (QK-norm + RoPE + K/V into the paged cache, one launch)", f"T={Tq}, 16+8 heads x {head_dim} f16",
               fused_bytes, ms, Tq)

        def separate():
            lib.check(L.b2_qk_norm_rope(q.data_ptr(), kk.data_ptr(), g.data_ptr(), g.data_ptr(), rpos.data_ptr(), qo.data_ptr(),
                                        ko.data_ptr(), Tq, 16, kv_heads, head_dim, 1e-6, 1e6, F16, None, s))
            lib.check(L.b2_paged_kv_prefill_copy(ko.data_ptr(), vv.data_ptr(), storage.data_ptr(), table.data_ptr(), Tq,
                                                 table.numel(), 1, layers, total_blocks, block_size, kv_heads, head_dim, F16, None, s))
        ms = timed([separate], nreps(40))
        record("qk_norm_rope + paged_kv_prefill_copy (two launches)", f"T={Tq}, 16+8 heads x {head_dim} f16",
               fused_bytes + 2 * Tq * row_bytes, ms, Tq, note="moves the keys twice more; bytes counted per launch sequence")
        del storage, sets, q, kk, vv, qo, ko
        Bp, S = 64, 16
        padded = [randn(Bp, S, VOCAB, dtype=torch.float32) for _ in range(2)]
        lengths = torch.randint(1, S + 1, (Bp,), device=dev, dtype=torch.int32)
        out = torch.empty(Bp, VOCAB, device=dev)
        calls = [(lambda x=x: lib.check(L.b2_select_last_valid_rows(x.data_ptr(), lengths.data_ptr(), out.data_ptr(), Bp, S, VOCAB,
                                                                    F32, None, s))) for x in padded]
        ms = timed(calls, nreps(40))
        record("select_last_valid_rows", f"[{Bp},{S},{VOCAB}] f32 -> [{Bp},{VOCAB}]", 2 * Bp * VOCAB * 4 + 4 * Bp, ms, Bp)


def _headline_shape_ops(L, lib, dev, s, timed, record, randn, nreps):
    F16, FAST, half = lib.F16, lib.FAST, torch.float16
    # ---- plain RMSNorm and add at the headline shape
    rows, hidden = 65536, 4096
    a, b_, o = randn(rows, hidden), randn(rows, hidden), torch.empty(rows, hidden, device=dev, dtype=half)
    g = (torch.rand(hidden, device=dev) + 0.5).half()
    ms = timed([lambda: lib.check(L.b2_rms_norm(a.data_ptr(), g.data_ptr(), o.data_ptr(), rows, hidden, 1e-6, F16, FAST, s))], nreps(20))
    record("rms_norm", f"{rows}x{hidden} f16", 2 * rows * hidden * 2 + 2 * hidden, ms, rows)
    ms = timed([lambda: lib.check(L.b2_add(a.data_ptr(), b_.data_ptr(), o.data_ptr(), rows * hidden, F16, s))], nreps(20))
    record("add", f"{rows}x{hidden} f16", 3 * rows * hidden * 2, ms, rows)
    ms = timed([lambda: lib.check(L.b2_swiglu(a.data_ptr(), b_.data_ptr(), o.data_ptr(), rows * hidden, F16, FAST, s))], nreps(20))
    record("swiglu", f"{rows}x{hidden} f16", 3 * rows * hidden * 2, ms, rows)
    # the deterministic (reference-order) form of the fused add + norm: one warp per row, fp64 index-order sum
    o2 = torch.empty_like(o)
    small = 4096
    ms = timed([lambda: lib.check(L.b2_add_rms_norm(a.data_ptr(), b_.data_ptr(), g.data_ptr(), o.data_ptr(), o2.data_ptr(), small,
                                                    hidden, 1e-6, F16, lib.DETERMINISTIC, s))], nreps(20))
    record("add_rms_norm, deterministic (fp64 sum in index order)", f"{small}x{hidden} f16", 4 * small * hidden * 2 + 2 * hidden, ms, small,
           note="133 MB working set: L2-assisted")
    del a, b_, o, o2



def _config3(L, lib, dev, s, timed, record, randn, sets_for, nreps):
    F16, FAST, half = lib.F16, lib.FAST, torch.float16
    # ---- configuration 3: packed-prefill QK-norm + RoPE, T = 16384, 16 + 8 heads of 128
    T, HQ, HK, D = 16384, 16, 8, 128
    # the seeded draw of the configuration (positions: 64 concatenated ramps; q, k ~N(0,1); gammas ~U(0.5,1.5));
    # the further buffer sets that rotate the working set past L2 are fresh normal draws of the same shapes
    from cuda_llm_b200 import workloads
    c3 = workloads.config3()
    pos = torch.from_numpy(c3["positions"]).to(dev)
    gq, gk = torch.from_numpy(c3["gamma_q"]).to(dev), torch.from_numpy(c3["gamma_k"]).to(dev)
    per_set = 2 * T * (HQ + HK) * D * 2
    n = sets_for(per_set)
    bufs = [(torch.from_numpy(c3["q"]).to(dev) if i == 0 else randn(T, HQ, D),
             torch.from_numpy(c3["k"]).to(dev) if i == 0 else randn(T, HK, D),
             torch.empty(T, HQ, D, device=dev, dtype=half), torch.empty(T, HK, D, device=dev, dtype=half)) for i in range(n)]
    calls = [(lambda b=b: lib.check(L.b2_qk_norm_rope(b[0].data_ptr(), b[1].data_ptr(), gq.data_ptr(), gk.data_ptr(),
                                                       pos.data_ptr(), b[2].data_ptr(), b[3].data_ptr(), T, HQ, HK, D,
                                                       1e-6, 1e6, F16, None, s))) for b in bufs]
    ms = timed(calls, nreps(40))
    record("qk_norm_rope (fused)", f"T={T} {HQ}+{HK} heads x {D} f16", per_set + 4 * T + 512, ms, T)

    def unfused(b):
        lib.check(L.b2_rms_norm(b[0].data_ptr(), gq.data_ptr(), b[2].data_ptr(), T * HQ, D, 1e-6, F16, FAST, s))
        lib.check(L.b2_rms_norm(b[1].data_ptr(), gk.data_ptr(), b[3].data_ptr(), T * HK, D, 1e-6, F16, FAST, s))
        lib.check(L.b2_rope(b[2].data_ptr(), pos.data_ptr(), b[2].data_ptr(), T, HQ, D, 1e6, F16, FAST, None, s))
        lib.check(L.b2_rope(b[3].data_ptr(), pos.data_ptr(), b[3].data_ptr(), T, HK, D, 1e6, F16, FAST, None, s))
    ms = timed([(lambda b=b: unfused(b)) for b in bufs], nreps(40))
    record("rms_norm x2 + rope x2 (reference-shaped)", f"T={T} {HQ}+{HK} heads x {D} f16", 2 * per_set + 8 * T + 1024, ms, T,
           note="four launches; bytes counted per launch sequence")
    del bufs, calls



def _config4(L, lib, dev, s, timed, record, randn, sharded, world, rank, want, nreps):
    F16, FAST, half = lib.F16, lib.FAST, torch.float16
    # ---- configuration 4: SwiGLU and embedding gather, T = 262144 tokens split over the ranks
    T4 = 262144
    lo, hi = sharded.row_range(T4, world, rank)
    t_local = hi - lo
    for inter in ((3072, 12288) if want("swiglu") else ()):
        gate, up = randn(t_local, inter, sigma=2.0), randn(t_local, inter, sigma=2.0)
        out = torch.empty_like(gate)
        ms = timed([lambda: lib.check(L.b2_swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), t_local * inter, F16, FAST, s))], nreps(10))
        record("swiglu", f"T={T4}/{world} x I={inter} f16", 3 * t_local * inter * 2, ms, t_local, sharded_over=world)
        del gate, up, out
    if not want("gather"):
        return
    table_w = randn(VOCAB, 4096, sigma=0.02)
    ids = torch.randint(0, VOCAB, (t_local,), device=dev, dtype=torch.int32)
    out = torch.empty(t_local, 4096, device=dev, dtype=half)
    ms = timed([lambda: lib.check(L.b2_embedding_gather(table_w.data_ptr(), ids.data_ptr(), out.data_ptr(), t_local, 4096,
                                                         VOCAB, F16, None, s))], 10)
    record("embedding_gather", f"T={T4}/{world} x 4096 f16, table {VOCAB}x4096", 2 * t_local * 4096 * 2 + 4 * t_local, ms,
           t_local, sharded_over=world)
    del table_w, ids, out



def _exchange_phases(lib, sharded, ex, logits, c_lo, ids_out, world, barrier, calls=24):
    """Medians, over `calls` separate launches that all ranks enter together, of the phases of b2_argmax_rows_sharded
    on this rank: launch to last local row done, waiting for the peers' keys, combining; and when each peer's first
    key was seen, relative to the start of the wait."""
    import ctypes as C
    import statistics
    dev = logits[0].device
    trace = torch.zeros(4 + world, dtype=torch.int64, device=dev)
    ex.desc.trace = trace.data_ptr()
    local, wait, combine, total, peers = [], [], [], [], [[] for _ in range(world)]
    try:
        for i in range(calls):
            barrier()
            sharded.sharded_argmax_fused(logits[i % len(logits)], c_lo, ex, out=ids_out)
            torch.cuda.synchronize()
            t = trace.tolist()
            local.append(t[1] - t[0]); wait.append(t[2] - t[1]); combine.append(t[3] - t[2]); total.append(t[3] - t[0])
            for g in range(world):
                peers[g].append(t[4 + g] - t[1])
    finally:
        ex.desc.trace = None
    med = lambda v: round(statistics.median(v) / 1e3, 2)
    return {"op": "fused exchange, phases of one b2_argmax_rows_sharded call on rank 0 (device timer, medians)",
            "calls": calls, "us_first_block_to_last_row_done": med(local), "us_waiting_for_peers": med(wait),
            "us_combine_and_finish": med(combine), "us_kernel_total": med(total),
            "us_peer_first_key_seen_after_wait_began": [med(p) for p in peers],
            "note": "ranks enter each call from a host barrier, so the wait includes the launch skew between processes"}


def sharded_summary(table, world):
    """The multi-GPU numbers of the table in one small block: microseconds per call (max over ranks)."""
    def us(fragment, shape_fragment=""):
        for e in table:
            if fragment in e.get("op", "") and shape_fragment in e.get("shape", "") and "us" in e:
                return e["us"]
        return None
    out = {"n_gpus": world, "swiglu_3072_us": us("swiglu", "I=3072"), "swiglu_12288_us": us("swiglu", "I=12288"),
           "gather_us": us("embedding_gather")}
    if world == 1:
        out.update({"argmax_us": us("argmax_rows"), "softmax_us": us("softmax_rows"),
                    "lm_head_4rows_us": us("lm_head_argmax (ids only)", "4 x 1024 by 151936 x 1024 f16")})
    else:
        out.update({"argmax_fused_us": us("argmax (vocab-sharded, exchange fused into the kernel), eager"),
                    "argmax_fused_bound_us": us("argmax (vocab-sharded, exchange fused into the kernel), eager launch through"),
                    "argmax_fused_graph_us": us("argmax (vocab-sharded, exchange fused into the kernel), CUDA-graph"),
                    "argmax_nccl_us": us("argmax (vocab-sharded + all-reduce MAX of packed keys), eager"),
                    "argmax_nccl_graph_us": us("argmax (vocab-sharded + all-reduce MAX of packed keys), CUDA-graph"),
                    "softmax_fused_us": us("softmax (vocab-sharded, exchange fused into the statistics kernel), eager"),
                    "softmax_fused_bound_us": us("softmax (vocab-sharded, exchange fused into the statistics kernel), eager launches through"),
                    "softmax_fused_graph_us": us("softmax (vocab-sharded, exchange fused into the statistics kernel), CUDA-graph"),
                    "softmax_nccl_us": us("softmax (vocab-sharded + all-reduce MAX, SUM), eager"),
                    "softmax_nccl_graph_us": us("softmax (vocab-sharded + all-reduce MAX, SUM), CUDA-graph"),
                    "lm_head_fused_us": us("lm_head_argmax (vocab-parallel + keys exchange"),
                    "lm_head_nccl_us": us("lm_head_argmax (vocab-parallel + all-reduce"),
                    "argmax_one_gpu_us": us("argmax_rows, whole vocabulary on one GPU"),
                    "softmax_one_gpu_us": us("softmax_rows, whole vocabulary on one GPU")})
    return out


def _config5(L, lib, dev, s, timed, record, randn, sets_for, sharded, world, rank, want, nreps, table, barrier=None):
    from cuda_llm_b200 import ops
    F16, F32, FAST = lib.F16, lib.F32, lib.FAST
    # ---- configuration 5: LM-head reductions over [256, V], V split over the ranks
    R = 256
    c_lo, c_hi = sharded.column_range(VOCAB, world, rank)
    width = c_hi - c_lo
    per_set = R * width * 4
    n = sets_for(per_set)
    logits = [randn(R, width, sigma=4.0, dtype=torch.float32) for _ in range(n)]
    outs = [torch.empty(R, width, device=dev) for _ in range(min(n, 4))]
    if world == 1:
        ids_out = torch.empty(R, dtype=torch.int32, device=dev)
        ws = ops.argmax_workspace(dev, R)
        calls = [(lambda x=x: lib.check(L.b2_argmax_rows(x.data_ptr(), R, width, width, F32, ids_out.data_ptr(), ws.data_ptr(), s)))
                 for x in logits]
        ms = timed(calls, nreps(40))
        record("argmax_rows", f"{R}x{VOCAB} f32", per_set + 4 * R, ms, R)
        sws = ops.softmax_workspace(dev, R)
        calls = [(lambda x=x, i=i: lib.check(L.b2_softmax_rows(x.data_ptr(), outs[i % len(outs)].data_ptr(), R, width, F32,
                                                                FAST, sws.data_ptr(), s))) for i, x in enumerate(logits)]
        ms = timed(calls, nreps(40))
        record("softmax_rows", f"{R}x{VOCAB} f32", 2 * per_set, ms, R)
        # the kernels of the vocabulary-sharded forms with a world of one GPU (the exchange is with itself): what their
        # local part costs beside the plain kernels above
        ex = sharded.PeerExchange(max_rows=R)
        try:
            stats1 = torch.empty(2, R, dtype=torch.float32, device=dev)
            ms = timed([(lambda x=x: sharded.sharded_argmax_fused(x, 0, ex, out=ids_out)) for x in logits], nreps(40))
            record("argmax (exchange fused into the kernel), world of one GPU", f"{R}x{VOCAB} f32", per_set + 4 * R, ms, R)
            ms = timed([(lambda x=x, i=i: sharded.sharded_softmax_fused(x, ex, out=outs[i % len(outs)], stats=stats1))
                        for i, x in enumerate(logits)], nreps(40))
            record("softmax (statistics kernel with the exchange, then apply), world of one GPU", f"{R}x{VOCAB} f32", 3 * per_set, ms, R,
                   note="two passes over the logits (the second from L2 where it fits): bytes counted as read twice, written once")
        finally:
            ex.close()
    else:
        # the yardstick of the sharded forms, in the same run: the whole vocabulary on one GPU (every rank alike, no exchange)
        full = [randn(R, VOCAB, sigma=4.0, dtype=torch.float32) for _ in range(4)]
        full_out = [torch.empty(R, VOCAB, device=dev) for _ in range(2)]
        ids_full = torch.empty(R, dtype=torch.int32, device=dev)
        ws_full, sws_full = ops.argmax_workspace(dev, R), ops.softmax_workspace(dev, R)
        ms = timed([(lambda x=x: lib.check(L.b2_argmax_rows(x.data_ptr(), R, VOCAB, VOCAB, F32, ids_full.data_ptr(),
                                                             ws_full.data_ptr(), s))) for x in full], nreps(40))
        record("argmax_rows, whole vocabulary on one GPU (yardstick of the sharded forms)", f"{R}x{VOCAB} f32", R * VOCAB * 4 + 4 * R, ms, R)
        ms = timed([(lambda x=x, i=i: lib.check(L.b2_softmax_rows(x.data_ptr(), full_out[i % 2].data_ptr(), R, VOCAB, F32, FAST,
                                                                   sws_full.data_ptr(), s))) for i, x in enumerate(full)], nreps(40))
        record("softmax_rows, whole vocabulary on one GPU (yardstick of the sharded forms)", f"{R}x{VOCAB} f32", 2 * R * VOCAB * 4, ms, R)
        del full, full_out
        # eager: every launch and the collective are issued from Python, which dominates at this size
        calls = [(lambda x=x: sharded.sharded_argmax(x, c_lo)) for x in logits]
        ms = timed(calls, nreps(40))
        record("argmax (vocab-sharded + all-reduce MAX of packed keys), eager launches", f"{R}x{VOCAB}/{world} f32",
               per_set + 4 * R, ms, R, sharded_over=world, note="exchange is 2 KB per rank; host launch overhead included")
        table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
        calls = [(lambda x=x, i=i: sharded.sharded_softmax(x, out=outs[i % len(outs)])) for i, x in enumerate(logits)]
        ms = timed(calls, nreps(40))
        record("softmax (vocab-sharded + all-reduce MAX, SUM), eager launches", f"{R}x{VOCAB}/{world} f32", 2 * per_set, ms, R,
               sharded_over=world)
        table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
        # the exchange fused into the reduction kernel: peer stores over NVLink, no collective call
        ex = sharded.PeerExchange(max_rows=R)
        try:
            ids_f = torch.empty(R, dtype=torch.int32, device=dev)
            stats_f = torch.empty(2, R, dtype=torch.float32, device=dev)
            calls = [(lambda x=x: sharded.sharded_argmax_fused(x, c_lo, ex, out=ids_f)) for x in logits]
            ms = timed(calls, nreps(40))
            record("argmax (vocab-sharded, exchange fused into the kernel), eager launch", f"{R}x{VOCAB}/{world} f32",
                   per_set + 4 * R, ms, R, sharded_over=world, note="one launch per GPU; keys cross NVLink as peer stores")
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            calls = [(lambda x=x, i=i: sharded.sharded_softmax_fused(x, ex, out=outs[i % len(outs)], stats=stats_f))
                     for i, x in enumerate(logits)]
            ms = timed(calls, nreps(40))
            record("softmax (vocab-sharded, exchange fused into the statistics kernel), eager launches",
                   f"{R}x{VOCAB}/{world} f32", 2 * per_set, ms, R, sharded_over=world)
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            # the same launches with the interpreter's per-call work (argument checks, pointer and stream look-ups) done once
            calls = [sharded.bind_argmax_fused(x, c_lo, ex, ids_f) for x in logits]
            ms = timed(calls, nreps(40))
            record("argmax (vocab-sharded, exchange fused into the kernel), eager launch through a bound call",
                   f"{R}x{VOCAB}/{world} f32", per_set + 4 * R, ms, R, sharded_over=world)
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            calls = [sharded.bind_softmax_fused(x, ex, outs[i % len(outs)], stats_f) for i, x in enumerate(logits)]
            ms = timed(calls, nreps(40))
            record("softmax (vocab-sharded, exchange fused into the statistics kernel), eager launches through a bound call",
                   f"{R}x{VOCAB}/{world} f32", 2 * per_set, ms, R, sharded_over=world)
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            # device-side time per call, free of the host's launch pacing: 16 calls over the rotating buffers recorded
            # into ONE graph and replayed
            stream = torch.cuda.current_stream()
            K = 16
            ga = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ga, stream=stream):
                for i in range(K):
                    sharded.sharded_argmax_fused(logits[i % n], c_lo, ex, out=ids_f)
            ms = timed([ga.replay], nreps(10)) / K
            record("argmax (vocab-sharded, exchange fused into the kernel), CUDA-graph replay", f"{R}x{VOCAB}/{world} f32",
                   per_set + 4 * R, ms, R, sharded_over=world, note=f"{K} calls per graph")
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            gs = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gs, stream=stream):
                for i in range(K):
                    sharded.sharded_softmax_fused(logits[i % n], ex, out=outs[i % len(outs)], stats=stats_f)
            ms = timed([gs.replay], nreps(10)) / K
            record("softmax (vocab-sharded, exchange fused into the statistics kernel), CUDA-graph replay",
                   f"{R}x{VOCAB}/{world} f32", 2 * per_set, ms, R, sharded_over=world, note=f"{K} calls per graph")
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            del ga, gs
            # where the time of one fused argmax call goes on this GPU: the kernel's own stamps of its nanosecond timer
            try:
                table.append(_exchange_phases(lib, sharded, ex, logits, c_lo, ids_f, world, barrier))
            except Exception as exc:
                table.append({"op": "fused exchange, phases of one call", "error": str(exc)[:200]})
            if ex.timed_out():
                table.append({"op": "vocab-sharded reductions, fused exchange", "error": "a bounded wait for a peer ran out"})
        except Exception as exc:
            table.append({"op": "vocab-sharded reductions, fused exchange", "error": str(exc)[:200]})
        finally:
            ex.close()
        # the same calls recorded once into CUDA graphs (kernels + NCCL all-reduces) and replayed
        try:
            stream = torch.cuda.current_stream()
            keys = [torch.empty(R, dtype=torch.int64, device=dev) for _ in logits]
            ids = [torch.empty(R, dtype=torch.int32, device=dev) for _ in logits]
            stats = [torch.empty(3, R, dtype=torch.float32, device=dev) for _ in logits]
            ops.argmax_workspace(dev, R)
            graphs_a, graphs_s = [], []
            for i, x in enumerate(logits):
                ga = torch.cuda.CUDAGraph()
                with torch.cuda.graph(ga, stream=stream):
                    sharded.sharded_argmax(x, c_lo, keys=keys[i], out=ids[i])
                graphs_a.append(ga)
                gs = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gs, stream=stream):
                    sharded.sharded_softmax(x, out=outs[i % len(outs)], stats=stats[i])
                graphs_s.append(gs)
            ms = timed([g.replay for g in graphs_a], nreps(40))
            record("argmax (vocab-sharded + all-reduce MAX of packed keys), CUDA-graph replay", f"{R}x{VOCAB}/{world} f32",
                   per_set + 4 * R, ms, R, sharded_over=world)
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
            ms = timed([g.replay for g in graphs_s], nreps(40))
            record("softmax (vocab-sharded + all-reduce MAX, SUM), CUDA-graph replay", f"{R}x{VOCAB}/{world} f32", 2 * per_set,
                   ms, R, sharded_over=world)
            table[-1]["rows_per_s"] = round(R / (ms * 1e-3), 1)
        except Exception as exc:   # graph capture of the collective is an optimisation, not a requirement
            table.append({"op": "vocab-sharded reductions, CUDA-graph replay", "error": str(exc)[:200]})


def main():
    """python opbench.py [--only GROUP] [--reps-scale X]: the single-GPU table, one line per entry."""
    import argparse
    from cuda_llm_b200 import build, lib
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--reps-scale", type=float, default=1.0)
    ap.add_argument("--sampler-rows", type=int, default=256, help="rows of the sampler entries (profiler captures use a few)")
    args = ap.parse_args()
    build.build()
    L = lib.load()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        rows = run(L, lib, dev, stream, 1, 0, torch.cuda.synchronize, lambda ms: ms, only=args.only,
                   reps_scale=args.reps_scale, sampler_rows=args.sampler_rows)
    for e in rows:
        print(json.dumps(e))


if __name__ == "__main__":
    main()
