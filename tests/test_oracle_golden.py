"""Pins the CPU oracle (oracle/oracle.c) before anything is compared against it:
the reference's own known-answer tests, its exported fixtures, and — where oracle/_ref
was built from the reference tree — bit equality with the reference's compiled ops_cpu."""
import math

import numpy as np
import pytest

from cuda_llm_b200 import workloads as wl
from util import f16_bits


# ---- closed-form answers of reference tests/test_ops_cpu.cpp:13-19 ------------------------

def _impls(port, ref):
    return [("port", port)] + ([("ref", ref)] if ref is not None else [])


def test_known_answers(port, ref):
    for name, o in _impls(port, ref):
        w = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
        e = o.embedding_lookup(w, [2, 0])
        assert e.shape == (2, 2) and e[0, 0] == 5 and (e[1] == [1, 2]).all(), name
        with pytest.raises(IndexError):
            o.embedding_lookup(w, [3])
        x = np.array([[2, 3]], np.float32)
        n = o.rms_norm(x, np.ones(2, np.float32), 0.0)
        assert abs(n[0, 0] - 2 / math.sqrt(6.5)) <= 1e-4, name
        r0 = o.rope(np.array([[[1, 2, 3, 4]]], np.float32), [0], 10000.0)
        assert np.abs(r0.ravel() - [1, 2, 3, 4]).max() <= 1e-4, name
        r1 = o.rope(np.array([[[1, 2, 3, 4]]], np.float32), [1], 10000.0).ravel()
        want = [math.cos(1) - 3 * math.sin(1), 2 * math.cos(.01) - 4 * math.sin(.01),
                math.sin(1) + 3 * math.cos(1), 2 * math.sin(.01) + 4 * math.cos(.01)]
        assert np.abs(r1 - want).max() <= 1e-4, name
        with pytest.raises(ValueError):
            o.rope(np.zeros((1, 1, 3), np.float32), [0], 10000.0)
        sm = o.softmax(np.array([[1000, 1001]], np.float32))
        assert abs(sm.sum() - 1) <= 1e-4 and np.isfinite(sm).all(), name
        assert o.swiglu(x, x)[0, 0] > 0, name
        assert o.add(x, x)[0, 0] == 4, name


# ---- fp16 codec edge cases of reference tests/test_tensor.cpp:11-18 -----------------------

def test_f16_decode_edges(port, ref):
    for bits, want in [(0x0001, 2.0 ** -24), (0x03ff, 2.0 ** -14 - 2.0 ** -24), (0x0400, 2.0 ** -14)]:
        assert port.decode_f16([bits])[0] == np.float32(want)
    neg0 = port.decode_f16([0x8000])[0]
    assert neg0 == 0 and np.signbit(neg0)
    assert np.isposinf(port.decode_f16([0x7c00])[0]) and np.isnan(port.decode_f16([0x7e00])[0])
    every = np.arange(65536, dtype=np.uint16)
    mine = port.decode_f16(every)
    numpy_view = every.view(np.float16).astype(np.float32)
    assert np.array_equal(mine.view(np.uint32)[~np.isnan(mine)], numpy_view.view(np.uint32)[~np.isnan(mine)])
    if ref is not None:
        theirs = np.array([ref.decode_f16(int(b)) for b in every[::7]], np.float32)
        ok = ~np.isnan(theirs)      # a scalar float return quiets signalling NaNs; payloads are not compared
        assert np.array_equal(np.isnan(theirs), np.isnan(mine[::7]))
        assert np.array_equal(theirs.view(np.uint32)[ok], mine[::7].view(np.uint32)[ok])


def test_f16_round_to_nearest_even_matches_numpy(port):
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(3),
        np.exp(rng.uniform(-30, 12, 200000)).astype(np.float32) * rng.choice([-1, 1], 200000).astype(np.float32),
        np.array([0, -0.0, 65504, 65519.99, 65520, 1e9, -1e9, np.inf, -np.inf, 2.0 ** -24, 2.0 ** -25,
                  1.5 * 2.0 ** -25, 2.0 ** -14, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11], np.float32)])
    assert np.array_equal(port.f32_to_f16_rn(x), x.astype(np.float16).view(np.uint16))


def test_reference_host_encoder_truncates(port, ref):
    # reference src/tensor.cpp:12 drops the low mantissa bits of normal numbers: fixtures must
    # never be quantised with it, or inputs differ from what the device would round.
    x = np.float32(1 + 3 * 2.0 ** -11)   # halfway plus: rounds up under nearest-even
    assert port.lib.orc_encode_f16_host(x) == 0x3c01 and port.f32_to_f16_rn([x])[0] == 0x3c02
    if ref is not None:
        assert ref.encode_f16(float(x)) == 0x3c01


# ---- the reference's exported layer-0 activations (HF Transformers fp32) --------------------
# tolerances of reference tests/test_qwen3_layer.cpp:24,27-28 and tests/test_qwen3_layer_cuda.cpp:92-95

def test_layer0_fixture_pairs(port, ref, golden):
    g = golden("layer0")
    eps, theta = float(g["rms_norm_eps"]), float(g["rope_theta"])
    pos = g["position_ids"].astype(np.int32)
    for name, o in _impls(port, ref):
        def close(got, want, tol, what):
            assert np.abs(got - want).max() <= tol, f"{name} {what}: {np.abs(got - want).max()}"
        close(o.rms_norm(g["hidden_states"], g["input_layernorm_weight"], eps), g["input_norm"], 1e-4, "input_norm")
        qn = o.rms_norm(g["q_linear"].reshape(-1, 128), g["q_norm_weight"], eps).reshape(4, 16, 128)
        kn = o.rms_norm(g["k_linear"].reshape(-1, 128), g["k_norm_weight"], eps).reshape(4, 8, 128)
        close(qn, g["q_norm_output"], 1e-4, "q_norm_output")
        close(kn, g["k_norm_output"], 5e-4, "k_norm_output")
        close(o.rope(g["q_norm_output"], pos, theta), g["q_rope"], 1e-4, "q_rope")
        close(o.rope(g["k_norm_output"], pos, theta), g["k_rope"], 5e-4, "k_rope")
        res, nrm = o.add_rms_norm(g["hidden_states"], g["o_proj_output"], g["post_attention_layernorm_weight"], eps)
        close(res, g["attention_residual"], 1e-4, "attention_residual")
        close(nrm, g["post_attention_norm"], 1e-4, "post_attention_norm")
        close(o.swiglu(g["gate_proj_output"], g["up_proj_output"]), g["swiglu_output"], 1e-4, "swiglu_output")
        close(o.add(g["attention_residual"], g["down_proj_output"]), g["layer_output"], 1e-4, "layer_output")


# ---- argmax: reference tests/test_argmax_cuda.cpp:42-52 and the recorded greedy ids ---------

def test_argmax_known_cases(port):
    am = lambda a: int(port.argmax_rows(np.asarray(a, np.float32))[-1])
    assert am([[-1, 2, 3, 4, 5], [1, 9, 2, 8, 3]]) == 1
    assert am([[4, 7, 7, 1, 7, 2]]) == 1                      # tie -> lowest index
    assert am([[-1, -2, -3, -4]]) == 0
    two = np.full((2, wl.VOCAB), -10, np.float32)
    two[0, 11] = 100
    two[1, 12345] = 101
    assert am(two) == 12345
    tie = np.full((1, wl.VOCAB), -10, np.float16)
    tie[0, 11], tie[0, 12345], tie[0, wl.VOCAB - 1] = 100, 101, 101
    assert int(port.argmax_rows(f16_bits(tie))[0]) == 12345   # f16 tie at 12345 vs 151935
    assert am([[np.nan, -np.inf, -3.4028235e38]]) == 0          # nothing can win -> 0
    assert am([[-np.inf, -3.4028235e38, -np.inf]]) == 0          # -FLT_MAX is the fold's start value: it never wins
    assert am([[-np.inf, -3.4028235e38, -3.4028233e38]]) == 2    # the next float above it does
    assert am([[np.nan, 1, np.nan, 1]]) == 1


def test_argmax_recorded_greedy_ids(port, golden):
    g = golden("logits_last_rows")
    for case, want in (("case_seq4", 1095), ("case_seq8", 13724)):
        row = g[case + "_last_row"]
        assert int(g[case + "_greedy_id"][0]) == want
        assert int(port.argmax_rows(row[None])[0]) == want
        work = row.copy()
        for k in range(5):                                    # top-5 by repeated argmax
            i = int(port.argmax_rows(work[None])[0])
            assert i == int(g[case + "_top5_ids"][k])
            assert abs(work[i] - g[case + "_top5_logits"][k]) <= 1e-6 * abs(work[i])
            work[i] = -np.inf


def test_argmax_key_packing(port):
    rng = np.random.default_rng(11)
    vals = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 5,
                           np.array([0.0, -0.0, 1e-45, -1e-45, 3e38, -3e38, np.inf], np.float32)])
    idx = rng.integers(0, 2 ** 31 - 1, vals.size)   # ids are int32
    keys = [port.argmax_key(float(v), int(i)) for v, i in zip(vals, idx)]
    for a in range(0, vals.size, 37):
        for b in range(1, vals.size, 41):
            if vals[a] != vals[b]:
                assert (keys[a] > keys[b]) == (vals[a] > vals[b])
            elif idx[a] != idx[b]:
                assert (keys[a] > keys[b]) == (idx[a] < idx[b])
    assert all(port.argmax_key_index(k) == i for k, i in zip(keys, idx))
    for bad in (np.nan, -np.inf, -3.4028235e38):
        assert port.argmax_key(bad, 5) == -(1 << 63) and port.argmax_key_index(-(1 << 63)) == 0


# ---- the restatement equals the reference's compiled code, bit for bit ----------------------

def test_port_equals_reference_bitwise(port, ref, golden):
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(2024)
    bits = lambda a: np.ascontiguousarray(a).view(np.uint32)
    x, y = wl.normal(rng, (37, 300)), wl.normal(rng, (37, 300))
    w = wl.gamma(rng, 300)
    assert np.array_equal(bits(port.rms_norm(x, w, 1e-6)), bits(ref.rms_norm(x, w, 1e-6)))
    assert np.array_equal(bits(port.add(x, y)), bits(ref.add(x, y)))
    for a, b in zip(port.add_rms_norm(x, y, w, 1e-6), ref.add_rms_norm(x, y, w, 1e-6)):
        assert np.array_equal(bits(a), bits(b))
    g = wl.normal(rng, (37, 300), 4.0)
    assert np.array_equal(bits(port.swiglu(g, y)), bits(ref.swiglu(g, y)))
    q = wl.normal(rng, (50, 3, 64))
    pos = rng.integers(0, 40000, 50).astype(np.int32)
    for theta in (1e4, 1e6):
        assert np.array_equal(bits(port.rope(q, pos, theta)), bits(ref.rope(q, pos, theta)))
    lg = wl.normal(rng, (5, 3001), 4.0)
    assert np.array_equal(bits(port.softmax(lg)), bits(ref.softmax(lg)))
    ids = rng.integers(0, 37, 20)
    assert np.array_equal(bits(port.embedding_lookup(x, ids)), bits(ref.embedding_lookup(x, ids)))


def test_port_reproduces_committed_reference_outputs(port, golden):
    """c1_reference.npz / small_reference.npz were produced by the reference's compiled CPU
    operators (tests/golden/make_golden.py); the restatement must give the same bits."""
    c = wl.config1()
    g = golden("c1_reference")
    same = lambda a, b: np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))
    res, nrm = port.add_rms_norm(c["x"], c["res"], c["gamma"], wl.EPS)
    assert same(res, g["residual"]) and same(nrm, g["normalized"])
    qn = port.rms_norm(c["q"].reshape(-1, 128), c["gamma_q"], wl.EPS).reshape(c["q"].shape)
    kn = port.rms_norm(c["k"].reshape(-1, 128), c["gamma_k"], wl.EPS).reshape(c["k"].shape)
    assert same(qn, g["q_norm"]) and same(kn, g["k_norm"])
    assert same(port.rope(qn, c["positions"], wl.THETA), g["q_rope"])
    assert same(port.rope(kn, c["positions"], wl.THETA), g["k_rope"])
    assert same(port.swiglu(c["gate"], c["up"]), g["swiglu"])
    assert np.array_equal(c["ids"], g["ids"]) and same(port.embedding_lookup(c["table"], c["ids"]), g["gather"])
    s = golden("small_reference")
    c5 = wl.config5(rows=4, vocab=8192, seed=5002)
    assert same(port.softmax(c5["logits"]), s["c5_softmax"])
    c2 = wl.config2(64, 1024)
    f = {k: port.decode_f16(f16_bits(v)).reshape(v.shape) for k, v in c2.items()}
    res, nrm = port.add_rms_norm(f["x"], f["res"], f["gamma"], wl.EPS)
    assert same(res, s["c2_residual"]) and same(nrm, s["c2_normalized"])


# ---- linear / lm_head (reference src/ops_cpu.cpp:9,17) ---------------------------------------

def test_linear_known_answer_and_reference_bits(port, ref, golden):
    """reference tests/test_ops_cpu.cpp:14,19: [2,3] x [[1,2],[3,4],[5,6]]^T = [8,18,28], lm_head == linear;
    then bit equality with the reference's compiled lm_head and with its committed outputs."""
    x = np.array([[2, 3]], np.float32)
    w = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    assert port.linear(x, w).tolist() == [[8.0, 18.0, 28.0]]
    bits = lambda a: np.ascontiguousarray(a).view(np.uint32)
    lm = wl.lm_head_case(rows=4, hidden=1024, vocab=640, seed=6002, dtype=np.float16)
    got = port.linear(port.decode_f16(f16_bits(lm["hidden"])).reshape(4, 1024),
                      port.decode_f16(f16_bits(lm["table"])).reshape(640, 1024))
    assert np.array_equal(bits(got), bits(golden("small_reference")["lm_head_logits"]))
    if ref is None:
        return
    assert ref.lm_head(x, w).tolist() == [[8.0, 18.0, 28.0]]
    rng = np.random.default_rng(77)
    h, t = wl.normal(rng, (3, 333)), wl.normal(rng, (211, 333), 0.02)
    assert np.array_equal(bits(port.linear(h, t)), bits(ref.lm_head(h, t)))


# ---- the device-order restatement (deterministic mode's target) ------------------------------

def test_device_order_restatement_is_consistent(port):
    rng = np.random.default_rng(5)
    x, y, w = wl.normal(rng, (9, 1024)), wl.normal(rng, (9, 1024)), wl.gamma(rng, 1024)
    # fp32: differs from the CPU operator only through the fp64 sum -> a few fp32 ulps
    assert np.abs(port.dev_rms_norm(x, w, 1e-6) - port.rms_norm(x, w, 1e-6)).max() <= 1e-5
    res, nrm = port.dev_add_rms_norm(x, y, w, 1e-6)
    assert np.array_equal(res, x + y)
    assert np.array_equal(nrm, port.dev_rms_norm(res, w, 1e-6))          # fp32: nothing is rounded away
    # fp16: the residual is rounded, the sum is not; the norm re-reads the rounded residual
    x16, y16, w16 = (a.astype(np.float16) for a in (x, y, w))
    res16, nrm16 = port.dev_add_rms_norm(f16_bits(x16), f16_bits(y16), f16_bits(w16), 1e-6)
    exact = x16.astype(np.float32) + y16.astype(np.float32)
    assert np.array_equal(res16, f16_bits(exact.astype(np.float16)))
    ss = (exact.astype(np.float64) ** 2).sum(axis=1, keepdims=True)
    inv = (1.0 / np.sqrt(ss / 1024 + np.float64(np.float32(1e-6)))).astype(np.float32)
    want = ((res16.view(np.float16).astype(np.float32) * inv) * w16.astype(np.float32)).astype(np.float16)
    assert np.array_equal(nrm16, f16_bits(want))
    assert np.array_equal(port.dev_add(f16_bits(x16), f16_bits(y16)), f16_bits(exact.astype(np.float16)))


# ---- the sampler restatement against the reference's own sampler test (tests/test_sampling_cuda.cpp:18-56)

def test_sampler_restatement_on_the_reference_test_cases(port):
    f = np.float32
    two = np.array([2, 9, 1, 7, 3, 5], f)
    assert port.sample_row(two, 1.0, 1, 1.0, 0, 0)[0] == 1                          # top_k = 1 is greedy
    assert port.sample_row(two, 1.0, 3, 1.0, 42, 7)[0] == port.sample_row(two, 1.0, 3, 1.0, 42, 7)[0]
    small = np.array([10, 9, 0, -1, -2, -3], f)
    assert {port.sample_row(small, 1.0, 2, 1.0, 1, i)[0] for i in range(20)} <= {0, 1}      # top-k boundary
    assert {port.sample_row(small, 1.0, 3, 0.5, 2, i)[0] for i in range(20)} <= {0, 1}      # top-k with top-p
    crossing = np.array([np.log(f(0.505)), np.log(f(0.495)), -20, -20, -20, -20], f)
    assert {port.sample_row(crossing, 1.0, 0, 0.51, 77, o)[0] for o in range(64)} == {0, 1}   # the crossing token is kept
    ties = np.array([0, 0, 0, -10, -10, -10], f)
    assert {port.sample_row(ties, 1.0, 0, 0.30, 88, o)[0] for o in range(64)} == {0}          # equal maxima: lowest id
    # frequencies follow the retained, renormalised distribution
    rng = np.random.default_rng(3)
    row = (rng.standard_normal(500) * 2).astype(f)
    top = np.argsort(-row, kind="stable")[:10]
    draws = np.array([port.sample_row(row, 1.0, 10, 1.0, 5, o)[0] for o in range(3000)])
    assert set(np.unique(draws)) <= set(top.tolist())
    p = np.exp(row[top].astype(np.float64) - row[top[0]])
    p /= p.sum()
    assert np.abs(np.array([(draws == t).mean() for t in top]) - p).max() < 4 * np.sqrt(0.25 / 3000)


def test_kv_move_restatements_against_plain_indexing(port):
    """orc_paged_kv_write / orc_select_last_valid (the reference kernels' index arithmetic) against numpy indexing
    of the pool layout [layers, total_blocks, 2, block_size, kv_heads, head_dim]."""
    rng = np.random.default_rng(8)
    layers, total_blocks, block_size, kv_heads, head_dim = 2, 12, 4, 2, 8
    storage = rng.standard_normal((layers, total_blocks, 2, block_size, kv_heads, head_dim)).astype(np.float16)
    key = rng.standard_normal((3, kv_heads, head_dim)).astype(np.float16)
    value = rng.standard_normal((3, kv_heads, head_dim)).astype(np.float16)
    tables = np.array([[0, 1, 2], [5, 4, 3], [9, 8, 7]], np.int32)
    positions = np.array([0, 5, 11], np.int32)
    got = storage.copy()
    port.paged_kv_write(0, key, value, got, tables, positions, 1, total_blocks, block_size)
    want = storage.copy()
    for b in range(3):
        blk, slot = tables[b, positions[b] // block_size], positions[b] % block_size
        want[1, blk, 0, slot], want[1, blk, 1, slot] = key[b], value[b]
    assert np.array_equal(got, want)
    got = storage.copy()
    port.paged_kv_write(1, key, value, got, tables[1], np.zeros(1, np.int32), 0, total_blocks, block_size)
    want = storage.copy()
    for t in range(3):
        want[0, tables[1, t // block_size], 0, t % block_size] = key[t]
        want[0, tables[1, t // block_size], 1, t % block_size] = value[t]
    assert np.array_equal(got, want)
    padded = rng.standard_normal((3, 5, 7)).astype(np.float32)
    assert np.array_equal(port.select_last_valid(padded, [5, 1, 3]), padded[[0, 1, 2], [4, 0, 2]])
