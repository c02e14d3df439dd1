"""GPU parity of the decode-size LM head fused with the greedy pick (b2_lm_head_argmax), through the C ABI.

Oracle: the reference's CPU `lm_head` (= `linear`, src/ops_cpu.cpp:9,17) restated in oracle.c and pinned
bit for bit to the reference's compiled code, followed by the reference's arg-max rule
(src/ops_cuda.cu:562-563).  fp16 inputs are widened exactly and the oracle's fp32 logit is rounded to
fp16 (nearest even) where the stored logit is compared, as the reference's fp16 kernel stores it
(src/ops_cuda.cu:101-111).

Rules: deterministic mode - stored logits and indices bit-exact.  Fast mode - fp32 logits within
1e-5 * max(|ref|, sum_k |x_k w_k|) (the scale of the accumulation, where a bound relative to a
cancelled result means nothing), fp16 logits within one fp16 ulp plus that bound; the index is exactly
the reference rule applied to the stored logits, and equals the oracle's wherever the oracle's winner
leads by more than the bound.
"""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, workloads as wl
from util import f16_bits, ulp16

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()
RTOL = 1e-5


def _oracle(port, hidden, table):
    """fp32 logits of the CPU operator, their accumulation scale, and the stored form per dtype."""
    h32 = hidden.astype(np.float32) if hidden.dtype == np.float32 else port.decode_f16(f16_bits(hidden)).reshape(hidden.shape)
    t32 = table.astype(np.float32) if table.dtype == np.float32 else port.decode_f16(f16_bits(table)).reshape(table.shape)
    logits = port.linear(h32, t32)
    scale = np.abs(h32).astype(np.float64) @ np.abs(t32).astype(np.float64).T
    return logits, scale


def _stored(logits32, dtype):
    return logits32 if dtype == np.float32 else logits32.astype(np.float16)


def _argmax(port, stored):
    return port.argmax_rows(stored if stored.dtype == np.float32 else f16_bits(stored))


def _run(hidden, table, mode, with_logits=True):
    h, t = dev(hidden), dev(table)
    out = torch.empty(hidden.shape[0], table.shape[0], dtype=h.dtype, device=DEV) if with_logits else None
    ids = ops.lm_head_argmax(h, t, logits_out=out, mode=mode)
    return host(ids), (host(out) if with_logits else None)


SHAPES = [(1, 1024, 640), (2, 1024, 641), (3, 1024, 5003), (4, 1024, 2049), (5, 1024, 700), (7, 1024, 333),
          (1, 2048, 515), (2, 2048, 1030), (3, 2048, 77), (1, 4096, 300), (2, 4096, 129),
          (2, 384, 1000), (1, 8, 5), (4, 100, 257), (1, 8192, 40), (4, 4096, 300), (2, 8192, 40), (3, 3072, 200),
          (1, 1536, 100), (6, 1024, 500), (4, 2048, 9)]


@pytest.mark.parametrize("rows,hidden,vocab", SHAPES)
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_deterministic_mode_is_bit_exact(b2, port, rows, hidden, vocab, dtype):
    c = wl.lm_head_case(rows, hidden, vocab, seed=6100 + rows + hidden + vocab, dtype=dtype)
    want32, _ = _oracle(port, c["hidden"], c["table"])
    want = _stored(want32, dtype)
    ids, logits = _run(c["hidden"], c["table"], "deterministic")
    bits = lambda a: a.view(np.uint32 if a.dtype == np.float32 else np.uint16)
    assert np.array_equal(bits(logits), bits(want))
    assert np.array_equal(ids, _argmax(port, want))


@pytest.mark.parametrize("rows,hidden,vocab", SHAPES)
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_fast_mode_within_tolerance(b2, port, rows, hidden, vocab, dtype):
    c = wl.lm_head_case(rows, hidden, vocab, seed=6200 + rows + hidden + vocab, dtype=dtype)
    want32, scale = _oracle(port, c["hidden"], c["table"])
    ids, logits = _run(c["hidden"], c["table"], "fast")
    bound = RTOL * np.maximum(np.abs(want32.astype(np.float64)), scale)
    if dtype == np.float16:
        bound = bound + ulp16(want32)
    err = np.abs(logits.astype(np.float64) - want32.astype(np.float64))
    assert (err <= bound).all(), f"worst error / bound = {(err / bound).max():.3f}"
    assert np.array_equal(ids, _argmax(port, logits))            # the reference's rule on the stored logits
    ids_only, _ = _run(c["hidden"], c["table"], "fast", with_logits=False)
    assert np.array_equal(ids_only, ids)
    # where the oracle's winner leads every other stored logit by more than the bound, the index is the oracle's
    want = _stored(want32, dtype).astype(np.float64)
    want_ids = _argmax(port, _stored(want32, dtype))
    for r in range(rows):
        others = np.delete(want[r], want_ids[r])
        margin = want[r, want_ids[r]] - (others.max() if others.size else -np.inf)
        if margin > 4 * bound[r].max():
            assert ids[r] == want_ids[r]


def _planted(rows, hidden, vocab, dtype, seed):
    """Every row's own winner planted at a seeded index: that table row is 0.02 x the hidden row,
    so its logit is ~0.02 * hidden (about 20 at 1024) against N(0, 0.02^2 * hidden) elsewhere."""
    c = wl.lm_head_case(rows, hidden, vocab, seed=seed, dtype=dtype)
    rng = np.random.default_rng(seed + 1)
    planted = rng.choice(vocab, rows, replace=False).astype(np.int32)
    for r in range(rows):
        c["table"][planted[r]] = (c["hidden"][r].astype(np.float32) * np.float32(0.02)).astype(dtype)
    return c, planted


@pytest.mark.parametrize("rows,dtype", [(1, np.float16), (4, np.float16), (1, np.float32), (3, np.float32)])
@pytest.mark.parametrize("mode", ["fast", "deterministic"])
def test_full_vocabulary_planted_winners(b2, port, rows, dtype, mode):
    """Qwen3-0.6B's LM head at full size: 151936 x 1024."""
    c, planted = _planted(rows, 1024, wl.VOCAB, dtype, seed=6300 + rows)
    for with_logits in (False, True):
        ids, logits = _run(c["hidden"], c["table"], mode, with_logits)
        assert np.array_equal(ids, planted)
        assert np.array_equal(ids, _run(c["hidden"], c["table"], mode, with_logits)[0])   # scratch left clean
    if mode == "deterministic" and rows == 1:
        want32, _ = _oracle(port, c["hidden"], c["table"])
        want = _stored(want32, dtype)
        assert np.array_equal(logits.view(np.uint8), want.view(np.uint8))


def test_ties_nans_and_rows_without_a_winner(b2, port):
    f = np.float32
    lowest = np.finfo(f).min                             # -FLT_MAX: "nothing seen", never wins
    hidden = np.zeros((4, 1024), f)
    hidden[0, 0] = 1.0                                   # logits = table[:, 0]
    hidden[1, 1] = 1.0                                   # logits = table[:, 1]: all equal -> index 0
    hidden[2, 2] = np.inf                                # inf * 0 = NaN wherever table[:, 2] == 0
    hidden[3, 3] = 1.0                                   # logits = table[:, 3] = -FLT_MAX everywhere -> no winner -> 0
    table = np.zeros((3000, 1024), f)
    table[:, 0] = -5.0
    table[[17, 900, 2999], 0] = 7.0                      # three-way tie: lowest index wins
    table[:, 1] = 2.5
    table[1234, 2] = 1.0                                 # the only non-NaN logit of row 2 (+inf)
    table[:, 3] = lowest
    for mode in ("fast", "deterministic"):
        ids, logits = _run(hidden, table, mode)
        assert ids.tolist() == [17, 0, 1234, 0], mode
        assert np.isnan(logits[2, 0]) and logits[2, 1234] == np.inf and (logits[3] == lowest).all()
        assert np.array_equal(ids, _argmax(port, logits))
    table[:, 3] = -65504.0                               # fp16's lowest finite value: an ordinary logit there
    for mode in ("fast", "deterministic"):
        ids, logits = _run(hidden.astype(np.float16), table.astype(np.float16), mode)
        assert ids.tolist() == [17, 0, 1234, 0], mode


def test_fp16_ties_appear_only_after_rounding(b2, port):
    """Two logits that differ in fp32 but round to the same fp16 value: the reference picks from the
    stored fp16 logits, so the lower index wins."""
    hidden = np.zeros((1, 1024), np.float16)
    hidden[0, :2] = [1.0, 2.0 ** -12]
    table = np.zeros((100, 1024), np.float16)
    table[:, 0] = 1.0
    table[60, 0], table[60, 1] = 3.0, 1.0                # 3 + 2^-12 -> 3.0 in fp16
    table[20, 0] = 3.0                                   # exactly 3.0
    for mode in ("fast", "deterministic"):
        ids, logits = _run(hidden, table, mode)
        assert ids.tolist() == [20], mode
        assert logits[0, 60] == logits[0, 20] == np.float16(3.0)


def test_unaligned_pointers_take_the_element_wise_path(b2, port):
    c = wl.lm_head_case(2, 1024, 300, seed=6400, dtype=np.float16)
    big = torch.empty(300 * 1024 + 1, dtype=torch.float16, device=DEV)
    table = big[1:].view(300, 1024)
    table.copy_(dev(c["table"]))
    assert table.data_ptr() % 16 != 0 and table.is_contiguous()
    want32, _ = _oracle(port, c["hidden"], c["table"])
    for mode in ("fast", "deterministic"):
        out = torch.empty(2, 300, dtype=torch.float16, device=DEV)
        ids = ops.lm_head_argmax(dev(c["hidden"]), table, logits_out=out, mode=mode)
        assert np.array_equal(f16_bits(host(out)), f16_bits(want32.astype(np.float16)))
        assert np.array_equal(host(ids), _argmax(port, want32.astype(np.float16)))


def test_vocabulary_sharded_keys(b2, port):
    """The table split by rows over 4 "GPUs": keys with the shard's index base, one signed MAX, decode."""
    c, planted = _planted(4, 1024, 4000, np.float16, seed=6500)
    h = dev(c["hidden"])
    keys = []
    for g in range(4):
        lo, hi = wl.shard_range(4000, 4, g)
        k = torch.empty(4, dtype=torch.int64, device=DEV)
        ops.lm_head_argmax(h, dev(c["table"][lo:hi]), want_ids=False, keys_out=k, index_base=lo)
        keys.append(k)
    best = torch.stack(keys).max(dim=0).values
    ids = torch.empty(4, dtype=torch.int32, device=DEV)
    from cuda_llm_b200 import lib
    lib.check(b2.b2_argmax_decode_keys(best.data_ptr(), 4, ids.data_ptr(), torch.cuda.current_stream().cuda_stream))
    assert np.array_equal(host(ids), planted)
    assert np.array_equal(host(ids), host(ops.lm_head_argmax(h, dev(c["table"]))))


def test_shares_the_argmax_scratch_with_argmax_rows(b2, port):
    c = wl.lm_head_case(3, 1024, 2000, seed=6600, dtype=np.float32)
    h, t = dev(c["hidden"]), dev(c["table"])
    out = torch.empty(3, 2000, device=DEV)
    for _ in range(3):
        ids = ops.lm_head_argmax(h, t, logits_out=out)
        assert np.array_equal(host(ops.argmax_rows(out)), host(ids))


def test_argument_rules(b2):
    h = torch.zeros(2, 1024, device=DEV)
    t = torch.zeros(10, 1024, device=DEV)
    with pytest.raises(ValueError):
        ops.lm_head_argmax(h.cpu(), t)                                       # not CUDA
    with pytest.raises(ValueError):
        ops.lm_head_argmax(h, t.half())                                      # dtypes differ
    with pytest.raises(ValueError):
        ops.lm_head_argmax(h, t[:, :512].contiguous())                       # hidden_size mismatch
    with pytest.raises(ValueError):
        ops.lm_head_argmax(h[0], t)                                          # rank
    with pytest.raises(ValueError):
        ops.lm_head_argmax(h, t, logits_out=torch.zeros(2, 9, device=DEV))   # output shape
    with pytest.raises(ValueError):
        ops.lm_head_argmax(h, t, want_ids=False)                             # no output at all
    with pytest.raises(ValueError):
        ops.lm_head_argmax(torch.zeros(1, 9000, device=DEV), torch.zeros(3, 9000, device=DEV))   # hidden_size > 8192
    # no rows: nothing to do, nothing dereferenced (empty batches reach the C ABI as they are)
    from cuda_llm_b200 import lib
    ids = torch.full((1,), 7, dtype=torch.int32, device=DEV)
    assert b2.b2_lm_head_argmax(None, None, 0, 1024, 10, lib.F32, lib.FAST, 0, None, 10, ids.data_ptr(), None, None,
                                torch.cuda.current_stream().cuda_stream) == 0
    assert int(ids[0]) == 7
    assert b2.b2_lm_head_argmax(h.data_ptr(), t.data_ptr(), 2, 1024, 10, lib.F32, 5, 0, None, 10, ids.data_ptr(), None, None,
                                torch.cuda.current_stream().cuda_stream) == -1      # unknown mode



# ---- more rows than the matrix-vector kernels take: the tensor-core kernel (fp16, fast mode) ----------------------

MMA_SHAPES = [(5, 1024, 700), (8, 1024, 128), (16, 1024, 129), (17, 1024, 1000), (32, 1024, 4097), (33, 2048, 300),
              (64, 1024, 2500), (65, 1024, 513), (100, 1024, 260), (8, 64, 1000), (12, 192, 555), (64, 4096, 384),
              (16, 1024, 19000)]


@pytest.mark.parametrize("rows,hidden,vocab", MMA_SHAPES)
def test_many_rows_tensor_core_kernel_within_tolerance(b2, port, rows, hidden, vocab):
    """Same rules as the fast mode above; 65 and 100 rows take two passes over the table."""
    c = wl.lm_head_case(rows, hidden, vocab, seed=6700 + rows + hidden + vocab, dtype=np.float16)
    want32, scale = _oracle(port, c["hidden"], c["table"])
    ids, logits = _run(c["hidden"], c["table"], "fast")
    bound = RTOL * np.maximum(np.abs(want32.astype(np.float64)), scale) + ulp16(want32)
    err = np.abs(logits.astype(np.float64) - want32.astype(np.float64))
    assert (err <= bound).all(), f"worst error / bound = {(err / bound).max():.3f}"
    assert np.array_equal(ids, _argmax(port, logits))            # the reference's rule on the stored logits
    for _ in range(2):                                           # scratch left clean; without the logits the same ids
        ids_only, _ = _run(c["hidden"], c["table"], "fast", with_logits=False)
        assert np.array_equal(ids_only, ids)
    want = want32.astype(np.float16).astype(np.float64)
    want_ids = _argmax(port, want32.astype(np.float16))
    for r in range(rows):
        others = np.delete(want[r], want_ids[r])
        margin = want[r, want_ids[r]] - (others.max() if others.size else -np.inf)
        if margin > 4 * bound[r].max():
            assert ids[r] == want_ids[r]


@pytest.mark.parametrize("rows", [8, 16, 64])
def test_many_rows_full_vocabulary_planted_winners(b2, port, rows):
    """151936 x 1024 fp16, one pass over the table for all rows: planted winners, and the logits of a sample of
    table rows (among them the first and last tiles) against the CPU operator."""
    c, planted = _planted(rows, 1024, wl.VOCAB, np.float16, seed=6900 + rows)
    ids, _ = _run(c["hidden"], c["table"], "fast", with_logits=False)
    assert np.array_equal(ids, planted)
    ids, logits = _run(c["hidden"], c["table"], "fast", with_logits=True)
    assert np.array_equal(ids, planted)
    rng = np.random.default_rng(rows)
    sample = np.unique(np.concatenate([np.arange(130), np.arange(wl.VOCAB - 130, wl.VOCAB), rng.integers(0, wl.VOCAB, 700)]))
    want32, scale = _oracle(port, c["hidden"], c["table"][sample])
    bound = RTOL * np.maximum(np.abs(want32.astype(np.float64)), scale) + ulp16(want32)
    err = np.abs(logits[:, sample].astype(np.float64) - want32.astype(np.float64))
    assert (err <= bound).all(), f"worst error / bound = {(err / bound).max():.3f}"
    assert np.array_equal(ids, _argmax(port, logits))


def test_many_rows_ties_and_special_values(b2, port):
    """The pick of the tensor-core kernel follows the reference's rule: ties to the lowest index (within a thread's
    rows, across the threads of a tile and across thread blocks), NaN never wins, a row of nothing comparable gives 0."""
    rows, vocab = 8, 1000
    hidden = np.zeros((rows, 1024), np.float16)
    for r in range(rows):
        hidden[r, r] = 1.0                               # logits of row r = table[:, r]
    table = np.zeros((vocab, 1024), np.float16)
    table[:, 0] = -5.0
    table[[17, 17 + 128, 900], 0] = 7.0                  # a tie inside one thread (rows 17 and 145), and across tiles
    table[:, 1] = 2.5                                    # all equal -> 0
    table[:, 2] = -65504.0                               # fp16's lowest finite value is an ordinary logit -> 0
    table[999, 4] = 1.0                                  # last row of the last (partial) tile
    table[300, 7], table[301, 7] = 3.0, 3.0
    table[:, 5] = -1.0
    table[[511, 512], 5] = 0.5                           # last thread of one tile, first of the next
    ids, logits = _run(hidden, table, "fast")
    assert ids.tolist() == [17, 0, 0, 0, 999, 511, 0, 300]
    assert np.array_equal(ids, _argmax(port, logits))
    # values that never win.  (A zero of the hidden row times an infinity or a NaN of the table is a NaN, so these
    # cases use one column only and every hidden row is a multiple of the first unit vector.)
    hidden = np.zeros((rows, 1024), np.float16)
    hidden[:, 0] = [1.0, -1.0, 2.0, 0.5, 1.0, 1.0, 1.0, 1.0]
    table = np.zeros((vocab, 1024), np.float16)
    table[:, 0] = np.nan
    table[640, 0] = -3.0                                 # the only comparable logit of every row
    ids, logits = _run(hidden, table, "fast")
    assert (ids == 640).all() and np.isnan(logits[0, 0]) and logits[1, 640] == np.float16(3.0)
    table[:, 0] = -np.inf                                # -inf never wins -> 0
    ids, logits = _run(hidden, table, "fast")
    assert ids.tolist() == [0, 0, 0, 0, 0, 0, 0, 0] and logits[1, 5] == np.inf and logits[0, 5] == -np.inf
    assert np.array_equal(ids, _argmax(port, logits))
    hidden[:, 0] = np.float16(65504.0)
    table[:, 0] = 2.0                                    # overflow to +inf everywhere: all equal -> 0
    ids, logits = _run(hidden, table, "fast")
    assert (ids == 0).all() and np.isinf(logits).all()
