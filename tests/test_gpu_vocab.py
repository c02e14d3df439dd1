"""GPU parity of the vocabulary-wide reductions (argmax, softmax), through the C ABI."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, sharded, workloads as wl
from util import assert_within_1ulp_f16, f16_bits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()


# ---- argmax: bit-exact indices ------------------------------------------------------------------

def test_argmax_reference_test_cases(b2):
    """reference tests/test_argmax_cuda.cpp:42-57."""
    am = lambda a: ops.cuda_argmax_last_row(dev(np.asarray(a)))
    f = np.float32
    assert am(np.array([[-1, 2, 3, 4, 5], [1, 9, 2, 8, 3]], f)) == 1
    assert am(np.array([[-1, 2, 3, 4, 5], [1, 9, 2, 8, 3]], np.float16)) == 1
    assert am(np.array([[4, 7, 7, 1, 7, 2]], f)) == 1
    assert am(np.array([[-1, -2, -3, -4]], np.float16)) == 0
    two = np.full((2, wl.VOCAB), -10, f)
    two[0, 11], two[1, 12345] = 100, 101
    assert am(two) == 12345
    tie = np.full((1, wl.VOCAB), -10, np.float16)
    tie[0, 11], tie[0, 12345], tie[0, wl.VOCAB - 1] = 100, 101, 101
    assert am(tie) == 12345
    with pytest.raises(ValueError):
        ops.cuda_argmax_last_row(torch.zeros(1, 2))                                  # CPU input
    with pytest.raises(ValueError):
        ops.cuda_argmax_last_row(torch.zeros(2, 2, 1, device=DEV))                   # rank
    with pytest.raises(ValueError):
        ops.cuda_argmax_last_row(torch.zeros(1, 2, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):
        ops.cuda_argmax_last_row(torch.zeros(0, 2, device=DEV))


def test_argmax_recorded_greedy_ids(b2, golden):
    g = golden("logits_last_rows")
    for case in ("case_seq4", "case_seq8"):
        row = g[case + "_last_row"]
        assert ops.cuda_argmax_last_row(dev(row[None])) == int(g[case + "_greedy_id"][0])
        assert ops.cuda_argmax_last_row(dev(np.stack([row[::-1], row]))) == int(g[case + "_greedy_id"][0])


@pytest.mark.parametrize("rows,width", [(1, 1), (1, 5), (3, 1000), (4, wl.VOCAB), (256, 18992), (37, 4099), (600, 257),
                                        (2, 1 << 20)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_argmax_rows_random_and_ties(b2, port, rows, width, dtype):
    rng = np.random.default_rng(rows * 7 + width)
    x = wl.normal(rng, (rows, width), 4.0)
    x = np.round(x * 4) / 4                     # coarse grid: plenty of exact ties, in both dtypes
    x = x.astype(dtype)
    want = port.argmax_rows(x if dtype == np.float32 else f16_bits(x))
    for _ in range(2):                          # twice: the scratch must come back zeroed
        assert np.array_equal(host(ops.argmax_rows(dev(x))), want)


def test_argmax_special_values(b2, port):
    f = np.float32
    rows = np.array([[np.nan, -np.inf, -3.4028235e38, np.nan],          # nothing can win -> 0
                     [np.nan, 1, np.nan, 1],                             # NaN never wins, tie -> 1
                     [-np.inf, -3.4028235e38, -3.4028234e38, -np.inf],   # just above -FLT_MAX wins
                     [np.inf, np.inf, 0, 0],
                     [-0.0, 0.0, -0.0, 0.0]], f)                         # -0 == +0: lowest index
    assert np.array_equal(host(ops.argmax_rows(dev(rows))), port.argmax_rows(rows))
    wide = np.full((3, 70000), -np.inf, f)
    wide[1, 69999] = -1e30
    wide[2, :] = np.nan
    assert np.array_equal(host(ops.argmax_rows(dev(wide))), [0, 69999, 0])


def test_argmax_config1_and_config5(b2, port):
    c = wl.config1(with_table=False)
    assert np.array_equal(host(ops.argmax_rows(dev(c["logits"]))), port.argmax_rows(c["logits"]))
    c5 = wl.config5()
    got = host(ops.argmax_rows(dev(c5["logits"])))
    assert np.array_equal(got, c5["planted"]) and np.array_equal(got, port.argmax_rows(c5["logits"]))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_vocab_sharded_argmax_keys_single_gpu_emulation(b2, port, world):
    """All shards' kernels run on one GPU; the exchange is a max over the stacked keys, which is what
    the int64 all-reduce(MAX) computes.  Checks the key packing, index_base and tie rule across shards."""
    c5 = wl.config5(rows=64)
    x = np.round(c5["logits"])                   # ties across shards
    keys = []
    for r in range(world):
        lo, hi = sharded.column_range(wl.VOCAB, world, r)
        keys.append(sharded.argmax_keys(dev(x[:, lo:hi]), lo))
    merged = torch.stack(keys).max(dim=0).values
    assert np.array_equal([sharded.decode_key(int(k)) for k in host(merged)], port.argmax_rows(x))
    lo, hi = sharded.column_range(wl.VOCAB, world, 1)
    k0 = host(sharded.argmax_keys(dev(x[:3, lo:hi]), lo))
    for r in range(3):
        i = int(port.argmax_rows(x[r:r + 1, lo:hi])[0])
        assert int(k0[r]) == port.argmax_key(float(x[r, lo + i]), lo + i)
    empty = sharded.argmax_keys(dev(np.full((2, 4096), -np.inf, np.float32)), 4096)
    assert [int(k) for k in host(empty)] == [sharded.KEY_NONE] * 2


# ---- softmax ---------------------------------------------------------------------------------

def scaled_err(got, want):
    """max |got - want| / max(|want|, row max probability)."""
    want = np.asarray(want, dtype=np.float64)
    floor = want.max(axis=-1, keepdims=True)
    return float((np.abs(got.astype(np.float64) - want) / np.maximum(want, floor)).max())


def softmax_check(got, x, port, mode, what):
    """The CPU operator adds ~150k exponentials into one fp32 accumulator in index order
    (src/ops_cpu.cpp:13): once the sum is ~1, terms below half an ulp of it are dropped, and the
    result drifts from the exact softmax by up to a few 1e-4 at vocabulary width.  So:
      deterministic mode (same order, same fp32 accumulator) must match the CPU operator to 1e-5;
      fast mode (parallel partial sums) must match the EXACT softmax to 1e-5, and the CPU operator
      to 1e-5 plus that operator's own measured distance from the exact answer on this input."""
    cpu, exact = port.softmax(x), port.softmax_f64(x)
    if mode == "deterministic":
        assert scaled_err(got, cpu) <= 1e-5, f"{what}: {scaled_err(got, cpu):.3e} vs ops_cpu"
    else:
        assert scaled_err(got, exact) <= 1e-5, f"{what}: {scaled_err(got, exact):.3e} vs exact"
        drift = scaled_err(cpu, exact)
        assert scaled_err(got, cpu) <= 1e-5 + drift, f"{what}: {scaled_err(got, cpu):.3e} vs ops_cpu (its drift {drift:.3e})"
        assert abs(float(got.astype(np.float64).sum(axis=-1).max()) - 1) <= 1e-5


@pytest.mark.parametrize("rows,width", [(2, 4), (1, 1), (5, 1000), (3, 4099), (4, 8192), (7, 30000), (2, 151936),
                                        (1, 500000), (300, 128)])
@pytest.mark.parametrize("mode", ["fast", "deterministic"])
def test_softmax_f32(b2, port, rows, width, mode):
    rng = np.random.default_rng(rows + width)
    x = wl.normal(rng, (rows, width), 4.0)
    got = host(ops.cuda_softmax_last_dim(dev(x), mode))
    softmax_check(got, x, port, mode, f"softmax {mode} {rows}x{width}")
    assert ops.softmax_status(DEV, rows) == 0          # no bounded wait ran out


@pytest.mark.parametrize("rows,width,dtype", [(80, 151936, np.float32), (100, 60004, np.float32), (333, 30000, np.float32),
                                              (600, 4096, np.float16), (90, 151936, np.float16), (2000, 1000, np.float32)])
def test_softmax_many_rows_streaming_clusters(b2, port, rows, width, dtype):
    """More rows than clusters fit the GPU at once: the persistent kernel walks several rows per cluster
    (copy engine one row ahead, statistics exchanged through remote shared-memory stores).  Includes
    ragged last slices, slices and warps that are entirely masked (-inf), and one fully masked row."""
    rng = np.random.default_rng(rows * 7 + width)
    x = wl.normal(rng, (rows, width), 4.0).astype(dtype)
    x[1, : width // 2] = -np.inf            # whole slices of a row masked
    x[2, width // 3:] = -np.inf
    x[3, 5:] = -np.inf                      # nearly everything masked
    x[rows - 1, :] = -np.inf                # nothing left: 0/0 like the reference
    got = host(ops.cuda_softmax_last_dim(dev(x), "fast"))
    assert ops.softmax_status(DEV, rows) == 0
    assert np.isnan(got[rows - 1].astype(np.float32)).all()
    live = np.arange(rows) != rows - 1
    xf = x[live].astype(np.float32)
    if dtype == np.float32:
        softmax_check(got[live], xf, port, "fast", f"streaming softmax {rows}x{width}")
    else:
        assert_within_1ulp_f16(got[live], port.softmax_f64(xf), f"streaming softmax f16 {rows}x{width}")
    again = host(ops.cuda_softmax_last_dim(dev(x), "fast"))
    assert np.array_equal(got.view(np.uint8), again.view(np.uint8))     # run-to-run bit-identical


def test_softmax_reference_test_literals(b2, port):
    """reference tests/test_ops_cuda.cpp:142-151."""
    sm = np.array([[1000, 1001, -1000, -999], [1, 2, 3, 4]], np.float32)
    for mode in ("fast", "deterministic"):
        assert np.abs(host(ops.cuda_softmax_last_dim(dev(sm), mode)) - port.softmax(sm)).max() <= 1e-4
        sm16 = sm.astype(np.float16)
        got = host(ops.cuda_softmax_last_dim(dev(sm16), mode)).astype(np.float32)
        assert np.abs(got - port.softmax(sm16.astype(np.float32))).max() <= 5e-3
        assert np.abs(got.sum(axis=1) - 1).max() <= 5e-3
    masked = np.array([[-np.inf, 0, 1, -np.inf, 2]], np.float32)
    assert np.abs(host(ops.cuda_softmax_last_dim(dev(masked))) - port.softmax(masked)).max() <= 1e-6
    with pytest.raises(ValueError):
        ops.cuda_softmax_last_dim(torch.zeros(2, 0, device=DEV))


def test_softmax_committed_reference_output_and_config5(b2, port, golden):
    c5 = wl.config5(rows=4, vocab=8192, seed=5002)
    want = golden("small_reference")["c5_softmax"]          # the reference's compiled softmax_last_dim
    got = host(ops.cuda_softmax_last_dim(dev(c5["logits"]), "deterministic"))
    assert scaled_err(got, want) <= 1e-5
    got = host(ops.cuda_softmax_last_dim(dev(c5["logits"]), "fast"))
    assert scaled_err(got, want) <= 1e-5 + scaled_err(want, port.softmax_f64(c5["logits"]))
    full = wl.config5(rows=16)
    for mode in ("fast", "deterministic"):
        softmax_check(host(ops.cuda_softmax_last_dim(dev(full["logits"]), mode)), full["logits"], port, mode,
                      f"config5 {mode}")


@pytest.mark.parametrize("world", [2, 8])
def test_vocab_sharded_softmax_single_gpu_emulation(b2, port, world):
    """stats -> max exchange -> rebase -> sum exchange -> apply, with the exchanges done as torch
    reductions over the shards' statistics on one GPU."""
    from cuda_llm_b200 import lib
    L = lib.load()
    c5 = wl.config5(rows=8)
    x = c5["logits"]
    shards = [dev(x[:, slice(*sharded.column_range(wl.VOCAB, world, r))]) for r in range(world)]
    mx = [torch.empty(8, device=DEV) for _ in shards]
    sm = [torch.empty(8, device=DEV) for _ in shards]
    s = torch.cuda.current_stream().cuda_stream
    for t, m, z in zip(shards, mx, sm):
        lib.check(L.b2_softmax_stats(t.data_ptr(), 8, t.shape[1], 0, m.data_ptr(), z.data_ptr(), s))
    gmax = torch.stack(mx).max(dim=0).values
    for m, z in zip(mx, sm):
        lib.check(L.b2_softmax_rebase(m.data_ptr(), gmax.data_ptr(), z.data_ptr(), 8, s))
    gsum = torch.stack(sm).sum(dim=0)
    outs = []
    for t in shards:
        o = torch.empty_like(t)
        lib.check(L.b2_softmax_apply(t.data_ptr(), o.data_ptr(), 8, t.shape[1], 0, gmax.data_ptr(), gsum.data_ptr(), s))
        outs.append(host(o))
    softmax_check(np.concatenate(outs, axis=1), x, port, "fast", f"sharded softmax world={world}")
    # preallocated buffers (the form recorded into CUDA graphs together with the all-reduces)
    keys, ids = torch.empty(8, dtype=torch.int64, device=DEV), torch.empty(8, dtype=torch.int32, device=DEV)
    stats, out = torch.empty(3, 8, device=DEV), torch.empty(8, wl.VOCAB, device=DEV)
    assert sharded.sharded_argmax(dev(x), 0, keys=keys, out=ids) is ids
    assert np.array_equal(host(ids), port.argmax_rows(x))
    assert sharded.sharded_softmax(dev(x), out=out, stats=stats) is out
    softmax_check(host(out), x, port, "fast", "sharded softmax, preallocated")
    # the driver function itself, as a world of one (no process group initialised)
    softmax_check(host(sharded.sharded_softmax(dev(x))), x, port, "fast", "sharded softmax, one rank")
    assert np.array_equal(host(sharded.sharded_argmax(dev(x), 0)), port.argmax_rows(x))
