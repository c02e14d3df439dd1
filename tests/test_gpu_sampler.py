"""GPU parity of temperature / top-k / top-p sampling (b2_sample_rows) through the C ABI:
the reference's own sampler test cases (tests/test_sampling_cuda.cpp), bit equality with the
reference's own CudaSampler recompiled for this GPU, and agreement with the C restatement."""
import numpy as np
import pytest
import torch

import oracle
from cuda_llm_b200 import ops, workloads as wl
from cuda_llm_b200.ops import CudaSampler, SamplingConfig

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()


def test_reference_sampler_test_cases(b2):
    """reference tests/test_sampling_cuda.cpp:18-70."""
    sampler = CudaSampler(151936)
    x = np.array([[-3, 1, 8, 2, 4, 0], [2, 9, 1, 7, 3, 5]], np.float32)
    xf, x16 = dev(x), dev(x.astype(np.float16))
    zero = SamplingConfig(temperature=0, top_k=0, top_p=0.0)               # top_p ignored at temperature zero
    assert sampler.sample_last_row(xf, zero, 0) == ops.cuda_argmax_last_row(xf) == 1
    assert sampler.sample_last_row(x16, zero, 0) == ops.cuda_argmax_last_row(x16)
    one = SamplingConfig(temperature=1, top_k=1, top_p=1)
    assert sampler.sample_last_row(xf, one, 0) == 1                          # top_k = 1 is greedy
    d = SamplingConfig(temperature=1, top_k=3, top_p=1, seed=42)
    assert sampler.sample_last_row(xf, d, 7) == sampler.sample_last_row(xf, d, 7)
    small = dev(np.array([[10, 9, 0, -1, -2, -3]], np.float32))
    k2 = SamplingConfig(temperature=1, top_k=2, top_p=1, seed=1)
    assert all(sampler.sample_last_row(small, k2, i) in (0, 1) for i in range(20))
    combo = SamplingConfig(temperature=1, top_k=3, top_p=0.5, seed=2)
    assert all(sampler.sample_last_row(small, combo, i) in (0, 1) for i in range(20))
    crossing_cpu = np.array([[np.log(np.float32(0.505)), np.log(np.float32(0.495)), -20, -20, -20, -20]], np.float32)
    cfg = SamplingConfig(temperature=1.0, top_k=0, top_p=0.51, seed=77)
    for t in (dev(crossing_cpu), dev(crossing_cpu.astype(np.float16))):
        seen = [sampler.sample_last_row(t, cfg, o) for o in range(64)]
        assert set(seen) == {0, 1}                                          # truncated tokens never, the crossing token sometimes
    ties_cpu = np.array([[0, 0, 0, -10, -10, -10]], np.float32)
    tie = SamplingConfig(temperature=1.0, top_k=0, top_p=0.30, seed=88)
    for t in (dev(ties_cpu), dev(ties_cpu.astype(np.float16))):
        assert all(sampler.sample_last_row(t, tie, o) == 0 for o in range(64))   # equal maxima: the lowest id
    large = np.full((1, 151936), -2, np.float32)
    large[0, 123456] = 8
    assert sampler.sample_last_row(dev(large), zero, 0) == 123456
    assert sampler.sample_last_row(dev(large.astype(np.float16)), zero, 0) == 123456
    # rejections (:62-69)
    with pytest.raises(ValueError):
        sampler.sample_last_row(torch.from_numpy(x), one, 0)                 # CPU tensor
    with pytest.raises(ValueError):
        sampler.sample_last_row(torch.zeros(1, 2, 1, device=DEV), one, 0)    # rank
    with pytest.raises(ValueError):
        sampler.sample_last_row(torch.zeros(1, 2, device=DEV, dtype=torch.bfloat16), one, 0)
    with pytest.raises(ValueError):
        sampler.sample_last_row(torch.zeros(0, 2, device=DEV), one, 0)
    with pytest.raises(ValueError):
        sampler.sample_last_row(xf, SamplingConfig(temperature=-1, top_k=1, top_p=1), 0)
    with pytest.raises(ValueError):
        sampler.sample_last_row(xf, SamplingConfig(temperature=1, top_k=7, top_p=1), 0)
    with pytest.raises(ValueError):
        sampler.sample_last_row(xf, SamplingConfig(temperature=1, top_k=1, top_p=0), 0)


# top_k values on both sides of every path boundary: 1, small (sampled threshold), 2048 (largest for that path),
# 3000 (whole-row sort), 0 (everything)
CONFIGS = [SamplingConfig(1.0, 0, 1.0, 11), SamplingConfig(0.7, 50, 1.0, 12), SamplingConfig(1.3, 0, 0.9, 13),
           SamplingConfig(0.8, 40, 0.95, 14), SamplingConfig(1.0, 2048, 0.5, 15), SamplingConfig(2.0, 3000, 0.999, 16),
           SamplingConfig(1.0, 1, 1.0, 17), SamplingConfig(0.5, 0, 0.3, 18), SamplingConfig(1.1, 700, 0.98, 19),
           SamplingConfig(0.9, 2048, 1.0, 20), SamplingConfig(1.0, 5, 0.7, 21)]


def rows_for(width, rows, seed, dtype, kind="ties"):
    rng = np.random.default_rng(seed)
    x = wl.normal(rng, (rows, width), 4.0)
    if kind == "ties":
        x[1, : width // 2] = x[1, 0]                # a long run of equal scores: the tie rule decides
        x[2, :] = 0.0                               # every score equal
        if width > 100:
            x[3, 7], x[3, 99] = 30.0, 30.0          # two equal maxima
    elif kind == "narrow":
        x = 16.0 + rng.random((rows, width), dtype=np.float32)   # every score in one binade: the coarse cut cannot separate them
    return x.astype(dtype)


@pytest.mark.parametrize("width,dtype,kind", [(6, np.float32, "ties"), (1000, np.float32, "ties"), (4096, np.float16, "ties"),
                                              (5000, np.float32, "ties"), (151936, np.float32, "ties"),
                                              (151936, np.float16, "ties"), (151936, np.float32, "plain"),
                                              (151936, np.float16, "plain"), (40000, np.float32, "plain"),
                                              (151936, np.float32, "narrow")])
def test_every_row_equals_the_references_own_sampler_and_the_restatement(b2, port, width, dtype, kind):
    """"plain" rows take the two-pass top-k path alone; "ties" and "narrow" rows crowd the cut bin and send the
    call through the exact radix select; top_k == 0 and top_k > 2048 sort the whole row."""
    refcu = oracle.ref_cuda()
    rows = 8
    x = rows_for(width, rows, width, dtype, kind)
    t = dev(x)
    xf = x.astype(np.float32)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    offsets = np.arange(rows, dtype=np.int64) * 1000003 + 5
    code = 0 if dtype == np.float32 else 1
    for cfg in CONFIGS:
        if cfg.top_k > width:
            continue
        ops.sample_rows_out(t, cfg, dev(offsets), out)
        got = host(out)
        for r in range(rows):
            if refcu is not None and (width <= 5000 or r < 4):
                want = refcu.sample_row(t, rows, width, code, r, cfg.temperature, cfg.top_k, cfg.top_p, cfg.seed, int(offsets[r]))
                assert int(got[r]) == want, f"row {r} {cfg}: {int(got[r])} vs the reference's {want}"
            token, margin = port.sample_row(xf[r], cfg.temperature, cfg.top_k, cfg.top_p, cfg.seed, int(offsets[r]))
            assert int(got[r]) == token or margin < 1e-5, f"row {r} {cfg}: {int(got[r])} vs the restatement's {token}"
    again = torch.empty_like(out)
    repeat = CONFIGS[3] if width >= 40 else CONFIGS[2]
    ops.sample_rows_out(t, repeat, dev(offsets), again)
    ops.sample_rows_out(t, repeat, dev(offsets), out)
    assert torch.equal(out, again)


@pytest.mark.parametrize("temperature", [1e-7, 3e7])
def test_extreme_temperatures_take_the_exact_path(b2, port, temperature):
    """logits / temperature overflows (tiny temperature) or flushes towards zero (huge): scores of different logits
    collapse and the index order decides, which only the exact select over the true scores gets right."""
    refcu = oracle.ref_cuda()
    rows, width = 4, 151936
    x = rows_for(width, rows, 99, np.float32, "plain")
    x[0, :20000] *= 1e32                         # overflows to +-inf at the small temperature
    x[1] *= 1e-33                                # denormal scores at the large temperature
    t = dev(x)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    offsets = np.arange(rows, dtype=np.int64) + 3
    for cfg in (SamplingConfig(temperature, 50, 1.0, 5), SamplingConfig(temperature, 7, 0.9, 6)):
        ops.sample_rows_out(t, cfg, dev(offsets), out)
        got = host(out)
        for r in range(rows):
            if refcu is not None:
                want = refcu.sample_row(t, rows, width, 0, r, cfg.temperature, cfg.top_k, cfg.top_p, cfg.seed, int(offsets[r]))
                assert int(got[r]) == want, f"row {r} {cfg}: {int(got[r])} vs the reference's {want}"


def test_draws_follow_the_retained_distribution(b2, port):
    """Frequencies over many draw offsets match the truncated, renormalised softmax (a property the
    reference's tests do not check, independent of any oracle)."""
    rng = np.random.default_rng(5)
    row = wl.normal(rng, (1, 2000), 2.0)
    n = 4000
    x = dev(np.repeat(row, n, axis=0))
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    cfg = SamplingConfig(temperature=1.0, top_k=20, top_p=1.0, seed=9)
    ops.sample_rows_out(x, cfg, dev(np.arange(n, dtype=np.int64)), out)
    got = host(out)
    top = np.argsort(-row[0], kind="stable")[:20]
    assert set(np.unique(got)) <= set(top.tolist())
    p = np.exp(row[0, top].astype(np.float64) - row[0, top[0]])
    p /= p.sum()
    freq = np.array([(got == t).mean() for t in top])
    assert np.abs(freq - p).max() < 4 * np.sqrt(0.25 / n)


def test_rows_handed_back_by_the_top_p_route_inside_a_graph_and_before_other_kernels(b2, port):
    """Rows the top-p route cannot settle (flat rows, long ties) are redone by kernels launched from the device.
    The same call recorded into a CUDA graph and replayed, with another operator of the library queued right
    behind it (a kernel that may start early under programmatic serialisation), gives the same tokens."""
    from cuda_llm_b200 import lib
    L = b2
    rows, width = 8, wl.VOCAB
    x = rows_for(width, rows, 4242, np.float32, "ties")          # rows 1 and 2 are flat: they take the whole-row route
    t = dev(x)
    cfg = SamplingConfig(1.0, 0, 0.9, 31)
    offsets = np.arange(rows, dtype=np.int64) * 7 + 1
    off = dev(offsets)
    want = [port.sample_row(x[r], cfg.temperature, cfg.top_k, cfg.top_p, cfg.seed, int(offsets[r])) for r in range(rows)]
    ws = torch.zeros(L.b2_sampler_workspace_bytes(rows, width), dtype=torch.uint8, device=DEV)
    a = torch.ones(1 << 20, dtype=torch.float16, device=DEV)
    b = torch.full((1 << 20,), 2.0, dtype=torch.float16, device=DEV)
    c = torch.zeros(1 << 20, dtype=torch.float16, device=DEV)

    def step(out, stream):
        lib.check(L.b2_sample_rows(t.data_ptr(), rows, width, width, lib.F32, cfg.temperature, cfg.top_k, cfg.top_p, cfg.seed,
                                   off.data_ptr(), out.data_ptr(), ws.data_ptr(), stream))
        lib.check(L.b2_add(a.data_ptr(), b.data_ptr(), c.data_ptr(), a.numel(), lib.F16, stream))

    eager = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    for _ in range(3):
        step(eager, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for r in range(rows):
        assert int(eager[r]) == want[r][0] or want[r][1] < 1e-5, f"row {r}"
    assert float(c[12345]) == 3.0
    replayed = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step(replayed, side.cuda_stream)
    for _ in range(2):
        replayed.fill_(-1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(replayed, eager)


def test_c_abi_argument_rules(b2):
    from cuda_llm_b200 import lib
    L = b2
    x = dev(np.zeros((2, 8), np.float32))
    out = torch.empty(2, dtype=torch.int32, device=DEV)
    ws = torch.empty(L.b2_sampler_workspace_bytes(2, 8), dtype=torch.uint8, device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    call = lambda t, k, p: L.b2_sample_rows(x.data_ptr(), 2, 8, 8, lib.F32, t, k, p, 1, None, out.data_ptr(), ws.data_ptr(), s)
    assert call(1.0, 0, 1.0) == 0
    assert call(float("nan"), 0, 1.0) == -1 and call(-1.0, 0, 1.0) == -1
    assert call(1.0, 9, 1.0) == -1 and call(1.0, -1, 1.0) == -1
    assert call(1.0, 0, 0.0) == -1 and call(1.0, 0, 1.5) == -1
    assert call(0.0, 99, 0.0) == 0          # ignored at temperature zero, as in the reference
    torch.cuda.synchronize()
    assert host(out).tolist() == [0, 0]
