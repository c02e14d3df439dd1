"""Second oracle: the reference's OWN CUDA operators (src/ops_cuda.cu), recompiled for sm_100a into
oracle/_ref/libref_cuda.so, run on the same GPU and the same device buffers.

Deterministic mode exists so that the reference's bit-level regressions can still be run: where the
arithmetic is IEEE-exact (RMSNorm family, add, gather, argmax) it must reproduce the reference kernels
bit for bit.  SwiGLU, RoPE and softmax go through device libm functions compiled from different source
text, so they are held to an fp32 ulp-level bound instead.  Fast mode is compared at the tolerances the
reference's own GPU tests use (1e-4 for F32, 5e-3 for F16: tests/test_ops_cuda.cpp:121-151)."""
import numpy as np
import pytest
import torch

import oracle
from cuda_llm_b200 import lib, ops, workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def refcu(b2):
    r = oracle.ref_cuda()
    if r is None:
        pytest.skip("oracle/_ref/libref_cuda.so not built (reference tree absent at build time)")
    return r


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def code(t):
    return lib.F32 if t.dtype == torch.float32 else lib.F16


def bits(t):
    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


@pytest.mark.parametrize("rows,hidden", [(4, 1024), (65, 2048), (3, 4096), (96, 128), (5, 1000), (512, 4096)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_deterministic_norms_equal_reference_kernels_bitwise(refcu, rows, hidden, dtype):
    rng = np.random.default_rng(rows + hidden)
    x, r = dev(wl.normal(rng, (rows, hidden), dtype=dtype)), dev(wl.normal(rng, (rows, hidden), dtype=dtype))
    w = dev(wl.gamma(rng, hidden, dtype=dtype))
    want = torch.empty_like(x)
    refcu.rms_norm(x, w, want, rows, hidden, wl.EPS, code(x))
    got = ops.cuda_rms_norm(x, w, wl.EPS, "deterministic")
    assert torch.equal(bits(got), bits(want))
    want_res, want_nrm = torch.empty_like(x), torch.empty_like(x)
    refcu.add_rms_norm(x, r, w, want_res, want_nrm, rows, hidden, wl.EPS, code(x))
    res, nrm = torch.empty_like(x), torch.empty_like(x)
    ops.cuda_add_rms_norm_out(x, r, w, wl.EPS, res, nrm, "deterministic")
    assert torch.equal(bits(res), bits(want_res)) and torch.equal(bits(nrm), bits(want_nrm))
    # fast mode: the reference's own GPU-test tolerances
    tol = 1e-4 if dtype == np.float32 else 5e-3
    fast_res, fast_nrm = torch.empty_like(x), torch.empty_like(x)
    ops.cuda_add_rms_norm_out(x, r, w, wl.EPS, fast_res, fast_nrm, "fast")
    assert torch.equal(bits(fast_res), bits(want_res))
    scale = max(1.0, float(want_nrm.float().abs().max()))
    assert float((fast_nrm.float() - want_nrm.float()).abs().max()) <= tol * scale
    want_add = torch.empty_like(x)
    refcu.add(x, r, want_add, rows * hidden, code(x))
    assert torch.equal(bits(ops.cuda_add(x, r)), bits(want_add))


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_gather_and_argmax_equal_reference_kernels(refcu, dtype):
    rng = np.random.default_rng(8)
    table = dev(wl.normal(rng, (3000, 1024), 0.02, dtype))
    ids = rng.integers(0, 3000, 257).astype(np.int32)
    want = torch.empty(257, 1024, dtype=table.dtype, device=DEV)
    refcu.embedding_lookup(table, ids, want, 1024, 3000, code(table))
    assert torch.equal(bits(ops.cuda_embedding_lookup(table, ids.tolist())), bits(want))
    logits = np.round(wl.normal(rng, (3, wl.VOCAB), 4.0) * 2) / 2            # ties
    logits = dev(logits.astype(dtype))
    assert ops.cuda_argmax_last_row(logits) == refcu.argmax_last_row(logits, 3, wl.VOCAB, code(logits))
    each = [refcu.argmax_last_row(logits[r:r + 1].contiguous(), 1, wl.VOCAB, code(logits)) for r in range(3)]
    assert ops.argmax_rows(logits).tolist() == each


def test_argmax_lowest_finite_value_against_the_reference_kernel(refcu, port):
    """What the reference's fold starts from decides rows whose only candidates are -inf and -FLT_MAX.  Its
    source starts at -CUDART_INF_F, and with the headers that file includes that macro is the file's own
    fallback, 3.402823466e+38F (src/ops_cuda.cu:21-23): -FLT_MAX is the start value and never wins, so such a
    row gives index 0.  The reference's compiled kernel on this GPU is the judge of that reading."""
    f = np.float32
    lowest = np.finfo(f).min
    cases = [[-np.inf, lowest, -np.inf], [lowest, lowest, lowest], [-np.inf, lowest, np.nextafter(lowest, f(0))],
             [np.nan, -np.inf, lowest, np.nan]]
    for row in cases:
        x = dev(np.asarray([row], f))
        want = refcu.argmax_last_row(x, 1, len(row), code(x))
        assert ops.cuda_argmax_last_row(x) == want, row
        assert int(port.argmax_rows(np.asarray([row], f))[0]) == want, row


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_deterministic_swiglu_rope_softmax_track_reference_kernels(refcu, dtype):
    rng = np.random.default_rng(21)
    tol = 4e-7 if dtype == np.float32 else 0.0     # relative, a few fp32 ulps; fp16 outputs must round identically
    g, u = dev(wl.normal(rng, 100003, 2.0, dtype)), dev(wl.normal(rng, 100003, 2.0, dtype))
    want = torch.empty_like(g)
    refcu.swiglu(g, u, want, g.numel(), code(g))
    got = ops.cuda_swiglu(g, u, "deterministic")
    if dtype == np.float16:
        assert float((bits(got).int() - bits(want).int()).abs().max()) <= 1          # same formula, same rounding: <= 1 ulp
        assert float((bits(got) != bits(want)).float().mean()) < 1e-3
    else:
        assert float(((got - want).abs() / want.abs().clamp_min(1e-30)).max()) <= tol
    # RoPE: the all-fp32 angle of the reference kernel (src/ops_cuda.cu:133), positions up to a prefill's length
    x = dev(wl.normal(rng, (300, 16, 128), dtype=dtype))
    pos = rng.integers(0, 512, 300).astype(np.int32)
    want = torch.empty_like(x)
    refcu.rope(x, pos, want, 300, 16, 128, 1e6, code(x))
    got = ops.cuda_rope(x, pos.tolist(), 1e6, "deterministic")
    bound = 2e-6 if dtype == np.float32 else 2 ** -9
    assert float((got.float() - want.float()).abs().max()) <= bound * max(1.0, float(x.float().abs().max()))
    if dtype == np.float16:
        tp = torch.empty_like(x)
        refcu.rope_token_positions(x, dev(pos), tp, 300, 16, 1e6)
        assert torch.equal(bits(tp), bits(want))             # the reference's two entry points agree with each other
    # softmax: same order, same fp32 accumulator
    lg = dev(wl.normal(rng, (4, 8192), 4.0, dtype))
    want = torch.empty_like(lg)
    refcu.softmax(lg, want, 4, 8192, code(lg))
    got = ops.cuda_softmax_last_dim(lg, "deterministic")
    peak = want.float().max(dim=1, keepdim=True).values
    assert float(((got.float() - want.float()).abs() / torch.maximum(want.float(), peak)).max()) <= (2e-6 if dtype == np.float32 else 2e-3)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows", [1, 4])
def test_lm_head_argmax_against_the_reference_decode_tail(refcu, rows, dtype):
    """The reference's decode tail on the same GPU: cuda_lm_head (its library GEMM) into a logits tensor, then
    cuda_argmax_last_row.  Its summation order is the GEMM library's, so logits are compared at the reference's own
    GPU-test tolerances (1e-4 / 5e-3), the index of the last row exactly (a planted winner decides it)."""
    c = wl.lm_head_case(rows, 1024, wl.VOCAB, seed=6700 + rows, dtype=dtype)
    planted = 1000 + 37 * rows
    c["table"][planted] = (c["hidden"][rows - 1].astype(np.float32) * np.float32(0.02)).astype(dtype)
    h, t = dev(c["hidden"]), dev(c["table"])
    want_logits = torch.empty(rows, wl.VOCAB, dtype=h.dtype, device=DEV)
    want_id = refcu.lm_head_argmax(h, t, rows, 1024, wl.VOCAB, code(h), want_logits)
    assert want_id == planted
    tol = 1e-4 if dtype == np.float32 else 5e-3
    for mode in ("fast", "deterministic"):
        got_logits = torch.empty_like(want_logits)
        ids = ops.lm_head_argmax(h, t, logits_out=got_logits, mode=mode)
        assert int(ids[rows - 1]) == want_id
        scale = max(1.0, float(want_logits.float().abs().max()))
        assert float((got_logits.float() - want_logits.float()).abs().max()) <= tol * scale

