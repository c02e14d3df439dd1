"""b2_ordered_sums: the fp32 running sums of descending terms, added one after the other in index order as the single
thread of the reference's sampler_select does (src/ops_cuda.cu:587-603), computed by a thread block.  The check is
exact: numpy float32 additions in a Python loop ARE that sequential sum."""
import ctypes as C

import numpy as np
import pytest
import torch

from cuda_llm_b200 import lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def sequential(rows):
    out = np.empty_like(rows)
    for r in range(rows.shape[0]):
        s = np.float32(0)
        for i in range(rows.shape[1]):
            s = np.float32(s + rows[r, i])
            out[r, i] = s
    return out


def run(L, rows):
    t = torch.from_numpy(np.ascontiguousarray(rows)).to(DEV)
    out = torch.empty_like(t)
    lib.check(L.b2_ordered_sums(t.data_ptr(), rows.shape[0], rows.shape[1], out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out.cpu().numpy()


def softmax_terms(rng, n, sigma):
    x = np.sort((rng.standard_normal(n) * sigma).astype(np.float32))[::-1]
    return np.exp(x - x[0]).astype(np.float32)


@pytest.mark.parametrize("n", [1, 2, 63, 64, 65, 257, 1000, 2800, 4096])
def test_running_sums_equal_the_sequential_fp32_sum(b2, n):
    rng = np.random.default_rng(n)
    rows = []
    for sigma in (0.5, 1.0, 2.0, 4.0, 8.0):
        rows.append(softmax_terms(rng, n, sigma))                                   # what the sampler's head looks like
        e = softmax_terms(rng, n, sigma)
        rows.append(np.maximum(np.round(e * 1024) / 1024, np.float32(1 / 1024)).astype(np.float32))   # dyadic terms: ties everywhere
    rows.append(np.ones(n, dtype=np.float32))                                       # a flat row: the sum doubles again and again
    rows.append(np.full(n, np.float32(0.75)))
    rows.append((np.float32(1.0) / (1 + np.arange(n, dtype=np.float32))).astype(np.float32))       # harmonic
    rows.append(np.concatenate([[np.float32(1)], np.full(n - 1, np.float32(2.0 ** -24))]).astype(np.float32)[:n])  # halves of the unit
    rows.append(np.concatenate([[np.float32(1)], np.full(n - 1, np.float32(2.0 ** -23 * 1.5))]).astype(np.float32)[:n])  # ties at every term
    rows.append(np.zeros(n, dtype=np.float32))
    rows = np.stack(rows).astype(np.float32)
    got = run(b2, rows)
    want = sequential(rows)
    bad = np.nonzero(got.view(np.uint32) != want.view(np.uint32))
    assert bad[0].size == 0, f"row {bad[0][0]} index {bad[1][0]}: {got[bad[0][0], bad[1][0]]!r} vs {want[bad[0][0], bad[1][0]]!r}"


def test_in_place_and_argument_rules(b2):
    L = b2
    rng = np.random.default_rng(3)
    rows = np.stack([softmax_terms(rng, 3000, 4.0) for _ in range(4)])
    t = torch.from_numpy(rows).to(DEV)
    lib.check(L.b2_ordered_sums(t.data_ptr(), 4, 3000, t.data_ptr(), torch.cuda.current_stream().cuda_stream))
    assert np.array_equal(t.cpu().numpy().view(np.uint32), sequential(rows).view(np.uint32))
    s = torch.cuda.current_stream().cuda_stream
    assert L.b2_ordered_sums(t.data_ptr(), 1, 4097, t.data_ptr(), s) == -1
    assert L.b2_ordered_sums(None, 1, 8, t.data_ptr(), s) == -1
    assert L.b2_ordered_sums(None, 0, 8, None, s) == 0
