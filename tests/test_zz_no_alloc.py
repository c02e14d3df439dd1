"""The allocation-free argmax entry point (b2_argmax_rows_static), through the C ABI.

Some users of this library may not allocate device memory at all once they are running: a serving
process that hands every byte of the GPU to its own pool at start-up, or a plug-in that gets tensors
from its host but no allocator.  For them the argmax scratch sits in a fixed array inside the library.
This test calls that entry point twice in a row and checks both results against the ordinary entry
point (b2_argmax_rows with a caller workspace): indices are integers, so the match is exact.  The
second call proves the shared array is usable again after the first; a third, smaller call proves a
call only depends on the part of the array it clears.  The file name sorts last so a run that stops at
the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import lib, workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference_ids(L, x, stream):
    rows, width = x.shape
    ws = torch.zeros(L.b2_argmax_workspace_bytes(rows), dtype=torch.uint8, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    code = lib.F32 if x.dtype == torch.float32 else lib.F16
    lib.check(L.b2_argmax_rows(x.data_ptr(), rows, width, width, code, out.data_ptr(), ws.data_ptr(), stream))
    return out


def _static_ids(L, x, stream):
    rows, width = x.shape
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    code = lib.F32 if x.dtype == torch.float32 else lib.F16
    lib.check(L.b2_argmax_rows_static(x.data_ptr(), rows, width, width, code, out.data_ptr(), stream))
    return out


def test_static_scratch_argmax_matches_workspace_argmax_twice(b2, port):
    L = b2
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(99)
    first = np.round(wl.normal(rng, (256, 40000), 4.0) * 2) / 2          # coarse grid: real ties
    second = wl.config5(rows=64)["logits"]                                 # vocabulary width, planted maxima
    third = wl.normal(rng, (3, 5000), 4.0).astype(np.float16)
    for host_x in (first, second, third):
        x = torch.from_numpy(host_x).to(DEV)
        want = _reference_ids(L, x, stream)
        got = _static_ids(L, x, stream)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        oracle_ids = port.argmax_rows(host_x if host_x.dtype == np.float32 else host_x.view(np.uint16))
        assert np.array_equal(got.cpu().numpy(), oracle_ids)


def test_static_scratch_at_its_row_limit_and_with_split_rows(b2):
    """The full 4096 rows (one thread block per row, the scratch untouched by the kernel) and the largest row
    count whose rows are still split over several thread blocks, which then meet in the scratch's keys and tickets."""
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(100)
    for rows, width in ((4096, 6000), (592, 8192), (4096, 257)):
        x = torch.from_numpy(np.round(wl.normal(rng, (rows, width), 4.0) * 4) / 4).to(DEV)
        for _ in range(2):
            got = _static_ids(b2, x, stream)
            torch.cuda.synchronize()
            assert torch.equal(got, _reference_ids(b2, x, stream))


def test_static_scratch_capacity_is_enforced(b2):
    x = torch.zeros(lib.load().b2_argmax_workspace_bytes(1), device=DEV)   # any valid pointer: never read
    out = torch.empty(1, dtype=torch.int32, device=DEV)
    rc = b2.b2_argmax_rows_static(x.data_ptr(), 4097, 8, 8, lib.F32, out.data_ptr(), None)
    assert rc == -4 and b"4097 rows exceed" in b2.b2_last_error()
    assert b2.b2_argmax_rows_static(x.data_ptr(), 2, 0, 0, lib.F32, out.data_ptr(), None) == -1
    assert b2.b2_argmax_rows_static(None, 0, 8, 8, lib.F32, None, None) == 0
