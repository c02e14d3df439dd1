"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments before any CUDA call is made."""
import ctypes as C

import pytest

from cuda_llm_b200 import lib


def test_library_exports_every_declared_symbol(b2):
    names = lib.declared_symbols()
    assert len(names) >= 25 and "b2_add_rms_norm" in names and "b2_argmax_rows" in names
    for n in names:
        assert hasattr(b2, n), n
        assert n in lib._SIGNATURES, f"{n} has no ctypes signature"
    assert b2.b2_version() >= 100
    assert b2.b2_status_string(0) == b"ok" and b2.b2_status_string(-1) == b"invalid argument"


def test_missing_library_is_an_error_not_a_fallback(tmp_path):
    with pytest.raises(ImportError, match="no CPU or library fallback"):
        lib.load(str(tmp_path / "libb2ops.so"))


def test_validation_happens_before_any_launch(b2):
    """None of these reaches the CUDA runtime: every one is refused by argument checks."""
    p = C.c_void_p(16)   # never dereferenced
    bad = [
        b2.b2_rms_norm(p, p, p, 4, 8, 0.0, lib.F16, lib.FAST, None),            # eps must be > 0
        b2.b2_rms_norm(p, p, p, 4, 0, 1e-6, lib.F16, lib.FAST, None),           # hidden
        b2.b2_rms_norm(p, p, p, -1, 8, 1e-6, lib.F16, lib.FAST, None),          # rows
        b2.b2_rms_norm(p, p, p, 4, 8, 1e-6, 7, lib.FAST, None),                 # dtype
        b2.b2_rms_norm(p, p, p, 4, 8, 1e-6, lib.F16, 5, None),                  # mode
        b2.b2_rms_norm(None, p, p, 4, 8, 1e-6, lib.F16, lib.FAST, None),        # null
        b2.b2_add_rms_norm(p, p, p, p, p, 4, 8, 1e-6, lib.F16, lib.FAST, None),  # residual == normalized
        b2.b2_add(p, p, None, 4, lib.F32, None),
        b2.b2_swiglu(p, p, p, -3, lib.F32, lib.FAST, None),
        b2.b2_rope(p, p, p, 2, 1, 3, 1e4, lib.F32, lib.FAST, None, None),             # odd head_dim
        b2.b2_rope(p, p, p, 2, 1, 4, 0.0, lib.F32, lib.FAST, None, None),             # theta
        b2.b2_rope_batched(p, p, p, 2, 0, 1, 4, 1e4, lib.F32, lib.FAST, None, None),  # seq
        b2.b2_qk_norm_rope(p, None, p, None, p, p, None, 2, 16, 8, 128, 1e-6, 1e6, lib.F16, None, None),  # k missing
        b2.b2_embedding_gather(p, p, p, 4, 8, 0, lib.F16, None, None),          # vocab
        b2.b2_argmax_rows(p, 2, 8, 4, lib.F32, p, p, None),                     # stride < width
        b2.b2_argmax_keys(p, 2, 8, 8, lib.F32, 2 ** 32, p, p, None),            # index does not fit 32 bits
        b2.b2_softmax_rows(p, p, 2, 0, lib.F32, lib.FAST, p, None),
        b2.b2_softmax_stats(p, 2, 8, lib.F32, None, p, None),
    ]
    assert all(rc == -1 for rc in bad), bad
    assert b"b2_softmax_stats" in b2.b2_last_error()
    with pytest.raises(lib.InvalidArgument):
        lib.check(-1)
    # empty problems are accepted and launch nothing
    assert b2.b2_add(None, None, None, 0, lib.F32, None) == 0
    assert b2.b2_rms_norm(None, None, None, 0, 8, 1e-6, lib.F16, lib.FAST, None) == 0
    assert b2.b2_argmax_workspace_bytes(256) >= 256 * 12 and b2.b2_argmax_workspace_bytes(0) == 0
    assert b2.b2_softmax_workspace_bytes(256) >= 256 * 8
