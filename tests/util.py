"""Comparison rules of the parity tests.

fp32 outputs: |got - ref| <= 1e-5 * max(|ref|, floor), `floor` being the natural scale of the
operator where a pure relative bound is meaningless (cancellation in RoPE, near-underflow softmax
entries).  fp16 outputs: within 1 fp16 ulp of the oracle's fp32 value.  Integer and copy results:
bit-exact.
"""
import numpy as np

RTOL_F32 = 1e-5


def ulp16(x):
    """Spacing of fp16 numbers at |x| (subnormal spacing 2^-24 below 2^-14)."""
    a = np.abs(np.asarray(x, dtype=np.float64))
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -14)))
    return np.exp2(e - 10)


def worst_rel(got, ref, floor=0.0):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    scale = np.maximum(np.abs(ref), floor)
    err = np.abs(got - ref)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(scale > 0, err / scale, np.where(err == 0, 0.0, np.inf))
    return float(r.max()) if r.size else 0.0


def assert_close_f32(got, ref, floor=0.0, rtol=RTOL_F32, what=""):
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all() == np.isfinite(ref).all(), f"{what}: finiteness differs"
    w = worst_rel(got, ref, floor)
    assert w <= rtol, f"{what}: worst |got-ref|/max(|ref|,floor) = {w:.3e} > {rtol:.1e}"


def assert_within_1ulp_f16(got_half, ref_f32, what="", ulps=1.0):
    """got_half: np.float16 array; ref_f32: the oracle's fp32 result."""
    got = got_half.astype(np.float64)
    ref = np.asarray(ref_f32, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    err = np.abs(got - ref) / ulp16(ref)
    assert float(err.max()) <= ulps, f"{what}: worst error {float(err.max()):.3f} fp16 ulp > {ulps}"


def f16_bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def dequant(port, a16):
    """Exact fp16 -> fp32 widening through the oracle's decoder (not numpy's)."""
    return port.decode_f16(f16_bits(a16)).reshape(a16.shape)
