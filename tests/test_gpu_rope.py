"""GPU parity of rotary embedding (all entry points) and the fused QK-norm + RoPE, through the C ABI."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, workloads as wl
from util import assert_close_f32, assert_within_1ulp_f16, dequant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()


def pair_scale(x):
    """max(|a|, |b|) of the rotated pair behind every output element: a*c - b*s cancels, so a bound
    relative to the output alone is meaningless."""
    half = x.shape[-1] // 2
    m = np.maximum(np.abs(x[..., :half]), np.abs(x[..., half:]))
    return np.concatenate([m, m], axis=-1)


def close_rope_f32(got, want, x, what):
    err = np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), pair_scale(x))
    assert float(err.max()) <= 1e-5, f"{what}: worst scaled error {float(err.max()):.3e}"


CASES = [(4, 16, 128, 1e6), (4, 8, 128, 1e6), (2, 1, 4, 1e4), (33, 3, 64, 1e4), (17, 5, 256, 1e6), (9, 2, 6, 1e4),
         (5, 4, 512, 5e5), (600, 24, 128, 1e6)]


@pytest.mark.parametrize("tokens,heads,dim,theta", CASES)
@pytest.mark.parametrize("mode", ["fast", "deterministic"])
def test_rope_f32(b2, port, tokens, heads, dim, theta, mode):
    rng = np.random.default_rng(tokens * 31 + dim)
    x = wl.normal(rng, (tokens, heads, dim))
    pos = rng.integers(0, 4096, tokens).astype(np.int32)
    pos[0] = 0
    got = host(ops.cuda_rope(dev(x), pos.tolist(), theta, mode))
    want = port.rope(x, pos, theta)
    if mode == "fast":
        close_rope_f32(got, want, x, f"rope f32 {tokens}x{heads}x{dim}")
    else:
        # the reference kernel's all-fp32 angle (src/ops_cuda.cu:133) loses ~pos*2^-24 rad: its own test
        # bound is 1e-4 absolute at unit scale (tests/test_ops_cuda.cpp:136-137)
        assert np.abs(got - want).max() <= 1e-4 * max(1.0, pos.max() / 64) * np.abs(x).max()


@pytest.mark.parametrize("tokens,heads,dim,theta", CASES)
@pytest.mark.parametrize("mode", ["fast", "deterministic"])
def test_rope_f16(b2, port, tokens, heads, dim, theta, mode):
    rng = np.random.default_rng(tokens * 37 + dim)
    x = wl.normal(rng, (tokens, heads, dim), dtype=np.float16)
    pos = rng.integers(0, 512, tokens).astype(np.int32)
    got = host(ops.cuda_rope(dev(x), pos.tolist(), theta, mode))
    want = port.rope(dequant(port, x), pos, theta)
    if mode == "fast":
        # 1 fp16 ulp of the output, or of the larger input of the pair where the output cancelled
        err = np.abs(got.astype(np.float64) - want)
        from util import ulp16
        assert float((err / ulp16(np.maximum(np.abs(want), pair_scale(dequant(port, x))))).max()) <= 1.0
    else:
        assert np.abs(got.astype(np.float32) - want).max() <= 5e-3 * max(1.0, np.abs(want).max())


def test_rope_large_positions_fast_mode(b2, port):
    """fp64 angle + fp64 range reduction: accurate at any int32 position."""
    rng = np.random.default_rng(9)
    x = wl.normal(rng, (6, 2, 128))
    pos = np.array([0, 1, 40000, 1 << 20, (1 << 30) + 12345, 2 ** 31 - 1], np.int32)
    got = host(ops.cuda_rope(dev(x), pos.tolist(), 1e6))
    close_rope_f32(got, port.rope(x, pos, 1e6), x, "rope large positions")


def test_reference_cuda_test_literals(b2, port):
    """reference tests/test_ops_cuda.cpp:134-140,204-205."""
    x = np.array([1, 2, 3, 4, 2, -1, .5, 3], np.float32).reshape(2, 1, 4)
    assert np.abs(host(ops.cuda_rope(dev(x), [0, 1], 10000.0)) - port.rope(x, [0, 1], 10000.0)).max() <= 1e-4
    x16 = x.astype(np.float16)
    got = host(ops.cuda_rope(dev(x16), [0, 1], 10000.0)).astype(np.float32)
    assert np.abs(got - port.rope(x16.astype(np.float32), [0, 1], 10000.0)).max() <= 5e-3
    with pytest.raises(ValueError):
        ops.cuda_rope(dev(x), [0, 1], 0.0)              # theta
    with pytest.raises(ValueError):
        ops.cuda_rope(dev(x), [0], 10000.0)             # positions length
    with pytest.raises(ValueError):
        ops.cuda_rope(dev(x.reshape(2, 4)), [0, 1], 10000.0)
    for _ in range(100):                                 # allocation loop of the reference test (:206)
        ops.cuda_rope(dev(x), [0, 1], 10000.0)
    torch.cuda.synchronize()


def test_batched_and_token_position_entry_points_agree(b2, port):
    """cuda_rope_batched / _out share positions over the batch; *_positions_out take one position per row.
    No direct reference test exists for them: they are pinned by equality with cuda_rope on the same
    numbers and by the oracle."""
    rng = np.random.default_rng(12)
    b, s, h, d = 3, 5, 16, 128
    x = wl.normal(rng, (b, s, h, d), dtype=np.float16)
    pos = rng.integers(0, 300, s).astype(np.int32)
    got = host(ops.cuda_rope_batched(dev(x), pos.tolist(), 1e6))
    want = np.stack([port.rope(dequant(port, x[i]), pos, 1e6) for i in range(b)])
    from util import ulp16
    err = np.abs(got.astype(np.float64) - want) / ulp16(np.maximum(np.abs(want), pair_scale(dequant(port, x))))
    assert float(err.max()) <= 1.0
    flat = host(ops.cuda_rope(dev(x.reshape(b * s, h, d)), np.tile(pos, b).tolist(), 1e6)).reshape(x.shape)
    assert np.array_equal(got.view(np.uint16), flat.view(np.uint16))
    out = torch.empty_like(dev(x))
    # positions buffer typed F32 holding int32 bits, larger than S (include/llm/qwen3_decode_workspace.h:85-90)
    pos_buf = torch.zeros(8, dtype=torch.float32, device=DEV)
    pos_buf.view(torch.int32)[:s] = dev(pos)
    ops.cuda_rope_batched_out(dev(x), pos_buf, 1e6, out)
    assert np.array_equal(host(out).view(np.uint16), got.view(np.uint16))
    rows = b * s
    out2 = torch.empty(rows, h, d, dtype=torch.float16, device=DEV)
    ops.cuda_rope_token_positions_out(dev(x.reshape(rows, h, d)), dev(np.tile(pos, b)), 1e6, out2)
    assert np.array_equal(host(out2).view(np.uint16).ravel(), got.view(np.uint16).ravel())
    q = dev(x.reshape(rows, h, d))
    ops.cuda_rope_batched_positions_out(q, dev(np.tile(pos, b)), 1e6, q)           # in place (:800-801)
    assert np.array_equal(host(q).view(np.uint16).ravel(), got.view(np.uint16).ravel())
    with pytest.raises(ValueError):
        ops.cuda_rope_token_positions_out(dev(x.reshape(rows, h, d)), dev(pos), 1e6, out2)   # positions shape


def test_layer0_and_config1_fixtures(b2, golden):
    g = golden("layer0")
    theta, pos = float(g["rope_theta"]), g["position_ids"].astype(np.int32).tolist()
    assert np.abs(host(ops.cuda_rope(dev(g["q_norm_output"]), pos, theta)) - g["q_rope"]).max() <= 1e-4
    assert np.abs(host(ops.cuda_rope(dev(g["k_norm_output"]), pos, theta)) - g["k_rope"]).max() <= 5e-4
    c, r = wl.config1(with_table=False), golden("c1_reference")
    close_rope_f32(host(ops.cuda_rope(dev(r["q_norm"]), c["positions"].tolist(), wl.THETA)), r["q_rope"], r["q_norm"], "c1 q_rope")
    close_rope_f32(host(ops.cuda_rope(dev(r["k_norm"]), c["positions"].tolist(), wl.THETA)), r["k_rope"], r["k_norm"], "c1 k_rope")


def _fused(q, k, gq, gk, pos, dtype_t):
    qo, ko = torch.empty_like(dev(q)), torch.empty_like(dev(k))
    ops.qk_norm_rope_out(dev(q), dev(k), dev(gq), dev(gk), dev(pos), wl.EPS, wl.THETA, qo, ko)
    return host(qo), host(ko)


def test_fused_qk_norm_rope_f32_config1(b2, port, golden):
    c, r = wl.config1(with_table=False), golden("c1_reference")
    qo, ko = _fused(c["q"], c["k"], c["gamma_q"], c["gamma_k"], c["positions"], torch.float32)
    close_rope_f32(qo, r["q_rope"], r["q_norm"], "fused q")
    close_rope_f32(ko, r["k_rope"], r["k_norm"], "fused k")
    g = golden("layer0")
    qo, ko = _fused(g["q_linear"].reshape(4, 16, 128), g["k_linear"].reshape(4, 8, 128), g["q_norm_weight"],
                    g["k_norm_weight"], g["position_ids"].astype(np.int32), torch.float32)
    assert np.abs(qo - g["q_rope"]).max() <= 1e-4 and np.abs(ko - g["k_rope"]).max() <= 5e-4


@pytest.mark.parametrize("tokens", [64, 16384])
def test_fused_qk_norm_rope_f16_config3(b2, port, golden, tokens):
    """Configuration 3: packed prefill, positions restart at 0 per sequence.  The fused kernel keeps the
    normalised value in fp32, so it is compared with the fp32 oracle chain rms_norm -> rope at 1 fp16 ulp;
    the reference-shaped unfused calls round to fp16 between the two steps and get 2 ulp."""
    from util import ulp16
    c = wl.config3(tokens=tokens)
    qo, ko = _fused(c["q"], c["k"], c["gamma_q"], c["gamma_k"], c["positions"], torch.float16)
    if tokens == 64:
        s = golden("small_reference")
        want_q, want_k = s["c3_q"], s["c3_k"]
        pick = slice(None)
    else:
        rng = np.random.default_rng(1)
        pick = np.unique(np.r_[0:32, tokens - 32:tokens, rng.integers(0, tokens, 192)])
        chain = lambda x, gm: port.rope(port.rms_norm(dequant(port, x[pick]).reshape(-1, 128), dequant(port, gm),
                                                      wl.EPS).reshape(-1, x.shape[1], 128), c["positions"][pick], wl.THETA)
        want_q, want_k = chain(c["q"], c["gamma_q"]), chain(c["k"], c["gamma_k"])
    for got, want, x, gm in ((qo[pick], want_q, c["q"], c["gamma_q"]), (ko[pick], want_k, c["k"], c["gamma_k"])):
        nrm = port.rms_norm(dequant(port, x[pick]).reshape(-1, 128), dequant(port, gm), wl.EPS).reshape(want.shape)
        err = np.abs(got.astype(np.float64) - want) / ulp16(np.maximum(np.abs(want), pair_scale(nrm)))
        assert float(err.max()) <= 1.0, f"fused c3 worst {float(err.max()):.3f} ulp"
    # reference-shaped sequence of four calls on the same inputs
    qn, kn = ops.cuda_rms_norm(dev(c["q"]), dev(c["gamma_q"]), wl.EPS), ops.cuda_rms_norm(dev(c["k"]), dev(c["gamma_k"]), wl.EPS)
    pos = dev(c["positions"])
    ops.cuda_rope_token_positions_out(qn, pos, wl.THETA, qn)
    ops.cuda_rope_token_positions_out(kn, pos, wl.THETA, kn)
    for got, want, x, gm in ((host(qn)[pick], want_q, c["q"], c["gamma_q"]), (host(kn)[pick], want_k, c["k"], c["gamma_k"])):
        nrm = port.rms_norm(dequant(port, x[pick]).reshape(-1, 128), dequant(port, gm), wl.EPS).reshape(want.shape)
        err = np.abs(got.astype(np.float64) - want) / ulp16(np.maximum(np.abs(want), pair_scale(nrm)))
        assert float(err.max()) <= 2.0


def test_fused_scalar_fallback_and_q_only(b2, port):
    rng = np.random.default_rng(4)
    q, gq = wl.normal(rng, (7, 3, 6)), wl.gamma(rng, 6)          # head_dim 6: no vector path
    pos = rng.integers(0, 100, 7).astype(np.int32)
    qo = torch.empty_like(dev(q))
    ops.qk_norm_rope_out(dev(q), None, dev(gq), None, dev(pos), wl.EPS, 1e4, qo, None)
    nrm = port.rms_norm(q.reshape(-1, 6), gq, wl.EPS).reshape(q.shape)
    close_rope_f32(host(qo), port.rope(nrm, pos, 1e4), nrm, "fused scalar")


def test_no_bulk_copy_wait_ran_out(b2):
    """The bulk-copy kernels bound every wait; a healthy run never exhausts one (runs after the tests above)."""
    import ctypes
    n = ctypes.c_uint32(12345)
    assert b2.b2_bulk_copy_timeouts(ctypes.byref(n)) == 0 and n.value == 0
    assert ops.rope_status(DEV) == 0          # the status word every call above was given says the same


def test_status_argument_is_optional_and_left_alone_by_a_healthy_call(b2):
    from cuda_llm_b200 import lib
    c = wl.config3(tokens=512)
    q, k = dev(c["q"]), dev(c["k"])
    gq, gk, pos = dev(c["gamma_q"]), dev(c["gamma_k"]), dev(c["positions"])
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    s = torch.cuda.current_stream().cuda_stream
    status = torch.full((1,), 8, dtype=torch.int32, device=DEV)     # an unrelated bit that must survive
    for st in (None, status.data_ptr()):
        lib.check(b2.b2_qk_norm_rope(q.data_ptr(), k.data_ptr(), gq.data_ptr(), gk.data_ptr(), pos.data_ptr(), qo.data_ptr(),
                                     ko.data_ptr(), 512, 16, 8, 128, wl.EPS, wl.THETA, lib.F16, st, s))
        lib.check(b2.b2_rope(q.data_ptr(), pos.data_ptr(), qo.data_ptr(), 512, 16, 128, wl.THETA, lib.F16, lib.FAST, st, s))
        lib.check(b2.b2_rope_batched(q.data_ptr(), pos.data_ptr(), qo.data_ptr(), 2, 256, 16, 128, wl.THETA, lib.F16, lib.FAST, st, s))
    torch.cuda.synchronize()
    assert int(status.item()) == 8
