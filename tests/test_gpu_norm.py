"""GPU parity of the RMSNorm family against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, workloads as wl
from util import assert_close_f32, assert_within_1ulp_f16, dequant, f16_bits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def host(t):
    return t.cpu().numpy()


SHAPES = [(1, 1024), (4, 1024), (64, 2048), (7, 4096), (1, 128), (96, 128), (33, 384), (5, 8192), (3, 16384),
          (2, 40000), (4, 1000), (9, 130), (3, 7)]


@pytest.mark.parametrize("rows,hidden", SHAPES)
def test_rms_norm_fast_f32(b2, port, rows, hidden):
    rng = np.random.default_rng(rows * 100003 + hidden)
    x, w = wl.normal(rng, (rows, hidden)), wl.gamma(rng, hidden)
    got = host(ops.cuda_rms_norm(dev(x), dev(w), wl.EPS))
    assert_close_f32(got, port.rms_norm(x, w, wl.EPS), what=f"rms_norm f32 {rows}x{hidden}")


@pytest.mark.parametrize("rows,hidden", SHAPES)
def test_rms_norm_fast_f16(b2, port, rows, hidden):
    rng = np.random.default_rng(rows * 100019 + hidden)
    x, w = wl.normal(rng, (rows, hidden), dtype=np.float16), wl.gamma(rng, hidden, dtype=np.float16)
    got = host(ops.cuda_rms_norm(dev(x), dev(w), wl.EPS))
    assert_within_1ulp_f16(got, port.rms_norm(dequant(port, x), dequant(port, w), wl.EPS), f"rms_norm f16 {rows}x{hidden}")


@pytest.mark.parametrize("rows,hidden", SHAPES)
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_add_rms_norm_fast(b2, port, rows, hidden, dtype):
    rng = np.random.default_rng(rows * 100043 + hidden)
    x, r = wl.normal(rng, (rows, hidden), dtype=dtype), wl.normal(rng, (rows, hidden), dtype=dtype)
    w = wl.gamma(rng, hidden, dtype=dtype)
    res, nrm = torch.empty_like(dev(x)), torch.empty_like(dev(x))
    ops.cuda_add_rms_norm_out(dev(x), dev(r), dev(w), wl.EPS, res, nrm)
    if dtype == np.float32:
        want_res, want_nrm = port.add_rms_norm(x, r, w, wl.EPS)
        assert np.array_equal(host(res), want_res)                       # one fp32 add: exact
        assert_close_f32(host(nrm), want_nrm, what="add_rms_norm f32 normalized")
    else:
        want_res, want_nrm = port.add_rms_norm(dequant(port, x), dequant(port, r), dequant(port, w), wl.EPS)
        assert np.array_equal(f16_bits(host(res)), port.f32_to_f16_rn(want_res))   # correctly rounded sum
        assert_within_1ulp_f16(host(nrm), want_nrm, "add_rms_norm f16 normalized")


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (4, 1024), (65, 2048), (3, 4096), (96, 128), (5, 1000), (2, 5000)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_deterministic_mode_is_bit_exact(b2, port, rows, hidden, dtype):
    """Deterministic mode reproduces the reference kernels' arithmetic (fp64 running sum in index
    order, src/ops_cuda.cu:84-97,118-129): bit equality with the device-order restatement."""
    rng = np.random.default_rng(rows * 100057 + hidden)
    x, r = wl.normal(rng, (rows, hidden), dtype=dtype), wl.normal(rng, (rows, hidden), dtype=dtype)
    w = wl.gamma(rng, hidden, dtype=dtype)
    raw = (lambda a: a) if dtype == np.float32 else f16_bits
    view = (lambda a: a.view(np.uint32)) if dtype == np.float32 else f16_bits
    with ops.reduction_mode("deterministic"):
        got = host(ops.cuda_rms_norm(dev(x), dev(w), wl.EPS))
        res, nrm = torch.empty_like(dev(x)), torch.empty_like(dev(x))
        ops.cuda_add_rms_norm_out(dev(x), dev(r), dev(w), wl.EPS, res, nrm)
    assert np.array_equal(view(got), view(port.dev_rms_norm(raw(x), raw(w), wl.EPS)).reshape(got.shape))
    want_res, want_nrm = port.dev_add_rms_norm(raw(x), raw(r), raw(w), wl.EPS)
    assert np.array_equal(view(host(res)), view(want_res).reshape(x.shape))
    assert np.array_equal(view(host(nrm)), view(want_nrm).reshape(x.shape))
    # and it still agrees with the CPU operator within the parity tolerance
    if dtype == np.float32:
        assert_close_f32(got, port.rms_norm(x, w, wl.EPS), what="deterministic vs ops_cpu")


def test_config1_norms_against_committed_reference_outputs(b2, port, golden):
    """Configuration 1 (fp32, 4 tokens): fused add+norm and per-head QK-norm vs the reference's own
    compiled CPU operators (tests/golden/c1_reference.npz)."""
    c, g = wl.config1(with_table=False), golden("c1_reference")
    res, nrm = torch.empty(4, 1024, device=DEV), torch.empty(4, 1024, device=DEV)
    ops.cuda_add_rms_norm_out(dev(c["x"]), dev(c["res"]), dev(c["gamma"]), wl.EPS, res, nrm)
    assert np.array_equal(host(res), g["residual"])
    assert_close_f32(host(nrm), g["normalized"], what="c1 normalized")
    assert_close_f32(host(ops.cuda_rms_norm(dev(c["q"]), dev(c["gamma_q"]), wl.EPS)), g["q_norm"], what="c1 q_norm")
    assert_close_f32(host(ops.cuda_rms_norm(dev(c["k"]), dev(c["gamma_k"]), wl.EPS)), g["k_norm"], what="c1 k_norm")


def test_layer0_fixture_norms(b2, golden):
    """The reference's exported layer-0 activations, with its own tolerances
    (tests/test_qwen3_layer_cuda.cpp:92-95: 1e-4, 5e-4 for the k nodes)."""
    g = golden("layer0")
    eps = float(g["rms_norm_eps"])
    got = host(ops.cuda_rms_norm(dev(g["hidden_states"]), dev(g["input_layernorm_weight"]), eps))
    assert np.abs(got - g["input_norm"]).max() <= 1e-4
    q = host(ops.cuda_rms_norm(dev(g["q_linear"].reshape(4, 16, 128)), dev(g["q_norm_weight"]), eps))
    k = host(ops.cuda_rms_norm(dev(g["k_linear"].reshape(4, 8, 128)), dev(g["k_norm_weight"]), eps))
    assert np.abs(q - g["q_norm_output"]).max() <= 1e-4 and np.abs(k - g["k_norm_output"]).max() <= 5e-4
    res, nrm = torch.empty(4, 1024, device=DEV), torch.empty(4, 1024, device=DEV)
    ops.cuda_add_rms_norm_out(dev(g["hidden_states"]), dev(g["o_proj_output"]),
                              dev(g["post_attention_layernorm_weight"]), eps, res, nrm)
    assert np.abs(host(res) - g["attention_residual"]).max() <= 1e-4
    assert np.abs(host(nrm) - g["post_attention_norm"]).max() <= 1e-4


def test_reference_cuda_test_literals(b2, port):
    """Inputs of reference tests/test_ops_cuda.cpp:111-125 with its tolerances (1e-4 / 5e-3)."""
    x = np.array([[1, -2, 3, 0], [.5, 2, -1, 4], [-3, 1, 2, -.5]], np.float32)
    w = np.array([1, .5, 2, -1], np.float32)
    assert np.abs(host(ops.cuda_rms_norm(dev(x), dev(w), 1e-5)) - port.rms_norm(x, w, 1e-5)).max() <= 1e-4
    x16, w16 = x.astype(np.float16), w.astype(np.float16)
    got = host(ops.cuda_rms_norm(dev(x16), dev(w16), 1e-5)).astype(np.float32)
    assert np.abs(got - port.rms_norm(x16.astype(np.float32), w16.astype(np.float32), 1e-5)).max() <= 5e-3


def test_in_place_views_and_guard_bands(b2, port):
    """In-place use (output aliases input, src/qwen3_layer_cuda.cu:703), views with a byte offset that
    is only element-aligned (Tensor::slice_first_dim), and sentinel pads around every output."""
    rng = np.random.default_rng(77)
    rows, hidden, pad = 6, 1024, 64
    x16 = wl.normal(rng, (rows, hidden), dtype=np.float16)
    w16 = wl.gamma(rng, hidden, dtype=np.float16)
    want = port.rms_norm(dequant(port, x16), dequant(port, w16), wl.EPS)
    buf = torch.full((pad + rows * hidden + pad,), 7.0, dtype=torch.float16, device=DEV)
    body = buf[pad:pad + rows * hidden].view(rows, hidden)
    body.copy_(dev(x16))
    ops.cuda_rms_norm_out(body, dev(w16), wl.EPS, body)                 # in place, 16-byte aligned view
    assert_within_1ulp_f16(host(body), want, "in-place rms_norm")
    assert (host(buf[:pad]) == 7).all() and (host(buf[-pad:]) == 7).all()
    # a view that starts 2 bytes past a 16-byte boundary takes the scalar path
    buf2 = torch.full((pad + 1 + rows * hidden + pad,), 7.0, dtype=torch.float16, device=DEV)
    odd = buf2[pad + 1:pad + 1 + rows * hidden].view(rows, hidden)
    odd.copy_(dev(x16))
    out = torch.full((pad + 1 + rows * hidden + pad,), 9.0, dtype=torch.float16, device=DEV)
    odd_out = out[pad + 1:pad + 1 + rows * hidden].view(rows, hidden)
    ops.cuda_rms_norm_out(odd, dev(w16), wl.EPS, odd_out)
    assert_within_1ulp_f16(host(odd_out), want, "misaligned rms_norm")
    assert (host(out[:pad + 1]) == 9).all() and (host(out[-pad:]) == 9).all()
    # fused form with the residual written over lhs
    r16 = wl.normal(rng, (rows, hidden), dtype=np.float16)
    lhs, nrm = dev(x16), torch.empty(rows, hidden, dtype=torch.float16, device=DEV)
    ops.cuda_add_rms_norm_out(lhs, dev(r16), dev(w16), wl.EPS, lhs, nrm)
    want_res, want_nrm = port.add_rms_norm(dequant(port, x16), dequant(port, r16), dequant(port, w16), wl.EPS)
    assert np.array_equal(f16_bits(host(lhs)), port.f32_to_f16_rn(want_res))
    assert_within_1ulp_f16(host(nrm), want_nrm, "fused, residual over lhs")


def test_rejections(b2):
    """Argument rules of the reference wrappers (src/ops_cuda.cu:672,675-690; tests/test_ops_cuda.cpp:197;
    tests/test_embedding_lm_head_cuda.cpp:24)."""
    x, w = torch.zeros(3, 4, device=DEV), torch.ones(4, device=DEV)
    with pytest.raises(ValueError):
        ops.cuda_rms_norm(x, w.half(), 1e-5)                 # dtype mismatch
    with pytest.raises(ValueError):
        ops.cuda_rms_norm(x, torch.ones(5, device=DEV), 1e-5)  # shape
    with pytest.raises(ValueError):
        ops.cuda_rms_norm(x, w, 0.0)                         # epsilon must be > 0 on the CUDA path
    with pytest.raises(ValueError):
        ops.cuda_rms_norm(x.cpu(), w, 1e-5)                  # CPU input
    with pytest.raises(ValueError):
        ops.cuda_rms_norm(x.to(torch.bfloat16), w.to(torch.bfloat16), 1e-5)
    with pytest.raises(ValueError):
        ops.cuda_add_rms_norm_out(x, x, w, 1e-5, torch.empty(3, 5, device=DEV), torch.empty_like(x))


def test_run_to_run_bit_identity(b2):
    rng = np.random.default_rng(5)
    x, w = dev(wl.normal(rng, (512, 4096), dtype=np.float16)), dev(wl.gamma(rng, 4096, dtype=np.float16))
    first = ops.cuda_rms_norm(x, w, wl.EPS)
    for _ in range(3):
        assert torch.equal(first, ops.cuda_rms_norm(x, w, wl.EPS))


def test_config2_sweep_sampled_rows(b2, port):
    """Configuration 2 at full size on the GPU; the oracle checks the first and last 64 rows and
    256 random rows of each shape (rows are independent)."""
    for rows in wl.C2_ROWS:
        for hidden in wl.C2_HIDDEN:
            c = wl.config2(rows, hidden)
            x, r, w = dev(c["x"]), dev(c["res"]), dev(c["gamma"])
            res, nrm = torch.empty_like(x), torch.empty_like(x)
            ops.cuda_add_rms_norm_out(x, r, w, wl.EPS, res, nrm)
            rng = np.random.default_rng(rows + hidden)
            pick = np.unique(np.concatenate([np.arange(min(rows, 64)), np.arange(max(0, rows - 64), rows),
                                             rng.integers(0, rows, min(rows, 256))]))
            want_res, want_nrm = port.add_rms_norm(dequant(port, c["x"][pick]), dequant(port, c["res"][pick]),
                                                   dequant(port, c["gamma"]), wl.EPS)
            idx = torch.from_numpy(pick).to(DEV)
            assert np.array_equal(f16_bits(host(res[idx])), port.f32_to_f16_rn(want_res)), (rows, hidden)
            assert_within_1ulp_f16(host(nrm[idx]), want_nrm, f"c2 {rows}x{hidden}")


def test_host_buffer_pipeline_matches_oracle(b2, port):
    """Host buffers in, host buffers out, in overlapped row chunks: same results as one device call."""
    from cuda_llm_b200 import hostio
    rows, hidden = 1000, 2048
    c = wl.config2(4096, 2048)
    hx, hr = (torch.from_numpy(c[k][:rows]).pin_memory() for k in ("x", "res"))
    h_res, h_nrm = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
    pipe = hostio.AddRmsNormHostPipeline(rows, hidden, DEV, chunks=7)
    for _ in range(2):                                      # the second call reuses buffers of the first
        pipe(hx, hr, dev(c["gamma"]), h_res, h_nrm, wl.EPS).synchronize()
    want_res, want_nrm = port.add_rms_norm(dequant(port, c["x"][:rows]), dequant(port, c["res"][:rows]),
                                           dequant(port, c["gamma"]), wl.EPS)
    assert np.array_equal(f16_bits(h_res.numpy()), port.f32_to_f16_rn(want_res))
    assert_within_1ulp_f16(h_nrm.numpy(), want_nrm, "host pipeline")
