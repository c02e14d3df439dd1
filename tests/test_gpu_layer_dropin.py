"""Layer-level drop-in proof: the reference's OWN decoder-layer code (src/qwen3_layer_cuda.cu,
compiled unmodified) run twice on the same inputs -- linked with the reference's operators, and
with RMSNorm, RoPE, add and SwiGLU replaced by this repository's namespace-llm functions (which
were compiled against the reference's headers; cuda_linear and attention stay the reference's).
All 17 trace nodes are compared with the thresholds of the reference's own layer tests
(tests/test_qwen3_layer_cuda.cpp:92-131 for F32, tests/test_qwen3_layer_cuda_fp16.cpp:53-58 for F16).
Weights are seeded synthetic draws of the Qwen3-0.6B layer shapes: the model package is not
available, and both sides get identical bits."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
EPS, THETA = 1e-6, 1e6


@pytest.fixture(scope="module")
def libs(b2):
    pair = oracle.layer_libs()
    if pair is None:
        pytest.skip("oracle/_ref/liblayer_*.so not built (needs the reference tree at build time)")
    ref, dropin = pair
    assert not ref.replaced and dropin.replaced
    return ref, dropin


def make_inputs(seq, seed):
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in oracle.LAYER_WEIGHTS:
        if len(shape) == 1:
            w[name] = (rng.random(shape, dtype=np.float32) + 0.5).astype(np.float32)     # norm weights ~U(0.5, 1.5)
        else:
            w[name] = (rng.standard_normal(shape, dtype=np.float32) * 0.02).astype(np.float32)
    hidden = rng.standard_normal((seq, 1024), dtype=np.float32)
    return hidden, np.arange(seq, dtype=np.int32), w


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


@pytest.mark.parametrize("seq", [4, 32])
def test_f32_layer_trace_with_replaced_operators(libs, seq):
    ref, dropin = libs
    hidden, pos, w = make_inputs(seq, 100 + seq)
    want = ref.trace(hidden, pos, w, EPS, THETA, half=False)
    dropin.select_reductions(False)
    got = dropin.trace(hidden, pos, w, EPS, THETA, half=False)
    for name in oracle.LAYER_NODES:
        tol = 5e-4 if name in ("k_norm_output", "k_rope") else 1e-4
        err = float(np.abs(got[name] - want[name]).max())
        assert err <= tol and cosine(got[name], want[name]) >= 0.99999, f"{name}: max abs error {err:.3e}"
    # deterministic reductions reproduce the reference's kernels exactly where the arithmetic is IEEE-exact:
    # every node up to and including the per-head norms is bit-identical
    dropin.select_reductions(True)
    exact = dropin.trace(hidden, pos, w, EPS, THETA, half=False)
    dropin.select_reductions(False)
    for name in ("input_norm", "q_linear", "k_linear", "v_linear", "q_norm_output", "k_norm_output"):
        assert np.array_equal(exact[name].view(np.uint32), want[name].view(np.uint32)), name
    for name in oracle.LAYER_NODES:
        assert float(np.abs(exact[name] - want[name]).max()) <= 2e-6, name


def test_f16_layer_trace_with_replaced_operators(libs):
    ref, dropin = libs
    hidden, pos, w = make_inputs(8, 7)
    want = ref.trace(hidden, pos, w, EPS, THETA, half=True)
    got = dropin.trace(hidden, pos, w, EPS, THETA, half=True)
    for name in oracle.LAYER_NODES:
        floor = 1e-2 if name in ("k_norm_output", "k_rope") else 5e-3
        tol = np.maximum(floor, 1e-3 * np.abs(want[name]))
        assert bool((np.abs(got[name] - want[name]) <= tol).all()), f"{name}: {float(np.abs(got[name] - want[name]).max()):.3e}"
        assert cosine(got[name], want[name]) >= 0.9999, name


def test_the_reference_layer_still_rejects_what_it_rejected(libs):
    """Argument errors of the layer code and of the replaced operators surface as exceptions, as before."""
    _, dropin = libs
    hidden, pos, w = make_inputs(4, 1)
    with pytest.raises(RuntimeError):
        dropin.trace(hidden, pos, w, 0.0, THETA, half=False)        # non-positive epsilon
    with pytest.raises(RuntimeError):
        dropin.trace(hidden, pos, w, EPS, 0.0, half=False)          # non-positive rope theta
