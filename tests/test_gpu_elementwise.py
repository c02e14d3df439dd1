"""GPU parity of add, SwiGLU and the embedding gather against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, workloads as wl
from util import assert_close_f32, assert_within_1ulp_f16, dequant, f16_bits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()

COUNTS = [1, 7, 8, 1023, 4096, 12288, 100003, 4 * 3072, 1 << 20]


@pytest.mark.parametrize("n", COUNTS)
def test_add(b2, port, n):
    rng = np.random.default_rng(n)
    a, b = wl.normal(rng, n), wl.normal(rng, n)
    assert np.array_equal(host(ops.cuda_add(dev(a), dev(b))), port.add(a, b))            # fp32: exact
    a16, b16 = a.astype(np.float16), b.astype(np.float16)
    got = host(ops.cuda_add(dev(a16), dev(b16)))
    assert np.array_equal(f16_bits(got), port.dev_add(f16_bits(a16), f16_bits(b16)))     # one rounding: exact


@pytest.mark.parametrize("n", COUNTS)
@pytest.mark.parametrize("mode", ["fast", "deterministic"])
def test_swiglu(b2, port, n, mode):
    rng = np.random.default_rng(n + 1)
    g, u = wl.normal(rng, n, 2.0), wl.normal(rng, n, 2.0)
    assert_close_f32(host(ops.cuda_swiglu(dev(g), dev(u), mode)), port.swiglu(g, u), what=f"swiglu f32 {mode}")
    g16, u16 = g.astype(np.float16), u.astype(np.float16)
    got = host(ops.cuda_swiglu(dev(g16), dev(u16), mode))
    assert_within_1ulp_f16(got, port.swiglu(dequant(port, g16), dequant(port, u16)), f"swiglu f16 {mode}")


def test_swiglu_extremes_and_in_place(b2, port):
    g = np.array([-100, -88, -30, -10, -1e-3, 0, 1e-3, 10, 30, 88, 100, -65504, 65504], np.float32)
    u = np.linspace(-3, 3, g.size).astype(np.float32)
    assert_close_f32(host(ops.cuda_swiglu(dev(g), dev(u))), port.swiglu(g, u), floor=1e-30, what="swiglu extremes")
    g16, u16 = g.astype(np.float16), u.astype(np.float16)
    for mode in ("fast", "deterministic"):
        gate = dev(g16)
        ops.cuda_swiglu_out(gate, dev(u16), gate, mode)          # output aliases gate (src/qwen3_layer_cuda.cu:323)
        want = port.swiglu(dequant(port, g16), dequant(port, u16))
        finite = np.isfinite(want) & (np.abs(want) < 65504)
        assert_within_1ulp_f16(host(gate)[finite], want[finite], f"swiglu in place {mode}")


def test_misaligned_elementwise(b2, port):
    rng = np.random.default_rng(3)
    n = 5000
    a, b = wl.normal(rng, n + 3, dtype=np.float16), wl.normal(rng, n + 3, dtype=np.float16)
    da, db = dev(a), dev(b)
    out = torch.full((n + 3,), 5.0, dtype=torch.float16, device=DEV)
    ops.cuda_add_out(da[1:1 + n], db[1:1 + n], out[1:1 + n])
    assert np.array_equal(f16_bits(host(out[1:1 + n])), port.dev_add(f16_bits(a[1:1 + n]), f16_bits(b[1:1 + n])))
    assert host(out[0]) == 5 and (host(out[1 + n:]) == 5).all()


def test_layer0_and_config1_fixtures(b2, golden):
    g = golden("layer0")
    got = host(ops.cuda_swiglu(dev(g["gate_proj_output"]), dev(g["up_proj_output"])))
    assert np.abs(got - g["swiglu_output"]).max() <= 1e-4
    got = host(ops.cuda_add(dev(g["attention_residual"]), dev(g["down_proj_output"])))
    assert np.abs(got - g["layer_output"]).max() <= 1e-4
    c, r = wl.config1(with_table=False), golden("c1_reference")
    assert_close_f32(host(ops.cuda_swiglu(dev(c["gate"]), dev(c["up"]))), r["swiglu"], what="c1 swiglu")


def test_reference_cuda_test_literals(b2, port):
    """reference tests/test_ops_cuda.cpp:127-132."""
    x = np.array([[1, -2, 3, 0], [.5, 2, -1, 4], [-3, 1, 2, -.5]], np.float32)
    assert np.abs(host(ops.cuda_add(dev(x), dev(x))) - port.add(x, x)).max() <= 1e-4
    assert np.abs(host(ops.cuda_swiglu(dev(x), dev(x))) - port.swiglu(x, x)).max() <= 1e-4
    x16 = x.astype(np.float16)
    assert np.abs(host(ops.cuda_swiglu(dev(x16), dev(x16))).astype(np.float32)
                  - port.swiglu(x16.astype(np.float32), x16.astype(np.float32))).max() <= 5e-3
    with pytest.raises(ValueError):
        ops.cuda_add(dev(x), dev(x16))
    with pytest.raises(ValueError):
        ops.cuda_swiglu(dev(x), dev(x[:2]))


# ---- embedding gather ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("vocab,hidden,count", [(7, 4, 4), (1000, 1024, 513), (5000, 4096, 2048), (300, 130, 77),
                                                (64, 7, 33)])
def test_gather_bit_exact(b2, port, dtype, vocab, hidden, count):
    rng = np.random.default_rng(vocab + hidden)
    table = wl.normal(rng, (vocab, hidden), 0.02, dtype)
    ids = rng.integers(0, vocab, count).astype(np.int32)
    got = host(ops.cuda_embedding_lookup(dev(table), ids.tolist()))
    assert np.array_equal(got.view(np.uint8), table[ids].view(np.uint8))
    if dtype == np.float32:
        assert np.array_equal(got, port.embedding_lookup(table, ids))
    out = torch.empty(count, hidden, dtype=torch.from_numpy(table).dtype, device=DEV)
    ops.cuda_embedding_lookup_device_ids_out(dev(table), dev(ids), out)
    assert np.array_equal(host(out).view(np.uint8), table[ids].view(np.uint8))


def test_gather_reference_test_cases(b2, port):
    """reference tests/test_embedding_lm_head_cuda.cpp:19-24: literal table, exact f32, rejections."""
    ew = np.array([.01, .02, .03, .04, .10, .20, .30, .40, -.10, -.20, -.30, -.40, .50, .60, .70, .80, -.50, -.60,
                   -.70, -.80, .90, .80, .70, .60, -.90, -.80, -.70, -.60], np.float32).reshape(7, 4)
    ids = [0, 3, 6, 2]
    assert np.array_equal(host(ops.cuda_embedding_lookup(dev(ew), ids)), port.embedding_lookup(ew, ids))
    for bad in ([-1], [7], []):
        with pytest.raises(ValueError):
            ops.cuda_embedding_lookup(dev(ew), bad)
    with pytest.raises(ValueError):
        ops.cuda_embedding_lookup(torch.from_numpy(ew), ids)                 # CPU weight
    with pytest.raises(ValueError):
        ops.cuda_embedding_lookup(dev(ew).reshape(7, 4, 1), ids)             # rank


def test_gather_out_of_range_ids_never_touch_memory(b2):
    table = dev(np.arange(40, dtype=np.float32).reshape(10, 4) + 1)
    ids = dev(np.array([3, -1, 10, 9, 2 ** 31 - 1, -2 ** 31], np.int32))
    out = torch.full((6, 4), 123.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.cuda_embedding_lookup_device_ids_out(table, ids, out, status)
    got = host(out)
    assert (got[0] == host(table)[3]).all() and (got[3] == host(table)[9]).all()
    assert (got[[1, 2, 4, 5]] == 0).all() and int(status.item()) == 1
    status.zero_()
    ops.cuda_embedding_lookup_device_ids_out(table, dev(np.array([0, 9], np.int32)), out[:2], status)
    assert int(status.item()) == 0


def test_config1_gather_from_full_table(b2, golden):
    c, r = wl.config1(), golden("c1_reference")
    got = host(ops.cuda_embedding_lookup(dev(c["table"]), c["ids"].tolist()))
    assert np.array_equal(got, r["gather"])


def test_config4_shapes_sampled(b2, port):
    """Configuration 4 at reduced token count (the full T=262144 runs in the bench): fp16 SwiGLU rows
    against the oracle, and a full-table gather round trip (gather, then compare checksums of bytes)."""
    c = wl.config4_swiglu(2048, 12288)
    got = host(ops.cuda_swiglu(dev(c["gate"]), dev(c["up"])))
    pick = np.r_[0:32, 2016:2048]
    assert_within_1ulp_f16(got[pick], port.swiglu(dequant(port, c["gate"][pick]), dequant(port, c["up"][pick])), "c4 swiglu")
    g = wl.config4_gather(8192, hidden=4096, vocab=20000)
    out = host(ops.cuda_embedding_lookup(dev(g["table"]), g["ids"].tolist()))
    assert np.array_equal(out.view(np.uint16), g["table"][g["ids"]].view(np.uint16))
