"""Configurations 2-5 at their full benchmark sizes, checked through properties that do not need the
CPU oracle to finish millions of rows: exact identities (a gather is a copy, an fp32->fp16 add has one
rounding, SwiGLU is linear in `up`), invariants (softmax rows sum to 1, the planted maximum wins) and
agreement between independent code paths of the library (fast vs deterministic mode, fused vs unfused).
The oracle itself checks sampled rows of the same tensors in the per-operator test files."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _randn(*shape, sigma=1.0, dtype=torch.float16, seed=0):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * sigma).to(dtype)


def test_config2_largest_shape_fast_and_deterministic_agree():
    rows, hidden = 65536, 4096
    x, r = _randn(rows, hidden, seed=1), _randn(rows, hidden, seed=2)
    gamma = (torch.rand(hidden, device=DEV) + 0.5).half()
    res, nrm = torch.empty_like(x), torch.empty_like(x)
    ops.cuda_add_rms_norm_out(x, r, gamma, wl.EPS, res, nrm)
    assert torch.equal(res, (x.float() + r.float()).half())             # one rounding of an exact fp32 sum
    # every normalised row has unit RMS once the weights are divided out (fp16 output: ~1e-3)
    rms = (nrm.float() / gamma.float()).pow(2).mean(dim=1).sqrt()
    assert float((rms - 1).abs().max()) < 2e-3
    res_d, nrm_d = torch.empty_like(x), torch.empty_like(x)
    ops.cuda_add_rms_norm_out(x, r, gamma, wl.EPS, res_d, nrm_d, "deterministic")
    assert torch.equal(res, res_d)
    # the modes differ in the sum's precision and in which copy of the residual is scaled: at most 2 fp16 ulps
    a, b = nrm.view(torch.int16).int(), nrm_d.view(torch.int16).int()
    assert int((a - b).abs().max()) <= 2 and float((a != b).float().mean()) < 0.35


def test_config3_fused_equals_unfused_within_rounding():
    c = wl.config3()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    q, k, gq, gk, pos = dev(c["q"]), dev(c["k"]), dev(c["gamma_q"]), dev(c["gamma_k"]), dev(c["positions"])
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    ops.qk_norm_rope_out(q, k, gq, gk, pos, wl.EPS, wl.THETA, qo, ko)
    qn, kn = ops.cuda_rms_norm(q, gq, wl.EPS), ops.cuda_rms_norm(k, gk, wl.EPS)
    ops.cuda_rope_token_positions_out(qn, pos, wl.THETA, qn)
    ops.cuda_rope_token_positions_out(kn, pos, wl.THETA, kn)
    for fused, unfused in ((qo, qn), (ko, kn)):
        diff = (fused.float() - unfused.float()).abs()
        assert float(diff.max()) <= 2 ** -7                    # 2 fp16 ulps at |x| < 8
        assert float((diff > 0).float().mean()) < 0.5
    # rotation preserves the norm of every (low, high) pair: position 0 rows are unrotated
    first = (c["positions"] == 0).nonzero()[0]
    assert first.size == 64
    plain = ops.cuda_rms_norm(q, gq, wl.EPS)
    idx = torch.from_numpy(first).to(DEV)
    assert float((qo[idx].float() - plain[idx].float()).abs().max()) <= 2 ** -8


@pytest.mark.parametrize("inter", [3072, 12288])
def test_config4_swiglu_full_size_linearity(inter):
    tokens = 262144
    gate, up = _randn(tokens, inter, sigma=2.0, seed=3), _randn(tokens, inter, sigma=0.5, seed=4)
    out = ops.cuda_swiglu(gate, up)
    out2 = ops.cuda_swiglu(gate, up * 2)                        # doubling is exact in fp32 and in normal fp16
    for rows in (slice(None, None, 997), slice(-64, None)):
        a, b = out[rows].float(), out2[rows].float()
        normal = a.abs() >= 2.0 ** -13                          # subnormal halves round differently when doubled
        assert torch.equal(b[normal], a[normal] * 2)
        assert float((b - a * 2).abs().max()) <= 2.0 ** -24
    probe = slice(0, 4096)
    want = torch.nn.functional.silu(gate[probe].float()) * up[probe].float()
    assert float(((out[probe].float() - want).abs() / want.abs().clamp_min(1e-3)).max()) < 2e-3
    ops.cuda_swiglu_out(gate, up, gate)                         # in place over 1.6 / 6.4 GB
    assert torch.equal(gate[::991], out[::991]) and torch.equal(gate[-1], out[-1])


def test_config4_gather_full_size_is_a_copy():
    c = wl.config4_gather(262144)
    table = torch.from_numpy(c["table"]).to(DEV)
    ids = torch.from_numpy(c["ids"]).to(DEV)
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.float16, device=DEV)
    ops.cuda_embedding_lookup_device_ids_out(table, ids, out)
    want = table.view(torch.int16).index_select(0, ids.long())
    assert torch.equal(out.view(torch.int16), want)


def test_config5_full_size_argmax_and_softmax():
    c = wl.config5()
    logits = torch.from_numpy(c["logits"]).to(DEV)
    planted = torch.from_numpy(c["planted"]).to(DEV)
    assert torch.equal(ops.argmax_rows(logits), planted)
    for mode in ("fast", "deterministic"):
        p = ops.cuda_softmax_last_dim(logits, mode)
        assert torch.equal(p.argmax(dim=1).int(), planted)
        tol = 1e-5 if mode == "fast" else 5e-4     # the index-order fp32 sum of the reference drifts (see test_gpu_vocab)
        assert float((p.double().sum(dim=1) - 1).abs().max()) < tol
        assert float(p.min()) >= 0
    fast = ops.cuda_softmax_last_dim(logits, "fast")
    assert torch.equal(fast, ops.cuda_softmax_last_dim(logits, "fast"))   # run-to-run bit identity
    # vocabulary halves through the sharded entry points (one GPU standing in for two)
    from cuda_llm_b200 import sharded
    lo, hi = sharded.column_range(wl.VOCAB, 2, 1)
    keys = torch.stack([sharded.argmax_keys(logits[:, :lo].contiguous(), 0),
                        sharded.argmax_keys(logits[:, lo:hi].contiguous(), lo)]).max(dim=0).values
    assert [sharded.decode_key(int(k)) for k in keys.cpu()] == c["planted"].tolist()
