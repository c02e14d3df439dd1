"""GPU parity (bit-exact) of the row moves around the paged KV cache and of the last-valid-row gather,
through the C ABI, against the index arithmetic of the reference's kernels restated in oracle/oracle.c."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import lib, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()


def pool(rng, layers, total_blocks, block_size, kv_heads, head_dim, dtype):
    return rng.standard_normal((layers, total_blocks, 2, block_size, kv_heads, head_dim)).astype(dtype)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("batch,kv_heads,head_dim,block_size", [(1, 8, 128, 16), (4, 8, 128, 16), (64, 8, 128, 32), (7, 2, 24, 4),
                                                                (300, 1, 3, 5)])
def test_decode_batch_write(b2, port, dtype, batch, kv_heads, head_dim, block_size):
    rng = np.random.default_rng(batch + head_dim)
    layers, max_blocks = 3, 6
    total_blocks = batch * max_blocks + 2
    storage = pool(rng, layers, total_blocks, block_size, kv_heads, head_dim, dtype)
    key = rng.standard_normal((batch, kv_heads, head_dim)).astype(dtype)
    value = rng.standard_normal((batch, kv_heads, head_dim)).astype(dtype)
    tables = rng.permutation(total_blocks)[: batch * max_blocks].reshape(batch, max_blocks).astype(np.int32)   # disjoint blocks
    positions = rng.integers(0, max_blocks * block_size, batch).astype(np.int32)
    want = storage.copy()
    port.paged_kv_write(0, key, value, want, tables, positions, 1, total_blocks, block_size)
    got = dev(storage)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.paged_kv_write_decode_batch(dev(key), dev(value), got, 1, dev(tables), dev(positions), status)
    assert np.array_equal(host(got).view(np.uint8), want.view(np.uint8))
    assert int(status.item()) == 0


def test_single_decode_write_and_prefill_copy(b2, port):
    rng = np.random.default_rng(3)
    layers, total_blocks, block_size, kv_heads, head_dim = 2, 40, 16, 8, 128
    storage = pool(rng, layers, total_blocks, block_size, kv_heads, head_dim, np.float16)
    table = rng.permutation(total_blocks)[:20].astype(np.int32)
    # single decode: the token at cache_length - 1; nothing at cache_length 0
    for length in (0, 1, 16, 17, 320):
        key = rng.standard_normal((1, kv_heads, head_dim)).astype(np.float16)
        value = rng.standard_normal((1, kv_heads, head_dim)).astype(np.float16)
        want = storage.copy()
        port.paged_kv_write(2, key, value, want, table, np.array([length], np.int32), 0, total_blocks, block_size)
        got = dev(storage)
        ops.paged_kv_write_decode(dev(key[0]), dev(value[0]), got, 0, dev(table), dev(np.array([length], np.int32)))
        assert np.array_equal(host(got).view(np.uint16), want.view(np.uint16)), length
    # packed prefill: ragged token counts, including one that ends inside a block
    for tokens in (1, 15, 16, 100, 320):
        key = rng.standard_normal((tokens, kv_heads, head_dim)).astype(np.float16)
        value = rng.standard_normal((tokens, kv_heads, head_dim)).astype(np.float16)
        want = storage.copy()
        port.paged_kv_write(1, key, value, want, table, np.zeros(1, np.int32), 1, total_blocks, block_size)
        got = dev(storage)
        ops.paged_kv_prefill_copy_packed(dev(key), dev(value), got, dev(table), 1)
        assert np.array_equal(host(got).view(np.uint16), want.view(np.uint16)), tokens
    with pytest.raises(ValueError):
        ops.paged_kv_prefill_copy_packed(dev(key), dev(value), dev(storage), dev(table[:3]), 1)   # table too short
    with pytest.raises(ValueError):
        ops.paged_kv_prefill_copy_packed(dev(key), dev(value), dev(storage), dev(table), 2)       # layer out of range


def test_bad_block_ids_never_reach_memory(b2):
    rng = np.random.default_rng(4)
    storage = pool(rng, 1, 4, 4, 2, 8, np.float16)
    key = rng.standard_normal((3, 2, 8)).astype(np.float16)
    tables = np.array([[0, 1], [99, 2], [3, -1]], np.int32)
    positions = np.array([1, 0, 5], np.int32)           # row 1 -> block 99, row 2 -> block -1: both skipped
    got = dev(storage)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.paged_kv_write_decode_batch(dev(key), dev(key), got, 0, dev(tables), dev(positions), status)
    want = storage.copy()
    want[0, 0, 0, 1], want[0, 0, 1, 1] = key[0], key[0]
    assert np.array_equal(host(got), want) and int(status.item()) == 1


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("batch,seq,width", [(1, 1, 7), (3, 5, 1000), (4, 32, 151936), (64, 4, 4099)])
def test_select_last_valid_logits(b2, port, dtype, batch, seq, width):
    rng = np.random.default_rng(batch * seq + width)
    padded = rng.standard_normal((batch, seq, width)).astype(dtype)
    lengths = rng.integers(1, seq + 1, batch)
    lengths[0] = seq
    got = host(ops.select_last_valid_logits(dev(padded), [int(n) for n in lengths]))
    assert np.array_equal(got.view(np.uint8), port.select_last_valid(padded, lengths).view(np.uint8))
    with pytest.raises(ValueError):
        ops.select_last_valid_logits(dev(padded), [0] * batch)
    with pytest.raises(ValueError):
        ops.select_last_valid_logits(dev(padded), [seq + 1] * batch)
    with pytest.raises(ValueError):
        ops.select_last_valid_logits(dev(padded)[0], [1])


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("tokens,mode", [(1, "decode"), (7, "decode"), (256, "decode"), (100, "prefill"), (1000, "prefill")])
def test_qk_norm_rope_straight_into_the_paged_cache(b2, port, dtype, tokens, mode):
    """b2_qk_norm_rope_paged = b2_qk_norm_rope + the paged K/V write, bit for bit, and within the parity bound of
    the CPU oracle's rms_norm -> rope for the keys that land in the cache."""
    from cuda_llm_b200 import workloads as wl
    rng = np.random.default_rng(tokens)
    q_heads, kv_heads, head_dim, block_size, layers = 16, 8, 128, 16, 2
    q = wl.normal(rng, (tokens, q_heads, head_dim)).astype(dtype)
    k = wl.normal(rng, (tokens, kv_heads, head_dim)).astype(dtype)
    v = wl.normal(rng, (tokens, kv_heads, head_dim)).astype(dtype)
    gq, gk = wl.gamma(rng, head_dim).astype(dtype), wl.gamma(rng, head_dim).astype(dtype)
    if mode == "decode":
        max_blocks = 4
        total_blocks = tokens * max_blocks + 3
        tables = rng.permutation(total_blocks)[: tokens * max_blocks].reshape(tokens, max_blocks).astype(np.int32)
        positions = rng.integers(0, max_blocks * block_size, tokens).astype(np.int32)
        slots, per_table = positions, 1
    else:
        max_blocks = -(-tokens // block_size)
        total_blocks = max_blocks + 5
        tables = rng.permutation(total_blocks)[:max_blocks].astype(np.int32)
        positions = np.arange(tokens, dtype=np.int32) + 3          # rotary positions need not equal the cache slots
        slots, per_table = None, tokens
    storage = rng.standard_normal((layers, total_blocks, 2, block_size, kv_heads, head_dim)).astype(dtype)

    # the separate operators
    want_q, k_rot = torch.empty_like(dev(q)), torch.empty_like(dev(k))
    ops.qk_norm_rope_out(dev(q), dev(k), dev(gq), dev(gk), dev(positions), wl.EPS, wl.THETA, want_q, k_rot)
    want_storage = dev(storage)
    if mode == "decode":
        ops.paged_kv_write_decode_batch(k_rot, dev(v), want_storage, 1, dev(tables), dev(positions))
    else:
        ops.paged_kv_prefill_copy_packed(k_rot, dev(v), want_storage, dev(tables), 1)
    # one launch
    got_q, got_storage = torch.empty_like(want_q), dev(storage)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qk_norm_rope_paged_out(dev(q), dev(k), dev(v), dev(gq), dev(gk), dev(positions), wl.EPS, wl.THETA, got_q, got_storage, 1,
                               dev(tables), None if slots is None else dev(slots), per_table, status)
    assert torch.equal(got_q.view(torch.uint8), want_q.view(torch.uint8))
    assert torch.equal(got_storage.view(torch.uint8), want_storage.view(torch.uint8))
    assert int(status.item()) == 0
    # the keys in the cache against the CPU oracle
    # (1 fp16 ulp / 1e-5 of the output, or of the larger input of the rotated pair where the output cancelled:
    # the rule of the RoPE parity tests)
    from test_gpu_rope import pair_scale
    from util import ulp16
    kf = k.astype(np.float32)
    normed = port.rms_norm(kf.reshape(-1, head_dim), gk.astype(np.float32), wl.EPS).reshape(kf.shape)
    ref_k = port.rope(normed, positions, wl.THETA)
    scale = np.maximum(np.abs(ref_k), pair_scale(normed))
    got = host(got_storage)
    for t in (0, tokens // 2, tokens - 1):
        pos = int(positions[t]) if mode == "decode" else t
        blk = tables[t, pos // block_size] if mode == "decode" else tables[pos // block_size]
        row = got[1, blk, 0, pos % block_size].astype(np.float64)
        err = np.abs(row - ref_k[t])
        if dtype == np.float16:
            assert float((err / ulp16(scale[t])).max()) <= 1.0, f"cached key of token {t}"
        else:
            assert float((err / scale[t]).max()) <= 1e-5, f"cached key of token {t}"
        assert np.array_equal(got[1, blk, 1, pos % block_size], v[t])
