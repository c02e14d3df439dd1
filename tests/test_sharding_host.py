"""Host-side logic of the multi-GPU forms, on CPU: row/column ranges, the packed argmax key, and the
two exchange protocols run as two gloo ranks (the local arithmetic comes from the CPU oracle here; on
GPUs it is the CUDA kernels, see tests/test_gpu_vocab.py)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cuda_llm_b200 import sharded, workloads as wl


def test_row_ranges_partition_exactly():
    for total in (0, 1, 7, 256, 151936, 262144):
        for world in (1, 2, 3, 4, 8):
            spans = [sharded.row_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    assert [sharded.column_range(wl.VOCAB, 8, r) for r in (0, 7)] == [(0, 18992), (132944, 151936)]
    with pytest.raises(ValueError):
        sharded.row_range(10, 2, 2)


def test_key_decode_matches_oracle(port):
    rng = np.random.default_rng(3)
    for v, i in zip(rng.standard_normal(200).astype(np.float32), rng.integers(0, 2 ** 31 - 1, 200)):
        assert sharded.decode_key(port.argmax_key(float(v), int(i))) == int(i)
    assert sharded.decode_key(sharded.KEY_NONE) == 0 == port.argmax_key_index(sharded.KEY_NONE)
    assert port.argmax_key(float("nan"), 3) == sharded.KEY_NONE


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, tcp_port, rows, width, seed, result_dir):
    import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(tcp_port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    port = oracle.port()
    x = np.round(wl.config5(rows=rows, vocab=width, seed=seed)["logits"])      # rounded: ties across shards
    lo, hi = sharded.column_range(width, world, rank)
    mine = np.ascontiguousarray(x[:, lo:hi])
    # argmax: local keys -> all-reduce(MAX) -> decode
    local = port.argmax_rows(mine)
    keys = torch.tensor([port.argmax_key(float(mine[r, local[r]]), lo + int(local[r])) for r in range(rows)],
                        dtype=torch.int64)
    sharded.allreduce_argmax_keys(keys)
    ids = np.array([sharded.decode_key(int(k)) for k in keys], np.int32)
    # softmax: local (max, sum) -> all-reduce(MAX) -> rebase -> all-reduce(SUM) -> scale local columns
    m = mine.max(axis=1)
    s = np.exp(mine.astype(np.float64) - m[:, None]).sum(axis=1).astype(np.float32)

    def rebase(local_max, global_max, local_sum):
        local_sum.mul_(torch.exp(local_max - global_max))
    gmax, gsum = sharded.allreduce_softmax_stats(torch.from_numpy(m.copy()), torch.from_numpy(s.copy()), rebase)
    probs = np.exp(mine.astype(np.float64) - gmax.numpy()[:, None]) / gsum.numpy()[:, None].astype(np.float64)
    # vocabulary-parallel LM head: the table's rows split over the ranks, local logits -> keys -> the same exchange
    lm = wl.lm_head_case(3, 64, 500, seed=seed + 1, dtype=np.float32)
    tlo, thi = wl.shard_range(500, world, rank)
    part = port.linear(lm["hidden"], lm["table"][tlo:thi])
    best = port.argmax_rows(part)
    lm_keys = torch.tensor([port.argmax_key(float(part[r, best[r]]), tlo + int(best[r])) for r in range(3)], dtype=torch.int64)
    sharded.allreduce_argmax_keys(lm_keys)
    lm_ids = np.array([sharded.decode_key(int(k)) for k in lm_keys], np.int32)
    np.savez(os.path.join(result_dir, f"rank{rank}.npz"), ids=ids, probs=probs, lo=lo, hi=hi, lm_ids=lm_ids)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_vocab_sharded_protocols_over_gloo(port, tmp_path, world):
    rows, width, seed = 16, 4096, 5003
    mp.spawn(_worker, args=(world, _free_port(), rows, width, seed, str(tmp_path)), nprocs=world, join=True)
    x = np.round(wl.config5(rows=rows, vocab=width, seed=seed)["logits"])
    # rounded logits repeat values, which biases the CPU operator's fp32 running sum by up to 3e-5:
    # the protocol is checked against the exact (fp64) softmax instead
    want_ids, want_p = port.argmax_rows(x), port.softmax_f64(x)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    lm = wl.lm_head_case(3, 64, 500, seed=seed + 1, dtype=np.float32)
    want_lm = port.argmax_rows(port.linear(lm["hidden"], lm["table"]))
    for p in parts:
        assert np.array_equal(p["ids"], want_ids)               # every rank holds the global winner
        assert np.array_equal(p["lm_ids"], want_lm)
    probs = np.concatenate([p["probs"] for p in parts], axis=1)
    assert (np.abs(probs - want_p) <= 1e-5 * want_p.max(axis=1, keepdims=True)).all()
