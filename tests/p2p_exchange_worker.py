"""One rank of the two-GPU test of the fused exchange (launched by torch.distributed.run from
test_gpu_p2p_exchange.py): each rank holds half of the vocabulary; the fused calls must give the
oracle's indices / probabilities and the same answers as the NCCL-exchange forms, call after call."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from cuda_llm_b200 import sharded, workloads as wl  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    device = torch.device("cuda", torch.cuda.current_device())
    rows = 256
    x = wl.config5(rows=rows)["logits"]
    lo, hi = sharded.column_range(wl.VOCAB, world, rank)
    shard = torch.from_numpy(np.ascontiguousarray(x[:, lo:hi])).to(device)
    port = oracle.port()
    want_ids = port.argmax_rows(x)
    exact = port.softmax_f64(x)[:, lo:hi]
    ex = sharded.PeerExchange(max_rows=rows)
    try:
        for call in range(5):
            ids = sharded.sharded_argmax_fused(shard, lo, ex)
            assert np.array_equal(ids.cpu().numpy(), want_ids), f"rank {rank} call {call}: fused argmax"
            assert np.array_equal(sharded.sharded_argmax(shard, lo).cpu().numpy(), want_ids)
            got = sharded.sharded_softmax_fused(shard, ex).cpu().numpy().astype(np.float64)
            floor = port.softmax_f64(x).max(axis=-1, keepdims=True)
            err = float((np.abs(got - exact) / np.maximum(exact, floor)).max())
            assert err <= 1e-5, f"rank {rank} call {call}: fused softmax {err:.3e}"
            nccl = sharded.sharded_softmax(shard).cpu().numpy().astype(np.float64)
            assert float((np.abs(got - nccl) / np.maximum(exact, floor)).max()) <= 1e-5
        assert not ex.timed_out()
        # vocabulary-parallel LM head: every rank reads its rows of the tied embedding once; planted winners
        lm = wl.lm_head_case(4, 1024, wl.VOCAB, seed=6800, dtype=np.float16)
        planted = np.array([11, wl.VOCAB // 2 - 1, wl.VOCAB // 2, wl.VOCAB - 1], np.int32)
        for r in range(4):
            lm["table"][planted[r]] = (lm["hidden"][r].astype(np.float32) * np.float32(0.02)).astype(np.float16)
        tlo, thi = wl.shard_range(wl.VOCAB, world, rank)
        hidden = torch.from_numpy(lm["hidden"]).to(device)
        table_shard = torch.from_numpy(np.ascontiguousarray(lm["table"][tlo:thi])).to(device)
        for call in range(3):
            ids = sharded.sharded_lm_head_argmax(hidden, table_shard, tlo)
            assert np.array_equal(ids.cpu().numpy(), planted), f"rank {rank} call {call}: sharded LM head"
            ids = sharded.sharded_lm_head_argmax_fused(hidden, table_shard, tlo, ex)
            assert np.array_equal(ids.cpu().numpy(), planted), f"rank {rank} call {call}: sharded LM head, keys exchange"
        assert not ex.timed_out()
    finally:
        ex.close()
    dist.barrier()
    if rank == 0:
        print("P2P_EXCHANGE_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
