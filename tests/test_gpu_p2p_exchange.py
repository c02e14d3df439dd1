"""The vocabulary-sharded reductions with the inter-GPU exchange fused into the kernel
(b2_argmax_rows_sharded, b2_softmax_stats_sharded), through the C ABI.

On one GPU the ranks cannot run side by side (kernels that wait for one another must not share
a GPU), so they run ONE AFTER THE OTHER over exchange buffers that all live on this GPU: ranks
world-1 .. 1 go first with a few milliseconds of patience, push their partials into every buffer,
find nobody answering and report it through the status word (the bounded wait doing its job);
rank 0 goes last, finds every peer's partials already in its buffer and must produce the global result.
The real thing, two processes on two GPUs, runs when the box has them."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from cuda_llm_b200 import lib, ops, sharded, workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
host = lambda t: t.cpu().numpy()
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class LocalWorld:
    """`world` exchange buffers on one GPU and the descriptor each emulated rank would hold."""

    def __init__(self, L, world, max_rows, patience_ms):
        self.L, self.world = L, world
        size = L.b2_p2p_exchange_bytes(world, max_rows)
        self.buffers = [torch.zeros(size, dtype=torch.uint8, device=DEV) for _ in range(world)]
        self.status = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(world)]
        self.desc = []
        for r in range(world):
            d = lib.P2PExchange()
            for g in range(world):
                d.buffers[g] = self.buffers[g].data_ptr()
            d.world, d.rank, d.max_rows = world, r, max_rows
            d.timeout_ms = 2000 if r == 0 else patience_ms
            self.desc.append(d)


def stream():
    return torch.cuda.current_stream().cuda_stream


# 128 rows over 8 shards: short shards and enough rows to fill the GPU take the one-block-per-row form of the kernel
@pytest.mark.parametrize("world,rows", [(1, 64), (2, 64), (8, 64), (8, 128), (4, 256)])
def test_fused_argmax_ranks_in_turn(b2, port, world, rows):
    L = b2
    c5 = wl.config5(rows=rows)
    x = c5["logits"]
    x[5, :] = -np.inf                                   # no candidate anywhere: index 0
    x[6, 100], x[6, wl.VOCAB - 7] = 99.0, 99.0           # tie across shards: the lower index wins
    want = port.argmax_rows(x)
    shards = [dev(x[:, slice(*sharded.column_range(wl.VOCAB, world, r))]) for r in range(world)]
    lw = LocalWorld(L, world, rows, patience_ms=3)
    ws = ops.argmax_workspace(torch.device(DEV), rows)
    outs = [torch.full((rows,), -1, dtype=torch.int32, device=DEV) for _ in range(world)]
    for call in range(3):                                # three calls: both parities of the buffers, and reuse
        for r in reversed(range(world)):
            lo, _ = sharded.column_range(wl.VOCAB, world, r)
            lib.check(L.b2_argmax_rows_sharded(shards[r].data_ptr(), rows, shards[r].shape[1], shards[r].shape[1], lib.F32,
                                               lo, outs[r].data_ptr(), ws.data_ptr(), C.byref(lw.desc[r]),
                                               lw.status[r].data_ptr(), stream()))
            torch.cuda.synchronize()
        assert int(lw.status[0].item()) == 0
        assert np.array_equal(host(outs[0]), want), f"call {call}"
        for r in range(1, world):
            assert int(lw.status[r].item()) == 2          # nobody answered within its patience: reported, not hung
        outs[0].fill_(-1)
    assert ops.cuda_argmax_last_row(dev(x)) == int(want[-1])   # the context is fine after the timeouts


@pytest.mark.parametrize("world", [1, 2, 8])
def test_sharded_lm_head_keys_exchange_ranks_in_turn(b2, port, world):
    """Vocabulary-parallel LM head: every emulated rank runs b2_lm_head_argmax over its rows of the table (keys
    form), then b2_argmax_keys_exchange; rank 0, last, must hold the pick over the whole table."""
    L = b2
    rows, vocab = 5, 4096
    c = wl.lm_head_case(rows, 1024, vocab, seed=7100 + world, dtype=np.float16)
    f32 = lambda a: port.decode_f16(np.ascontiguousarray(a).view(np.uint16)).reshape(a.shape)
    stored = port.linear(f32(c["hidden"]), f32(c["table"])).astype(np.float16)
    want = port.argmax_rows(stored.view(np.uint16))
    hidden = dev(c["hidden"])
    shards = [dev(c["table"][slice(*wl.shard_range(vocab, world, r))]) for r in range(world)]
    lw = LocalWorld(L, world, rows, patience_ms=3)
    ws = ops.argmax_workspace(torch.device(DEV), rows)
    keys = [torch.zeros(rows, dtype=torch.int64, device=DEV) for _ in range(world)]
    outs = [torch.full((rows,), -1, dtype=torch.int32, device=DEV) for _ in range(world)]
    for call in range(3):
        for r in reversed(range(world)):
            lo, hi = wl.shard_range(vocab, world, r)
            lib.check(L.b2_lm_head_argmax(hidden.data_ptr(), shards[r].data_ptr(), rows, 1024, hi - lo, lib.F16, lib.DETERMINISTIC,
                                          lo, None, hi - lo, None, keys[r].data_ptr(), ws.data_ptr(), stream()))
            lib.check(L.b2_argmax_keys_exchange(keys[r].data_ptr(), rows, outs[r].data_ptr(), C.byref(lw.desc[r]),
                                                lw.status[r].data_ptr(), stream()))
            torch.cuda.synchronize()
        assert int(lw.status[0].item()) == 0
        assert np.array_equal(host(outs[0]), want), f"call {call}"
        for r in range(1, world):
            assert int(lw.status[r].item()) == 2          # nobody answered within its patience: reported, not hung
        outs[0].fill_(-1)


@pytest.mark.parametrize("world", [1, 4])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_fused_softmax_ranks_in_turn(b2, port, world, dtype):
    from test_gpu_vocab import softmax_check
    from util import assert_within_1ulp_f16
    L = b2
    rows = 24
    x = wl.config5(rows=rows)["logits"].astype(dtype)
    x[2, : wl.VOCAB // 2] = -np.inf                      # a whole shard of a row masked
    code = lib.F32 if dtype == np.float32 else lib.F16
    shards = [dev(x[:, slice(*sharded.column_range(wl.VOCAB, world, r))]) for r in range(world)]
    lw = LocalWorld(L, world, rows, patience_ms=3)
    stats = [torch.empty(2, rows, device=DEV) for _ in range(world)]
    for call in range(2):
        for r in reversed(range(world)):
            lib.check(L.b2_softmax_stats_sharded(shards[r].data_ptr(), rows, shards[r].shape[1], code, stats[r][0].data_ptr(),
                                                 stats[r][1].data_ptr(), C.byref(lw.desc[r]), lw.status[r].data_ptr(), stream()))
            torch.cuda.synchronize()
        assert int(lw.status[0].item()) == 0
        # rank 0 holds the statistics of the whole rows: apply them to EVERY shard and compare the full result
        outs = []
        for r in range(world):
            o = torch.empty_like(shards[r])
            lib.check(L.b2_softmax_apply(shards[r].data_ptr(), o.data_ptr(), rows, shards[r].shape[1], code,
                                         stats[0][0].data_ptr(), stats[0][1].data_ptr(), stream()))
            outs.append(host(o))
        got = np.concatenate(outs, axis=1)
        xf = x.astype(np.float32)
        if dtype == np.float32:
            softmax_check(got, xf, port, "fast", f"fused sharded softmax world={world} call {call}")
        else:
            assert_within_1ulp_f16(got, port.softmax_f64(xf), f"fused sharded softmax f16 world={world}")


def test_wait_for_a_silent_peer_runs_out_and_is_reported(b2, port):
    """A peer that never publishes: the kernel gives up after timeout_ms, says so in the status word,
    ends normally, and the context stays usable."""
    L = b2
    rows = 8
    x = wl.config5(rows=rows)["logits"]
    lw = LocalWorld(L, 2, rows, patience_ms=3)
    lw.desc[0].timeout_ms = 20
    ws = ops.argmax_workspace(torch.device(DEV), rows)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    t = dev(x)
    lib.check(L.b2_argmax_rows_sharded(t.data_ptr(), rows, wl.VOCAB, wl.VOCAB, lib.F32, 0, out.data_ptr(), ws.data_ptr(),
                                       C.byref(lw.desc[0]), lw.status[0].data_ptr(), stream()))
    torch.cuda.synchronize()
    assert int(lw.status[0].item()) == 2
    assert (host(out) == -1).all()                      # and the rows themselves say that they are not results
    assert np.array_equal(host(ops.argmax_rows(t)), port.argmax_rows(x))
    # argument errors
    bad = lib.P2PExchange()
    bad.world, bad.rank, bad.max_rows = 2, 5, rows
    assert L.b2_argmax_rows_sharded(t.data_ptr(), rows, wl.VOCAB, wl.VOCAB, lib.F32, 0, out.data_ptr(), ws.data_ptr(),
                                    C.byref(bad), None, stream()) == -1
    lw.desc[0].max_rows = 4
    assert L.b2_argmax_rows_sharded(t.data_ptr(), rows, wl.VOCAB, wl.VOCAB, lib.F32, 0, out.data_ptr(), ws.data_ptr(),
                                    C.byref(lw.desc[0]), None, stream()) == -4


def test_world_of_one_through_the_python_drivers(b2, port):
    x = wl.config5(rows=16)["logits"]
    ex = sharded.PeerExchange(max_rows=16)
    try:
        for _ in range(3):
            assert np.array_equal(host(sharded.sharded_argmax_fused(dev(x), 0, ex)), port.argmax_rows(x))
        from test_gpu_vocab import softmax_check
        softmax_check(host(sharded.sharded_softmax_fused(dev(x), ex)), x, port, "fast", "fused softmax, one rank")
        assert not ex.timed_out()
    finally:
        ex.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_per_gpu_over_nvlink(b2):
    """One rank per GPU of the box (2, 4 or 8) over NVLink peer mappings: fused results equal the NCCL-exchange
    results and the oracle's, call after call."""
    ranks = 8 if torch.cuda.device_count() >= 8 else 4 if torch.cuda.device_count() >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT + os.pathsep + os.path.join(ROOT, "tests"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(ROOT, "tests", "p2p_exchange_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "P2P_EXCHANGE_OK" in proc.stdout
