"""Multi-GPU forms of the operators: one process per GPU, torch.distributed plumbing.

Row-independent operators (RMSNorm family, RoPE, SwiGLU, add, gather) shard by
token rows with NO collective: each rank runs the single-GPU operator on its
contiguous row range (`row_range`).

The two vocabulary-wide reductions shard by columns and need one small exchange:

  argmax   every rank folds its columns to one packed (value, global index) key per
           row; a single all-reduce(MAX) over int64 keys picks the global winner with
           the reference's tie rule (largest value, lowest index).
  softmax  every rank computes (max, sum exp(x - max)) over its columns; all-reduce(MAX)
           of the maxima, re-base the sums to the global max, all-reduce(SUM), then
           scale the local columns.

The exchange helpers take any process group (NCCL over NVLink on GPUs; gloo in the
CPU protocol tests) and leave the arithmetic to the caller-supplied device kernels.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import lib as _lib
from . import ops as _ops

KEY_NONE = -(1 << 63)  # "no candidate in this shard": the minimum int64, decodes to index 0


def row_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) rows owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError("row_range: need world > 0, 0 <= rank < world, total >= 0")
    return total * rank // world, total * (rank + 1) // world


def column_range(width: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) vocabulary columns owned by `rank`."""
    return row_range(width, world, rank)


def decode_key(key: int) -> int:
    """Global index carried by a packed int64 key (host-side twin of b2_argmax_decode_keys)."""
    if key == KEY_NONE:
        return 0
    return 0xFFFFFFFF - (key & 0xFFFFFFFF)


def allreduce_argmax_keys(keys: torch.Tensor, group=None) -> torch.Tensor:
    """In-place all-reduce(MAX) of int64 keys [rows]; one message of rows*8 bytes per rank."""
    if keys.dtype != torch.int64:
        raise ValueError("allreduce_argmax_keys: keys must be int64")
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(keys, op=dist.ReduceOp.MAX, group=group)
    return keys


def allreduce_softmax_stats(row_max: torch.Tensor, row_sum: torch.Tensor,
                            rebase: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], None],
                            group=None, global_max: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Turns per-shard (max, sum) into the global (max, sum), in two small all-reduces.
    `rebase(local_max, global_max, local_sum)` multiplies local_sum by exp(local_max - global_max)
    in place (the b2_softmax_rebase kernel on GPUs).  row_sum is updated in place.  `global_max` may be a
    preallocated buffer (nothing is allocated then, which suits CUDA-graph capture)."""
    if global_max is None:
        global_max = row_max.clone()
    else:
        global_max.copy_(row_max)
    multi = dist.is_initialized() and dist.get_world_size(group) > 1
    if multi:
        dist.all_reduce(global_max, op=dist.ReduceOp.MAX, group=group)
    rebase(row_max, global_max, row_sum)
    if multi:
        dist.all_reduce(row_sum, op=dist.ReduceOp.SUM, group=group)
    return global_max, row_sum


# ---------------------------------------------------------------- GPU drivers

def argmax_keys(logits_shard: torch.Tensor, index_base: int, keys: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed keys [rows] of this rank's columns (b2_argmax_keys)."""
    _ops._logits_req(logits_shard, "sharded_argmax")
    rows, width = logits_shard.shape
    if keys is None:
        keys = torch.empty(rows, dtype=torch.int64, device=logits_shard.device)
    ws = _ops.argmax_workspace(logits_shard.device, rows)
    _lib.check(_lib.load().b2_argmax_keys(logits_shard.data_ptr(), rows, width, width, _ops._code(logits_shard),
                                          index_base, keys.data_ptr(), ws.data_ptr(), _ops._stream()))
    return keys


def sharded_argmax(logits_shard: torch.Tensor, index_base: int, group=None, keys: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Global row argmax (int32 [rows], on the device) of logits whose columns
    [index_base, index_base + shard width) live on this rank.  With `keys` (int64 [rows]) and `out`
    (int32 [rows]) given nothing is allocated, so the call can be recorded into a CUDA graph
    together with its all-reduce."""
    keys = allreduce_argmax_keys(argmax_keys(logits_shard, index_base, keys), group)
    if out is None:
        out = torch.empty(keys.shape[0], dtype=torch.int32, device=keys.device)
    _lib.check(_lib.load().b2_argmax_decode_keys(keys.data_ptr(), keys.shape[0], out.data_ptr(), _ops._stream()))
    return out


def _rebase_kernel(row_max: torch.Tensor, global_max: torch.Tensor, row_sum: torch.Tensor) -> None:
    _lib.check(_lib.load().b2_softmax_rebase(row_max.data_ptr(), global_max.data_ptr(), row_sum.data_ptr(),
                                             row_sum.shape[0], _ops._stream()))


def sharded_softmax(logits_shard: torch.Tensor, group=None, out: Optional[torch.Tensor] = None,
                    stats: Optional[torch.Tensor] = None) -> torch.Tensor:
    """This rank's columns of the row softmax taken over ALL ranks' columns.  `stats`: optional float32
    [3, rows] scratch (local max, local sum, global max); with it and `out` given nothing is allocated."""
    _ops._logits_req(logits_shard, "sharded_softmax")
    rows, width = logits_shard.shape
    L = _lib.load()
    if stats is None:
        stats = torch.empty(3, rows, dtype=torch.float32, device=logits_shard.device)
    row_max, row_sum, gmax_buf = stats[0], stats[1], stats[2]
    code = _ops._code(logits_shard)
    _lib.check(L.b2_softmax_stats(logits_shard.data_ptr(), rows, width, code, row_max.data_ptr(), row_sum.data_ptr(),
                                  _ops._stream()))
    global_max, global_sum = allreduce_softmax_stats(row_max, row_sum, _rebase_kernel, group, gmax_buf)
    if out is None:
        out = torch.empty_like(logits_shard)
    _lib.check(L.b2_softmax_apply(logits_shard.data_ptr(), out.data_ptr(), rows, width, code, global_max.data_ptr(),
                                  global_sum.data_ptr(), _ops._stream()))
    return out
