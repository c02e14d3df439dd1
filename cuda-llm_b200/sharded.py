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


def sharded_lm_head_argmax(hidden: torch.Tensor, table_shard: torch.Tensor, index_base: int, group=None,
                           keys: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy pick over a tied embedding whose rows [index_base, index_base + shard rows) live on this rank
    (a vocabulary-parallel LM head): every rank reads only its slice of the table once
    (b2_lm_head_argmax, keys form), then one all-reduce(MAX) of `rows` packed keys and the decode, exactly
    the exchange of sharded_argmax; no logits tensor exists anywhere."""
    rows = hidden.shape[0]
    if keys is None:
        keys = torch.empty(rows, dtype=torch.int64, device=hidden.device)
    _ops.lm_head_argmax(hidden, table_shard, want_ids=False, keys_out=keys, index_base=index_base)
    keys = allreduce_argmax_keys(keys, group)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=keys.device)
    _lib.check(_lib.load().b2_argmax_decode_keys(keys.data_ptr(), rows, out.data_ptr(), _ops._stream()))
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


# ---------------------------------------------------------------- exchange fused into the kernels

class PeerExchange:
    """Exchange buffers of a group of GPUs on one NVLink node, for the fused forms below.

    Every rank allocates one buffer, exports it as a CUDA IPC handle, gathers the handles over the
    process group (host side, once) and maps its peers' buffers.  After that a fused call is ONE kernel
    launch per GPU: the reduction kernel's last thread block stores this GPU's per-row partials into
    every peer's buffer through NVLink, publishes them with a release flag, waits (bounded by
    `timeout_ms`) for the peers' flags and finishes the rows (include/b2ops.h, b2_p2p_exchange).
    All ranks must make the same sequence of fused calls.  `status` is a device int32 that a kernel
    ORs 2 into when its wait ran out (the results of that call are invalid; call reset() on every rank).
    """

    def __init__(self, max_rows: int, group=None, device=None, timeout_ms: int = 2000):
        import ctypes as C
        self._C = C
        self.group = group
        multi = dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        if self.world > _lib.P2P_MAX_WORLD:
            raise ValueError(f"PeerExchange: at most {_lib.P2P_MAX_WORLD} ranks")
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.max_rows = int(max_rows)
        L = _lib.load()
        self._L = L
        with torch.cuda.device(self.device):
            size = L.b2_p2p_exchange_bytes(self.world, self.max_rows)
            if size == 0:
                raise ValueError("PeerExchange: max_rows out of range")
            self.buffer = L.b2_alloc(size)
            if not self.buffer:
                _lib.check(-2)      # B2_ERR_CUDA, with the library's message
            self._opened = []
            self.reset(_barrier=False)
            pointers = [None] * self.world
            pointers[self.rank] = self.buffer
            if multi:
                handle = (C.c_ubyte * 64)()
                _lib.check(L.b2_ipc_export(self.buffer, handle))
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
                for r, h in enumerate(handles):
                    if r == self.rank:
                        continue
                    p = C.c_void_p()
                    _lib.check(L.b2_ipc_open((C.c_ubyte * 64).from_buffer_copy(h), C.byref(p)))
                    pointers[r] = p.value
                    self._opened.append(p.value)
                dist.barrier(group=group)      # every buffer is initialised and mapped before the first call
        self.desc = _lib.P2PExchange()
        for r, p in enumerate(pointers):
            self.desc.buffers[r] = p
        self.desc.world, self.desc.rank = self.world, self.rank
        self.desc.max_rows, self.desc.timeout_ms = self.max_rows, int(timeout_ms)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def reset(self, _barrier: bool = True) -> None:
        """Zero this rank's buffer (epochs, flags, slots).  After a timeout every rank calls this."""
        torch.cuda.synchronize(self.device)
        _lib.check(self._L.b2_p2p_exchange_init(self.buffer, self.world, self.max_rows, _ops._stream()))
        torch.cuda.synchronize(self.device)
        if _barrier and self.world > 1:
            dist.barrier(group=self.group)

    def timed_out(self) -> bool:
        """Blocking read of the status word: True when some fused call's wait for its peers ran out."""
        return bool(int(self.status.item()) & 2)

    def close(self) -> None:
        if getattr(self, "buffer", None):
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)     # nobody unmaps while a peer may still store into it
            for p in self._opened:
                self._L.b2_ipc_close(p)
            self._opened = []
            self._L.b2_free(self.buffer)
            self.buffer = None


def sharded_argmax_fused(logits_shard: torch.Tensor, index_base: int, exchange: PeerExchange,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sharded_argmax as ONE kernel per GPU (b2_argmax_rows_sharded): the keys cross NVLink as plain
    stores from the reduction kernel itself; no collective library call, no second kernel."""
    _ops._logits_req(logits_shard, "sharded_argmax_fused")
    rows, width = logits_shard.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits_shard.device)
    ws = _ops.argmax_workspace(logits_shard.device, rows)
    import ctypes as C
    _lib.check(_lib.load().b2_argmax_rows_sharded(logits_shard.data_ptr(), rows, width, width, _ops._code(logits_shard),
                                                  index_base, out.data_ptr(), ws.data_ptr(), C.byref(exchange.desc),
                                                  exchange.status.data_ptr(), _ops._stream()))
    return out


def sharded_lm_head_argmax_fused(hidden: torch.Tensor, table_shard: torch.Tensor, index_base: int, exchange: PeerExchange,
                                 keys: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sharded_lm_head_argmax without a collective library call: the LM-head kernel leaves this GPU's packed keys
    on the device and one small kernel (b2_argmax_keys_exchange) stores them into every peer's exchange buffer over
    NVLink, waits (bounded) for the peers' and writes the global winners' indices."""
    rows = hidden.shape[0]
    if keys is None:
        keys = torch.empty(rows, dtype=torch.int64, device=hidden.device)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=hidden.device)
    _ops.lm_head_argmax(hidden, table_shard, want_ids=False, keys_out=keys, index_base=index_base)
    import ctypes as C
    _lib.check(_lib.load().b2_argmax_keys_exchange(keys.data_ptr(), rows, out.data_ptr(), C.byref(exchange.desc),
                                                   exchange.status.data_ptr(), _ops._stream()))
    return out


def sharded_softmax_fused(logits_shard: torch.Tensor, exchange: PeerExchange, out: Optional[torch.Tensor] = None,
                          stats: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sharded_softmax as two kernels per GPU and no collective library call: the statistics kernel
    exchanges (max, sum) pairs itself (b2_softmax_stats_sharded), then b2_softmax_apply scales this
    rank's columns.  `stats`: optional float32 [2, rows] scratch."""
    _ops._logits_req(logits_shard, "sharded_softmax_fused")
    rows, width = logits_shard.shape
    L = _lib.load()
    if stats is None:
        stats = torch.empty(2, rows, dtype=torch.float32, device=logits_shard.device)
    if out is None:
        out = torch.empty_like(logits_shard)
    code = _ops._code(logits_shard)
    import ctypes as C
    _lib.check(L.b2_softmax_stats_sharded(logits_shard.data_ptr(), rows, width, code, stats[0].data_ptr(),
                                          stats[1].data_ptr(), C.byref(exchange.desc), exchange.status.data_ptr(),
                                          _ops._stream()))
    _lib.check(L.b2_softmax_apply(logits_shard.data_ptr(), out.data_ptr(), rows, width, code, stats[0].data_ptr(),
                                  stats[1].data_ptr(), _ops._stream()))
    return out


# ---------------------------------------------------------------- bound calls

def _bound(fn, args):
    """fn(*args) as a zero-argument callable, the arguments converted to their C types once."""
    converted = [t(a) for t, a in zip(fn.argtypes, args)]
    check = _lib.check

    def call():
        rc = fn(*converted)
        if rc:
            check(rc)
    call.keepalive = args
    return call


def bind_argmax_fused(logits_shard: torch.Tensor, index_base: int, exchange: PeerExchange, out: torch.Tensor):
    """sharded_argmax_fused(logits_shard, index_base, exchange, out) as a callable that launches on the stream
    current NOW with every pointer fixed: for a decode loop that calls the same buffers every step, where the
    interpreter's per-call work (checks, pointer and stream look-ups) would otherwise cost more than the 10 us
    kernel.  The tensors must stay alive and in place; `out` receives the ids."""
    _ops._logits_req(logits_shard, "bind_argmax_fused")
    rows, width = logits_shard.shape
    ws = _ops.argmax_workspace(logits_shard.device, rows)
    import ctypes as C
    call = _bound(_lib.load().b2_argmax_rows_sharded,
                  (logits_shard.data_ptr(), rows, width, width, _ops._code(logits_shard), index_base, out.data_ptr(),
                   ws.data_ptr(), C.addressof(exchange.desc), exchange.status.data_ptr(), _ops._stream()))
    call.keepalive = (logits_shard, out, ws, exchange)
    return call


def bind_softmax_fused(logits_shard: torch.Tensor, exchange: PeerExchange, out: torch.Tensor, stats: torch.Tensor):
    """sharded_softmax_fused with every pointer fixed (see bind_argmax_fused): two launches per call."""
    _ops._logits_req(logits_shard, "bind_softmax_fused")
    rows, width = logits_shard.shape
    L = _lib.load()
    code = _ops._code(logits_shard)
    import ctypes as C
    first = _bound(L.b2_softmax_stats_sharded, (logits_shard.data_ptr(), rows, width, code, stats[0].data_ptr(),
                                               stats[1].data_ptr(), C.addressof(exchange.desc), exchange.status.data_ptr(),
                                               _ops._stream()))
    second = _bound(L.b2_softmax_apply, (logits_shard.data_ptr(), out.data_ptr(), rows, width, code, stats[0].data_ptr(),
                                         stats[1].data_ptr(), _ops._stream()))

    def call():
        first()
        second()
    call.keepalive = (logits_shard, out, stats, exchange)
    return call
