"""Operator functions with the reference's names and argument rules, over torch tensors.

Each ``cuda_*`` function mirrors one declaration of the reference's
include/llm/ops_cuda.h (lines given per function): same argument meaning, same
rejections (``ValueError`` stands for the reference's ``std::invalid_argument``).
torch is plumbing here: it owns device memory and streams; all arithmetic happens
in the sm_100a kernels behind the C ABI (include/b2ops.h).  Kernels are enqueued
on torch's current stream.

The ``*_out`` forms write caller-provided tensors (which may alias an input, as the
reference's callers do) and allocate nothing; the allocating forms make exactly the
output tensor.
"""
from __future__ import annotations

import contextlib
import threading
from typing import Optional, Sequence

import torch

from . import lib as _lib

_state = threading.local()


def _mode() -> int:
    return getattr(_state, "mode", _lib.FAST)


@contextlib.contextmanager
def reduction_mode(name: str):
    """Thread-local switch between "fast" and "deterministic" reductions (the idiom of
    the reference's CudaLinearModeGuard / CudaAttentionModeGuard, include/llm/ops_cuda.h:18-38)."""
    value = {"fast": _lib.FAST, "deterministic": _lib.DETERMINISTIC}[name]
    previous = _mode()
    _state.mode = value
    try:
        yield
    finally:
        _state.mode = previous


# ---------------------------------------------------------------- validation helpers
# reference src/ops_cuda.cu:62-73 (req, rank, same_dtype, output_req)

def _req(t: torch.Tensor, op: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{op}: requires contiguous CUDA tensor")
    if t.dtype not in (torch.float32, torch.float16):
        raise ValueError(f"{op}: supports only F32/F16")


def _same_dtype(op: str, *ts: torch.Tensor) -> None:
    if any(t.dtype != ts[0].dtype for t in ts):
        raise ValueError(f"{op}: all input dtypes must match; actual " + ", ".join(str(t.dtype) for t in ts))


def _output_req(out: torch.Tensor, shape, dtype, op: str) -> None:
    if (not isinstance(out, torch.Tensor) or not out.is_cuda or out.dtype != dtype or not out.is_contiguous()
            or tuple(out.shape) != tuple(shape)):
        raise ValueError(f"{op}: output must be CUDA/{dtype}/contiguous shape with the expected dimensions")


def _code(t: torch.Tensor) -> int:
    return _lib.F32 if t.dtype == torch.float32 else _lib.F16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _positions_device(positions: torch.Tensor, need: int, op: str, exact: bool) -> None:
    # int32 positions; the reference carries them in I32 tensors for the *_positions_out forms
    # (src/ops_cuda.cu:978,1090) and in F32-typed buffers holding int32 bits for
    # cuda_rope_batched_out (:709).  Both arrive here as 4-byte-element CUDA tensors.
    if (not isinstance(positions, torch.Tensor) or not positions.is_cuda or not positions.is_contiguous()
            or positions.dtype not in (torch.int32, torch.float32)):
        raise ValueError(f"{op}: positions must be a contiguous CUDA tensor of int32 values")
    if (exact and tuple(positions.shape) != (need,)) or positions.numel() < need:
        raise ValueError(f"{op}: positions length mismatch")


# ---------------------------------------------------------------- RMSNorm family

def cuda_rms_norm_out(x, weight, eps: float, out, mode: Optional[str] = None) -> None:
    """include/llm/ops_cuda.h:113-114.  Norm over the last dimension of any rank >= 1."""
    op = "cuda_rms_norm"
    _req(x, op); _req(weight, op); _same_dtype(op, x, weight)
    if weight.dim() != 1:
        raise ValueError(f"{op}: unexpected rank")
    if x.dim() < 1 or x.shape[-1] != weight.shape[0] or not eps > 0:
        raise ValueError(f"{op}: incompatible shape/epsilon")
    _output_req(out, x.shape, x.dtype, op)
    hidden = x.shape[-1]
    rows = x.numel() // hidden if hidden else 0
    m = _mode() if mode is None else {"fast": 0, "deterministic": 1}[mode]
    _lib.check(_lib.load().b2_rms_norm(_ptr(x), _ptr(weight), _ptr(out), rows, hidden, eps, _code(x), m, _stream()))


def cuda_rms_norm(x, weight, eps: float, mode: Optional[str] = None):
    """include/llm/ops_cuda.h:77."""
    _req(x, "cuda_rms_norm")
    out = torch.empty_like(x)
    cuda_rms_norm_out(x, weight, eps, out, mode)
    return out


def cuda_add_rms_norm_out(lhs, rhs, weight, eps: float, residual, normalized, mode: Optional[str] = None) -> None:
    """include/llm/ops_cuda.h:117-120.  residual = lhs + rhs; normalized = RMSNorm(residual) * weight."""
    op = "cuda_add_rms_norm"
    _req(lhs, op); _req(rhs, op); _req(weight, op)
    _same_dtype(op, lhs, rhs); _same_dtype(op, lhs, weight)
    if weight.dim() != 1:
        raise ValueError(f"{op}: unexpected rank")
    if lhs.shape != rhs.shape or lhs.dim() == 0 or lhs.shape[-1] != weight.shape[0] or not eps > 0:
        raise ValueError(f"{op}: incompatible shapes/epsilon")
    _output_req(residual, lhs.shape, lhs.dtype, op)
    _output_req(normalized, lhs.shape, lhs.dtype, op)
    hidden = lhs.shape[-1]
    rows = lhs.numel() // hidden if hidden else 0
    m = _mode() if mode is None else {"fast": 0, "deterministic": 1}[mode]
    _lib.check(_lib.load().b2_add_rms_norm(_ptr(lhs), _ptr(rhs), _ptr(weight), _ptr(residual), _ptr(normalized),
                                           rows, hidden, eps, _code(lhs), m, _stream()))


# ---------------------------------------------------------------- elementwise

def cuda_add_out(a, b, out) -> None:
    """include/llm/ops_cuda.h:115-116."""
    op = "cuda_add"
    _req(a, op); _req(b, op); _same_dtype(op, a, b)
    if a.shape != b.shape:
        raise ValueError(f"{op}: shapes must match")
    _output_req(out, a.shape, a.dtype, op)
    _lib.check(_lib.load().b2_add(_ptr(a), _ptr(b), _ptr(out), a.numel(), _code(a), _stream()))


def cuda_add(a, b):
    """include/llm/ops_cuda.h:78."""
    _req(a, "cuda_add")
    out = torch.empty_like(a)
    cuda_add_out(a, b, out)
    return out


def cuda_swiglu_out(gate, up, out, mode: Optional[str] = None) -> None:
    """include/llm/ops_cuda.h:121-122.  out may alias gate (src/qwen3_layer_cuda.cu:323)."""
    op = "cuda_swiglu"
    _req(gate, op); _req(up, op); _same_dtype(op, gate, up)
    if gate.shape != up.shape:
        raise ValueError(f"{op}: shapes must match")
    _output_req(out, gate.shape, gate.dtype, op)
    m = _mode() if mode is None else {"fast": 0, "deterministic": 1}[mode]
    _lib.check(_lib.load().b2_swiglu(_ptr(gate), _ptr(up), _ptr(out), gate.numel(), _code(gate), m, _stream()))


def cuda_swiglu(gate, up, mode: Optional[str] = None):
    """include/llm/ops_cuda.h:79."""
    _req(gate, "cuda_swiglu")
    out = torch.empty_like(gate)
    cuda_swiglu_out(gate, up, out, mode)
    return out


# ---------------------------------------------------------------- rotary embedding

_rope_status_words = {}


def rope_status_word(device) -> torch.Tensor:
    """The int32 device word that the rotary-embedding calls of this module hand to the C ABI as `status` (one per
    device, created zeroed).  Bit 0 set: a bounded wait inside a kernel ran out and some call's output is incomplete."""
    key = torch.device(device).index
    w = _rope_status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _rope_status_words[key] = w
    return w


def rope_status(device) -> int:
    """Blocking read of rope_status_word(device): 0 in a healthy run."""
    return int(rope_status_word(device).item())


def _rope_call(x, positions, theta, out, mode, batched_seq=None):
    m = _mode() if mode is None else {"fast": 0, "deterministic": 1}[mode]
    L = _lib.load()
    status = rope_status_word(x.device).data_ptr()
    if batched_seq is None:
        t, h, d = x.shape
        _lib.check(L.b2_rope(_ptr(x), _ptr(positions), _ptr(out), t, h, d, theta, _code(x), m, status, _stream()))
    else:
        b, s, h, d = x.shape
        _lib.check(L.b2_rope_batched(_ptr(x), _ptr(positions), _ptr(out), b, s, h, d, theta, _code(x), m, status, _stream()))


def cuda_rope(x, positions: Sequence[int], theta: float, mode: Optional[str] = None):
    """include/llm/ops_cuda.h:80.  x [T,H,D], host positions of length T (copied to the device per call,
    as the reference does, src/ops_cuda.cu:707)."""
    op = "cuda_rope"
    _req(x, op)
    if x.dim() != 3:
        raise ValueError(f"{op}: unexpected rank")
    t, h, d = x.shape
    if t == 0 or h == 0 or d == 0 or d % 2 or len(positions) == 0 or len(positions) != t or not theta > 0:
        raise ValueError(f"{op}: invalid or empty shape/positions/theta")
    pos = torch.tensor(list(positions), dtype=torch.int32).to(x.device)
    out = torch.empty_like(x)
    _rope_call(x, pos, theta, out, mode)
    return out


def cuda_rope_batched(x, positions: Sequence[int], theta: float, mode: Optional[str] = None):
    """include/llm/ops_cuda.h:81.  x [B,S,H,D], host positions of length S shared over the batch."""
    op = "cuda_rope_batched"
    _req(x, op)
    if x.dim() != 4:
        raise ValueError(f"{op}: unexpected rank")
    b, s, h, d = x.shape
    if b == 0 or s == 0 or h == 0 or d == 0 or d % 2 or len(positions) != s or not theta > 0:
        raise ValueError(f"{op}: invalid shape/positions/theta")
    pos = torch.tensor(list(positions), dtype=torch.int32).to(x.device)
    out = torch.empty_like(x)
    _rope_call(x, pos, theta, out, mode, batched_seq=s)
    return out


def cuda_rope_batched_out(x, positions_device, theta: float, out, mode: Optional[str] = None) -> None:
    """include/llm/ops_cuda.h:123-125.  positions_device holds at least S int32 values."""
    op = "cuda_rope_batched"
    _req(x, op)
    if x.dim() != 4:
        raise ValueError(f"{op}: unexpected rank")
    b, s, h, d = x.shape
    if b == 0 or s == 0 or h == 0 or d == 0 or d % 2 or not theta > 0:
        raise ValueError(f"{op}: invalid shape/theta")
    _positions_device(positions_device, s, op, exact=False)
    _output_req(out, x.shape, x.dtype, op)
    _rope_call(x, positions_device, theta, out, mode, batched_seq=s)


def cuda_rope_token_positions_out(x, positions_device, theta: float, out, mode: Optional[str] = None) -> None:
    """include/llm/ops_cuda.h:129-131 (and :126-128, cuda_rope_batched_positions_out, which has the same
    contract without a stream).  x [T,H,D] with one int32 position per row [T].  The reference restricts
    this entry to fp16, H in {16, 8} and D = 128 (src/ops_cuda.cu:1083-1093); any even D and any H are
    accepted here."""
    op = "cuda_rope_token_positions"
    _req(x, op)
    if x.dim() != 3 or x.shape[0] <= 0 or x.shape[2] % 2 or not theta > 0:
        raise ValueError(f"{op}: expected CUDA [T,H,D] with even D, and CUDA/I32 positions [T]")
    _positions_device(positions_device, x.shape[0], op, exact=True)
    _output_req(out, x.shape, x.dtype, op)
    _rope_call(x, positions_device, theta, out, mode)


cuda_rope_batched_positions_out = cuda_rope_token_positions_out


def qk_norm_rope_out(q, k, q_weight, k_weight, positions_device, eps: float, theta: float, q_out, k_out) -> None:
    """Fused per-head RMSNorm + RoPE of the query and key projections (no single reference counterpart:
    it stands for cuda_rms_norm_out x2 + cuda_rope_token_positions_out x2, src/qwen3_layer_cuda.cu:289-292).
    q [T,Hq,D], k [T,Hk,D] or None."""
    op = "qk_norm_rope"
    _req(q, op); _req(q_weight, op); _same_dtype(op, q, q_weight)
    if q.dim() != 3 or q.shape[2] % 2 or q_weight.shape != (q.shape[2],) or not eps > 0 or not theta > 0:
        raise ValueError(f"{op}: expected q [T,H,D] with even D, weight [D], eps > 0, theta > 0")
    _positions_device(positions_device, q.shape[0], op, exact=True)
    _output_req(q_out, q.shape, q.dtype, op)
    k_heads = 0
    if k is not None:
        _req(k, op); _req(k_weight, op); _same_dtype(op, q, k, k_weight)
        if k.dim() != 3 or k.shape[0] != q.shape[0] or k.shape[2] != q.shape[2] or k_weight.shape != q_weight.shape:
            raise ValueError(f"{op}: k must be [T,Hk,D] with the same T and D as q")
        _output_req(k_out, k.shape, k.dtype, op)
        k_heads = k.shape[1]
    t, hq, d = q.shape
    _lib.check(_lib.load().b2_qk_norm_rope(_ptr(q), _ptr(k), _ptr(q_weight), _ptr(k_weight), _ptr(positions_device),
                                           _ptr(q_out), _ptr(k_out), t, hq, k_heads, d, eps, theta, _code(q),
                                           rope_status_word(q.device).data_ptr(), _stream()))


# ---------------------------------------------------------------- embedding gather

def cuda_embedding_lookup_device_ids_out(weight, ids_device, out, status: Optional[torch.Tensor] = None) -> None:
    """include/llm/ops_cuda.h:151-153.  ids_device: rank-1 CUDA tensor of int32 values (the reference types
    it F32 and reinterprets the bits, src/ops_cuda.cu:875).  Unlike the reference, an out-of-range id is not
    dereferenced: its row becomes zeros and bit 0 of `status` (int32[1], zeroed by the caller) is set."""
    op = "cuda_embedding_lookup_device_ids"
    _req(weight, op)
    if weight.dim() != 2:
        raise ValueError(f"{op}: unexpected rank")
    if (not isinstance(ids_device, torch.Tensor) or not ids_device.is_cuda or not ids_device.is_contiguous()
            or ids_device.dtype not in (torch.int32, torch.float32) or ids_device.dim() != 1
            or ids_device.shape[0] <= 0):
        raise ValueError(f"{op}: ids must be CUDA/contiguous rank-1 int32 values")
    vocab, hidden = weight.shape
    _output_req(out, (ids_device.shape[0], hidden), weight.dtype, op)
    _lib.check(_lib.load().b2_embedding_gather(_ptr(weight), _ptr(ids_device), _ptr(out), ids_device.shape[0], hidden,
                                               vocab, _code(weight), _ptr(status), _stream()))


def cuda_embedding_lookup_out(weight, ids: Sequence[int], ids_device, out) -> None:
    """include/llm/ops_cuda.h:148-150.  Host ids are bounds-checked on the host, copied into the caller's
    `ids_device` scratch (numel >= len(ids)), then gathered."""
    op = "cuda_embedding_lookup"
    _req(weight, op)
    if weight.dim() != 2:
        raise ValueError(f"{op}: unexpected rank")
    if len(ids) == 0:
        raise ValueError(f"{op}: token_ids must be non-empty")
    vocab, hidden = weight.shape
    if vocab <= 0 or hidden <= 0:
        raise ValueError(f"{op}: weight shape must be positive")
    if any(i < 0 or i >= vocab for i in ids):
        raise ValueError(f"{op}: token id out of range")
    if (not isinstance(ids_device, torch.Tensor) or not ids_device.is_cuda or not ids_device.is_contiguous()
            or ids_device.dtype not in (torch.int32, torch.float32) or ids_device.numel() < len(ids)):
        raise ValueError(f"{op}: token storage must be CUDA/contiguous with room for the ids")
    _output_req(out, (len(ids), hidden), weight.dtype, op)
    staged = ids_device.view(torch.int32).reshape(-1)[:len(ids)]
    staged.copy_(torch.tensor(list(ids), dtype=torch.int32))
    _lib.check(_lib.load().b2_embedding_gather(_ptr(weight), _ptr(staged), _ptr(out), len(ids), hidden, vocab,
                                               _code(weight), None, _stream()))


def cuda_embedding_lookup(weight, ids: Sequence[int]):
    """include/llm/ops_cuda.h:155-156."""
    op = "cuda_embedding_lookup"
    _req(weight, op)
    if weight.dim() != 2:
        raise ValueError(f"{op}: unexpected rank")
    if len(ids) == 0:
        raise ValueError(f"{op}: token_ids must be non-empty")
    ids_device = torch.empty(len(ids), dtype=torch.int32, device=weight.device)
    out = torch.empty((len(ids), weight.shape[1]), dtype=weight.dtype, device=weight.device)
    cuda_embedding_lookup_out(weight, ids, ids_device, out)
    return out


# ---------------------------------------------------------------- vocabulary-wide reductions

_workspaces = {}


def argmax_workspace(device, rows: int) -> torch.Tensor:
    """Zero-filled scratch for the argmax kernels, cached per device and grown on demand.
    Every call leaves it zero-filled, so it is shared by all later calls on that device."""
    key = (torch.device(device).index, "argmax")
    need = _lib.load().b2_argmax_workspace_bytes(rows)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 4096), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def softmax_workspace(device, rows: int) -> torch.Tensor:
    key = (torch.device(device).index, "softmax")
    need = _lib.load().b2_softmax_workspace_bytes(rows)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 4096), dtype=torch.uint8, device=device)   # the trailing status word starts clear
        _workspaces[key] = ws
    return ws


def softmax_status(device, rows: int) -> int:
    """Status word of the softmax workspace used for `rows` rows (0 = every bulk copy completed)."""
    ws = softmax_workspace(device, rows)
    need = _lib.load().b2_softmax_workspace_bytes(rows)
    return int(ws[need - 16:need - 12].view(torch.int32).item())


def _logits_req(logits, op):
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda or not logits.is_contiguous():
        raise ValueError(f"{op}: requires contiguous CUDA tensor")
    if logits.dtype not in (torch.float32, torch.float16):
        raise ValueError(f"{op}: supports only F32/F16")
    if logits.dim() != 2:
        raise ValueError(f"{op}: unexpected rank")
    if logits.shape[0] <= 0 or logits.shape[1] <= 0:
        raise ValueError(f"{op}: shape dimensions must be > 0")


def argmax_rows_out(logits, out_ids) -> None:
    """Row-wise argmax of [R,V] logits into int32[R] on the device; no host round trip.
    (The reference reaches rows other than the last only through CudaSampler::sample_row,
    src/ops_cuda.cu:961-971, one blocking call per row.)"""
    op = "argmax_rows"
    _logits_req(logits, op)
    rows, width = logits.shape
    if not out_ids.is_cuda or out_ids.dtype != torch.int32 or tuple(out_ids.shape) != (rows,):
        raise ValueError(f"{op}: output must be CUDA int32 [rows]")
    ws = argmax_workspace(logits.device, rows)
    _lib.check(_lib.load().b2_argmax_rows(_ptr(logits), rows, width, width, _code(logits), _ptr(out_ids), _ptr(ws),
                                          _stream()))


def argmax_rows(logits):
    _logits_req(logits, "argmax_rows")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    argmax_rows_out(logits, out)
    return out


def cuda_argmax_last_row(logits) -> int:
    """include/llm/ops_cuda.h:154.  Argmax of the last row, returned to the host (blocking, like the reference)."""
    op = "cuda_argmax_last_row"
    _logits_req(logits, op)
    out = torch.empty(1, dtype=torch.int32, device=logits.device)
    argmax_rows_out(logits[-1:], out)
    return int(out.item())


def lm_head_argmax(hidden, table, logits_out=None, mode: Optional[str] = None, want_ids: bool = True,
                   keys_out=None, index_base: int = 0, ids_out=None):
    """Decode-size LM head fused with the greedy pick (b2_lm_head_argmax): int32[rows] arg-max of
    hidden[rows, H] x table[V, H]^T in one pass over the table.  ``logits_out`` ([rows, V], same dtype)
    also receives the logits, as cuda_lm_head (include/llm/ops_cuda.h:157; src/ops_cuda.cu:885) would
    return them; ``keys_out`` (int64[rows]) receives the packed keys of a vocabulary-sharded table whose
    first row has global index ``index_base``; with ``ids_out`` (int32[rows]) given nothing is allocated, so
    the call can be recorded into a CUDA graph.  Replaces cuda_lm_head + cuda_argmax_last_row
    (src/qwen3_cuda_model.cpp:1070-1071,1339) for decode batches."""
    op = "lm_head_argmax"
    _req(hidden, op)
    _req(table, op)
    _same_dtype(op, hidden, table)
    if hidden.dim() != 2 or table.dim() != 2:
        raise ValueError(f"{op}: hidden and embedding must be rank-2")
    if hidden.shape[1] != table.shape[1]:
        raise ValueError(f"{op}: hidden_size mismatch")
    rows, hsz = hidden.shape
    vocab = table.shape[0]
    stride = vocab
    if logits_out is not None:
        _output_req(logits_out, (rows, vocab), hidden.dtype, op)
    if keys_out is not None and (not keys_out.is_cuda or keys_out.dtype != torch.int64 or tuple(keys_out.shape) != (rows,)):
        raise ValueError(f"{op}: keys must be CUDA int64 [rows]")
    if ids_out is not None and (not ids_out.is_cuda or ids_out.dtype != torch.int32 or tuple(ids_out.shape) != (rows,)):
        raise ValueError(f"{op}: ids must be CUDA int32 [rows]")
    ids = ids_out if ids_out is not None else (torch.empty(rows, dtype=torch.int32, device=hidden.device) if want_ids else None)
    m = _mode() if mode is None else {"fast": 0, "deterministic": 1}[mode]
    ws = argmax_workspace(hidden.device, max(rows, 1))
    _lib.check(_lib.load().b2_lm_head_argmax(_ptr(hidden), _ptr(table), rows, hsz, vocab, _code(hidden), m, index_base,
                                             _ptr(logits_out), stride, _ptr(ids), _ptr(keys_out), _ptr(ws), _stream()))
    return ids


def cuda_softmax_last_dim(x, mode: Optional[str] = None):
    """include/llm/ops_cuda.h:82.  Softmax over the last dimension of any rank >= 1."""
    op = "cuda_softmax_last_dim"
    _req(x, op)
    if x.dim() == 0 or x.shape[-1] <= 0:
        raise ValueError(f"{op}: invalid last dimension")
    out = torch.empty_like(x)
    width = x.shape[-1]
    rows = x.numel() // width
    m = _mode() if mode is None else {"fast": 0, "deterministic": 1}[mode]
    ws = softmax_workspace(x.device, rows)
    _lib.check(_lib.load().b2_softmax_rows(_ptr(x), _ptr(out), rows, width, _code(x), m, _ptr(ws), _stream()))
    return out


# ---------------------------------------------------------------- sampling

import dataclasses
import math


@dataclasses.dataclass
class SamplingConfig:
    """include/llm/ops_cuda.h:46-51."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0


def sample_rows_out(logits, config: SamplingConfig, draw_offsets, out_ids, workspace=None) -> None:
    """One token per row of [R,V] logits into int32[R] on the device, all rows in one call and no host
    round trip (b2_sample_rows).  draw_offsets: CUDA int64 [R] (the bits are read as uint64), or None."""
    op = "sample_rows"
    _logits_req(logits, op)
    rows, width = logits.shape
    if not out_ids.is_cuda or out_ids.dtype != torch.int32 or tuple(out_ids.shape) != (rows,):
        raise ValueError(f"{op}: output must be CUDA int32 [rows]")
    if draw_offsets is not None and (not draw_offsets.is_cuda or draw_offsets.dtype != torch.int64
                                     or tuple(draw_offsets.shape) != (rows,)):
        raise ValueError(f"{op}: draw_offsets must be CUDA int64 [rows]")
    L = _lib.load()
    need = L.b2_sampler_workspace_bytes(rows, width)
    if workspace is None:
        key = (torch.device(logits.device).index, "sampler")
        workspace = _workspaces.get(key)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=logits.device)
            _workspaces[key] = workspace
    elif workspace.numel() < need:
        raise ValueError(f"{op}: workspace too small")
    _lib.check(L.b2_sample_rows(_ptr(logits), rows, width, width, _code(logits), float(config.temperature),
                                int(config.top_k), float(config.top_p), int(config.seed) & 0xFFFFFFFFFFFFFFFF,
                                _ptr(draw_offsets), _ptr(out_ids), _ptr(workspace), _stream()))


class CudaSampler:
    """include/llm/ops_cuda.h:53-74: the reference's sampler interface, one token per blocking call,
    with its argument rules (src/ops_cuda.cu:886-971)."""

    def __init__(self, max_vocab: int):
        if max_vocab <= 0:
            raise ValueError("CudaSampler: max_vocab must be > 0")
        self.max_vocab = int(max_vocab)

    def _sample(self, row, config: SamplingConfig, draw_offset: int, op: str) -> int:
        vocab = row.shape[-1]
        if vocab > self.max_vocab:
            raise ValueError(f"{op}: vocab exceeds sampler capacity")
        if not math.isfinite(config.temperature) or config.temperature < 0:
            raise ValueError(f"{op}: temperature must be finite and >= 0")
        if config.temperature > 0:
            if config.top_k < 0 or config.top_k > vocab:
                raise ValueError(f"{op}: top_k must be in [0,vocab]")
            if not math.isfinite(config.top_p) or config.top_p <= 0 or config.top_p > 1:
                raise ValueError(f"{op}: top_p must be finite in (0,1]")
        out = torch.empty(1, dtype=torch.int32, device=row.device)
        offsets = torch.tensor([draw_offset & 0x7FFFFFFFFFFFFFFF if draw_offset < (1 << 63) else draw_offset - (1 << 64)],
                               dtype=torch.int64, device=row.device)
        sample_rows_out(row, config, offsets, out)
        return int(out.item())

    @staticmethod
    def _check(logits, op, ranks):
        if not isinstance(logits, torch.Tensor) or not logits.is_cuda or not logits.is_contiguous():
            raise ValueError(f"{op}: requires contiguous CUDA tensor")
        if logits.dtype not in (torch.float32, torch.float16):
            raise ValueError(f"{op}: supports F32/F16 only")
        if logits.dim() not in ranks or logits.numel() == 0:
            raise ValueError(f"{op}: requires non-empty rank-{'/'.join(map(str, ranks))} logits")

    def sample_last_row(self, logits, config: SamplingConfig, draw_offset: int) -> int:
        op = "CudaSampler::sample_last_row"
        self._check(logits, op, (2,))
        return self._sample(logits[-1:], config, draw_offset, op)

    def sample_row(self, logits_bv, batch_index: int, config: SamplingConfig, draw_offset: int) -> int:
        op = "CudaSampler::sample_row"
        self._check(logits_bv, op, (2,))
        if not 0 <= batch_index < logits_bv.shape[0]:
            raise IndexError(f"{op}: batch_index out of range")
        return self._sample(logits_bv[batch_index:batch_index + 1], config, draw_offset, op)

    def sample_last_token_of_batch(self, logits_bsv, batch_index: int, config: SamplingConfig, draw_offset: int) -> int:
        op = "CudaSampler::sample_last_token_of_batch"
        self._check(logits_bsv, op, (3,))
        if not 0 <= batch_index < logits_bsv.shape[0]:
            raise IndexError(f"{op}: batch_index out of range")
        return self._sample(logits_bsv[batch_index, -1:], config, draw_offset, op)


# ---------------------------------------------------------------- paged KV cache writes, last-valid-row gather

def _pool_args(storage, key, value, op):
    for t in (storage, key, value):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{op}: requires contiguous CUDA tensors")
    if storage.dim() != 6 or storage.shape[2] != 2:
        raise ValueError(f"{op}: storage must be [layers, total_blocks, 2, block_size, kv_heads, head_dim]")
    if key.dtype != storage.dtype or value.dtype != storage.dtype or key.dtype not in (torch.float16, torch.float32):
        raise ValueError(f"{op}: key, value and storage must share one dtype, F16 or F32")
    if key.shape != value.shape or key.dim() != 3 or tuple(key.shape[1:]) != tuple(storage.shape[4:]):
        raise ValueError(f"{op}: key/value must be [tokens, kv_heads, head_dim] of the pool")
    return tuple(int(d) for d in storage.shape)


def _i32_device(t, shape, op, what):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.int32 or not t.is_contiguous() \
            or (shape is not None and tuple(t.shape) != tuple(shape)):
        raise ValueError(f"{op}: {what} must be CUDA/I32/contiguous" + (f" {list(shape)}" if shape else ""))


def paged_kv_write_decode_batch(key_bhd, value_bhd, storage, layer: int, block_tables_bm, positions_b, status=None) -> None:
    """cuda_paged_kv_write_decode_batch (include/llm/ops_cuda.h:183-186) on the pool's storage tensor."""
    op = "paged_kv_write_decode_batch"
    layers, total_blocks, _, block_size, kv_heads, head_dim = _pool_args(storage, key_bhd, value_bhd, op)
    batch = key_bhd.shape[0]
    if block_tables_bm.dim() != 2:
        raise ValueError(f"{op}: block tables must be CUDA/I32/contiguous [B,max_blocks]")
    _i32_device(block_tables_bm, (batch, block_tables_bm.shape[1]), op, "block tables")
    _i32_device(positions_b, (batch,), op, "positions")
    if not 0 <= layer < layers:
        raise ValueError(f"{op}: invalid KV cache dimensions")
    _lib.check(_lib.load().b2_paged_kv_write_decode_batch(_ptr(key_bhd), _ptr(value_bhd), _ptr(storage), _ptr(block_tables_bm),
                                                          _ptr(positions_b), batch, block_tables_bm.shape[1], layer, layers,
                                                          total_blocks, block_size, kv_heads, head_dim, _code(key_bhd),
                                                          _ptr(status), _stream()))


def paged_kv_write_decode(key_hd, value_hd, storage, layer: int, block_table, cache_length, status=None) -> None:
    """cuda_paged_kv_write_decode (include/llm/ops_cuda.h:178-182): one token at position *cache_length - 1."""
    op = "paged_kv_write_decode"
    layers, total_blocks, _, block_size, kv_heads, head_dim = _pool_args(storage, key_hd[None], value_hd[None], op)
    _i32_device(block_table, None, op, "device block table")
    _i32_device(cache_length, (1,), op, "device cache length")
    if block_table.dim() != 1 or block_table.numel() == 0 or not 0 <= layer < layers:
        raise ValueError(f"{op}: invalid block table or layer")
    _lib.check(_lib.load().b2_paged_kv_write_decode(_ptr(key_hd), _ptr(value_hd), _ptr(storage), _ptr(block_table),
                                                    _ptr(cache_length), block_table.numel(), layer, layers, total_blocks,
                                                    block_size, kv_heads, head_dim, _code(key_hd), _ptr(status), _stream()))


def paged_kv_prefill_copy_packed(key_thd, value_thd, storage, block_table, layer: int, status=None) -> None:
    """cuda_paged_kv_prefill_copy_packed (reference src/ops_cuda.cu:1123-1160): token t to slot t of one block table."""
    op = "paged_kv_prefill_copy_packed"
    layers, total_blocks, _, block_size, kv_heads, head_dim = _pool_args(storage, key_thd, value_thd, op)
    tokens = key_thd.shape[0]
    _i32_device(block_table, None, op, "block table")
    if tokens == 0 or block_table.numel() < (tokens + block_size - 1) // block_size or not 0 <= layer < layers:
        raise ValueError(f"{op}: invalid CUDA/F16 packed KV or pool metadata")
    _lib.check(_lib.load().b2_paged_kv_prefill_copy(_ptr(key_thd), _ptr(value_thd), _ptr(storage), _ptr(block_table), tokens,
                                                    block_table.numel(), layer, layers, total_blocks, block_size, kv_heads,
                                                    head_dim, _code(key_thd), _ptr(status), _stream()))


def select_last_valid_logits(padded_logits, valid_lengths: Sequence[int]):
    """select_last_valid_logits (include/llm/qwen3_padded_prefill.h:43; src/qwen3_padded_prefill.cpp:118-148), CUDA
    branch: [B,S,V] -> [B,V], the row of each prompt's last real token, in one launch."""
    op = "select_last_valid_logits"
    if not isinstance(padded_logits, torch.Tensor) or not padded_logits.is_cuda or not padded_logits.is_contiguous() \
            or padded_logits.dim() != 3:
        raise ValueError(f"{op}: padded logits must be contiguous rank-3 [B,S,V]")
    if padded_logits.dtype not in (torch.float32, torch.float16):
        raise ValueError(f"{op}: supports only F32/F16")
    batch, seq, vocab = padded_logits.shape
    if batch == 0 or seq == 0 or vocab == 0 or len(valid_lengths) != batch:
        raise ValueError(f"{op}: invalid padded logits shape or valid_lengths size")
    if any(n <= 0 or n > seq for n in valid_lengths):
        raise ValueError(f"{op}: valid length is outside padded logits sequence")
    lengths = torch.tensor(list(valid_lengths), dtype=torch.int32).to(padded_logits.device, non_blocking=True)
    out = torch.empty(batch, vocab, dtype=padded_logits.dtype, device=padded_logits.device)
    _lib.check(_lib.load().b2_select_last_valid_rows(_ptr(padded_logits), _ptr(lengths), _ptr(out), batch, seq, vocab,
                                                     _code(padded_logits), None, _stream()))
    return out


def qk_norm_rope_paged_out(q, k, v, q_weight, k_weight, positions_device, eps: float, theta: float, q_out, storage, layer: int,
                           block_tables, slot_positions=None, tokens_per_table: int = 1, status=None) -> None:
    """b2_qk_norm_rope_paged: per-head RMSNorm + RoPE of q and k in one launch, the rotated keys and the values
    written straight into the paged KV pool.  Decode batch: block_tables [B, max_blocks], slot_positions =
    positions_device, tokens_per_table = 1.  One packed sequence: block_tables [max_blocks], slot_positions None,
    tokens_per_table = tokens.  Raises lib.B2Error (status -3) for shapes only the scalar kernels take."""
    op = "qk_norm_rope_paged"
    layers, total_blocks, _, block_size, kv_heads, head_dim = _pool_args(storage, k, v, op)
    _req(q, op)
    _same_dtype(op, q, k, q_weight, k_weight)
    if q.dim() != 3 or q.shape[0] != k.shape[0] or q.shape[2] != head_dim:
        raise ValueError(f"{op}: q must be [tokens, q_heads, head_dim] with the pool's head_dim")
    if tuple(q_weight.shape) != (head_dim,) or tuple(k_weight.shape) != (head_dim,) or not (eps > 0) or not (theta > 0):
        raise ValueError(f"{op}: incompatible shape/epsilon/theta")
    _output_req(q_out, q.shape, q.dtype, op)
    tokens = q.shape[0]
    _positions_device(positions_device, tokens, op, exact=True)
    _i32_device(block_tables, None, op, "block tables")
    if slot_positions is not None:
        _i32_device(slot_positions, (tokens,), op, "slot positions")
    max_blocks = block_tables.shape[-1]
    rows_needed = -(-tokens // tokens_per_table)
    if block_tables.numel() < rows_needed * max_blocks or not 0 <= layer < layers or tokens_per_table < 1:
        raise ValueError(f"{op}: invalid block tables or layer")
    _lib.check(_lib.load().b2_qk_norm_rope_paged(_ptr(q), _ptr(k), _ptr(v), _ptr(q_weight), _ptr(k_weight), _ptr(positions_device),
                                                 _ptr(q_out), _ptr(storage), _ptr(block_tables), _ptr(slot_positions), tokens,
                                                 q.shape[1], kv_heads, head_dim, eps, theta, tokens_per_table, max_blocks, layer,
                                                 layers, total_blocks, block_size, _code(q), _ptr(status), _stream()))
