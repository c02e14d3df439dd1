"""ctypes doors into the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the bench's CPU-baseline leg may import this
package; the product (the CUDA library and its host side) never does.

``port``  -> oracle/liboracle.so, the C restatement in oracle.c
``ref``   -> oracle/_ref/liboracle_ref.so, the reference's own compiled CPU
             operators (present when oracle/Makefile's ``ref`` target was built
             where the reference tree exists; the binary then travels with the
             snapshot).  ``ref`` is None when that binary is absent.
``ref_cuda`` -> oracle/_ref/libref_cuda.so, the reference's own CUDA operators
             recompiled for sm_100a (``refcuda`` target): a second oracle for the
             deterministic mode and the "reference kernels on the same GPU" timings.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
F32, F16 = 0, 1  # dtype codes, the same as the product's C ABI


def reference_tree():
    """Root of the reference's source tree, or None: $REFERENCE when set, else a directory named
    ``reference`` beside this repository."""
    path = os.environ.get("REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return path if os.path.isfile(os.path.join(path, "src", "ops_cpu.cpp")) else None


def build(ref: bool = True) -> None:
    """Compile oracle.c and, when ``ref`` is set and the reference's source tree is found (reference_tree()),
    the reference-backed libraries under _ref/.  Prebuilt files under _ref/ are kept otherwise."""
    tree = reference_tree() if ref else None
    targets = ["all"] + (["ref", "refcuda", "layer", "REFERENCE=" + tree] if tree else [])
    subprocess.run(["make", "-C", _HERE] + targets, check=True, stdout=subprocess.DEVNULL)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


class Port:
    """The C restatement (oracle.c)."""

    def __init__(self):
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(ref=False)
        self.lib = C.CDLL(path)
        L = self.lib
        L.orc_decode_f16.restype = C.c_float
        L.orc_decode_f16.argtypes = [C.c_uint16]
        L.orc_f32_to_f16_rn.restype = C.c_uint16
        L.orc_f32_to_f16_rn.argtypes = [C.c_float]
        L.orc_encode_f16_host.restype = C.c_uint16
        L.orc_encode_f16_host.argtypes = [C.c_float]
        L.orc_argmax_row_f32.restype = C.c_int32
        L.orc_argmax_row_f16.restype = C.c_int32
        L.orc_argmax_key.restype = C.c_int64
        L.orc_argmax_key.argtypes = [C.c_float, C.c_int64]
        L.orc_argmax_key_index.restype = C.c_int32
        L.orc_argmax_key_index.argtypes = [C.c_int64]

    # --- codecs
    def decode_f16(self, bits) -> np.ndarray:
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, np.float32)
        self.lib.orc_decode_f16_array(_ptr(bits), _ptr(out), C.c_int64(bits.size))
        return out

    def f32_to_f16_rn(self, x) -> np.ndarray:
        x = _f32(x)
        out = np.empty(x.shape, np.uint16)
        self.lib.orc_f32_to_f16_rn_array(_ptr(x), _ptr(out), C.c_int64(x.size))
        return out

    # --- CPU operators (fp32)
    def rms_norm(self, x, w, eps):
        x, w = _f32(x), _f32(w)
        h = x.shape[-1]
        out = np.empty_like(x)
        self.lib.orc_cpu_rms_norm(_ptr(x), _ptr(w), C.c_float(eps), C.c_int64(x.size // h), C.c_int64(h), _ptr(out))
        return out

    def add(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self.lib.orc_cpu_add(_ptr(a), _ptr(b), C.c_int64(a.size), _ptr(out))
        return out

    def add_rms_norm(self, lhs, rhs, w, eps):
        lhs, rhs, w = _f32(lhs), _f32(rhs), _f32(w)
        h = lhs.shape[-1]
        res, nrm = np.empty_like(lhs), np.empty_like(lhs)
        self.lib.orc_cpu_add_rms_norm(_ptr(lhs), _ptr(rhs), _ptr(w), C.c_float(eps), C.c_int64(lhs.size // h),
                                      C.c_int64(h), _ptr(res), _ptr(nrm))
        return res, nrm

    def linear(self, x, w):
        """reference src/ops_cpu.cpp:9 / :17 (lm_head): [rows, in] x [out, in]^T in fp32, k ascending."""
        x, w = _f32(x), _f32(w)
        out = np.empty((x.shape[0], w.shape[0]), np.float32)
        self.lib.orc_cpu_linear(_ptr(x), _ptr(w), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_int64(w.shape[0]),
                                _ptr(out))
        return out

    def swiglu(self, gate, up):
        gate, up = _f32(gate), _f32(up)
        out = np.empty_like(gate)
        self.lib.orc_cpu_swiglu(_ptr(gate), _ptr(up), C.c_int64(gate.size), _ptr(out))
        return out

    def rope(self, x, positions, theta):
        x, positions = _f32(x), _i32(positions)
        t, h, d = x.shape
        out = np.empty_like(x)
        rc = self.lib.orc_cpu_rope(_ptr(x), _ptr(positions), C.c_float(theta), C.c_int64(t), C.c_int64(h),
                                   C.c_int64(d), _ptr(out))
        if rc:
            raise ValueError("rope: head_dim must be even and theta positive")
        return out

    def softmax(self, x):
        x = _f32(x)
        w = x.shape[-1]
        out = np.empty_like(x)
        self.lib.orc_cpu_softmax(_ptr(x), C.c_int64(x.size // w), C.c_int64(w), _ptr(out))
        return out

    def softmax_f64(self, x):
        x = _f32(x)
        w = x.shape[-1]
        out = np.empty(x.shape, np.float64)
        self.lib.orc_f64_softmax(_ptr(x), C.c_int64(x.size // w), C.c_int64(w), _ptr(out))
        return out

    def embedding_lookup(self, table, ids):
        table, ids = _f32(table), _i32(ids)
        out = np.empty((ids.size, table.shape[1]), np.float32)
        rc = self.lib.orc_cpu_embedding_lookup(_ptr(table), C.c_int64(table.shape[0]), C.c_int64(table.shape[1]),
                                               _ptr(ids), C.c_int64(ids.size), _ptr(out))
        if rc:
            raise IndexError("embedding_lookup: token id out of range")
        return out

    def argmax_rows(self, x) -> np.ndarray:
        """Row argmax with the reference's tie rule; accepts float32 or float16 bit patterns (uint16)."""
        x = np.ascontiguousarray(x)
        w = x.shape[-1]
        rows = x.reshape(-1, w)
        out = np.empty(rows.shape[0], np.int32)
        for r in range(rows.shape[0]):
            if rows.dtype == np.uint16:
                out[r] = self.lib.orc_argmax_row_f16(_ptr(rows[r]), C.c_int64(w))
            else:
                row = _f32(rows[r])
                out[r] = self.lib.orc_argmax_row_f32(_ptr(row), C.c_int64(w))
        return out

    def sample_row(self, logits_row, temperature, top_k, top_p, seed, offset):
        """(token id, decision margin) of the reference's sampling rule for one row of float32 logits."""
        row = _f32(logits_row).ravel()
        self.lib.orc_sample_row.restype = C.c_int32
        margin = C.c_double(0)
        token = self.lib.orc_sample_row(_ptr(row), C.c_int64(row.size), C.c_float(temperature), C.c_int32(top_k),
                                        C.c_float(top_p), C.c_uint64(seed), C.c_uint64(offset), C.byref(margin))
        return int(token), float(margin.value)

    def paged_kv_write(self, mode, key, value, storage, block_tables, positions, layer, total_blocks, block_size):
        """In-place on `storage` [layers, total_blocks, 2, block_size, kv_heads, head_dim] (any 2- or 4-byte dtype)."""
        key, value = np.ascontiguousarray(key), np.ascontiguousarray(value)
        tables, pos = _i32(block_tables), _i32(positions)
        tokens, kv_heads, head_dim = key.shape
        max_blocks = tables.shape[-1]
        assert storage.flags["C_CONTIGUOUS"] and storage.dtype == key.dtype
        self.lib.orc_paged_kv_write(C.c_int(mode), _ptr(key), _ptr(value), _ptr(storage), _ptr(tables), _ptr(pos),
                                    C.c_int64(tokens), C.c_int64(max_blocks), C.c_int64(layer), C.c_int64(total_blocks),
                                    C.c_int64(block_size), C.c_int64(kv_heads), C.c_int64(head_dim), C.c_int64(key.itemsize))

    def select_last_valid(self, padded, valid_lengths):
        padded = np.ascontiguousarray(padded)
        batch, seq, width = padded.shape
        out = np.empty((batch, width), padded.dtype)
        lengths = _i32(valid_lengths)
        self.lib.orc_select_last_valid(_ptr(padded), _ptr(lengths), _ptr(out), C.c_int64(batch), C.c_int64(seq),
                                       C.c_int64(width * padded.itemsize))
        return out

    def argmax_key(self, value: float, index: int) -> int:
        return int(self.lib.orc_argmax_key(C.c_float(value), C.c_int64(index)))

    def argmax_key_index(self, key: int) -> int:
        return int(self.lib.orc_argmax_key_index(C.c_int64(key)))

    # --- device-order arithmetic; arrays are float32 (dtype F32) or uint16 half bits (dtype F16)
    @staticmethod
    def _code(a: np.ndarray) -> int:
        if a.dtype == np.float32:
            return F32
        if a.dtype == np.uint16:
            return F16
        raise TypeError("device-order oracle takes float32 or uint16 (fp16 bits)")

    def dev_add(self, a, b):
        a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
        out = np.empty_like(a)
        self.lib.orc_dev_add(_ptr(a), _ptr(b), C.c_int64(a.size), _ptr(out), C.c_int(self._code(a)))
        return out

    def dev_rms_norm(self, x, w, eps):
        x, w = np.ascontiguousarray(x), np.ascontiguousarray(w)
        h = x.shape[-1]
        out = np.empty_like(x)
        self.lib.orc_dev_rms_norm(_ptr(x), _ptr(w), C.c_float(eps), C.c_int64(x.size // h), C.c_int64(h), _ptr(out),
                                  C.c_int(self._code(x)))
        return out

    def dev_add_rms_norm(self, lhs, rhs, w, eps):
        lhs, rhs, w = map(np.ascontiguousarray, (lhs, rhs, w))
        h = lhs.shape[-1]
        res, nrm = np.empty_like(lhs), np.empty_like(lhs)
        self.lib.orc_dev_add_rms_norm(_ptr(lhs), _ptr(rhs), _ptr(w), C.c_float(eps), C.c_int64(lhs.size // h),
                                      C.c_int64(h), _ptr(res), _ptr(nrm), C.c_int(self._code(lhs)))
        return res, nrm


class Ref:
    """The reference's own compiled CPU operators (oracle/_ref)."""

    def __init__(self, path: str):
        self.lib = C.CDLL(path)
        self.lib.ref_decode_f16.restype = C.c_float
        self.lib.ref_decode_f16.argtypes = [C.c_uint16]
        self.lib.ref_encode_f16.restype = C.c_uint16
        self.lib.ref_encode_f16.argtypes = [C.c_float]
        self.lib.ref_time_add_rms_norm.restype = C.c_double

    @staticmethod
    def _ok(rc, what):
        if rc == -2:
            raise IndexError(what)
        if rc:
            raise ValueError(what)

    def rms_norm(self, x, w, eps):
        x, w = _f32(x), _f32(w)
        h = x.shape[-1]
        out = np.empty_like(x)
        self._ok(self.lib.ref_rms_norm(_ptr(x), _ptr(w), C.c_float(eps), C.c_int64(x.size // h), C.c_int64(h),
                                       _ptr(out)), "rms_norm")
        return out

    def add(self, a, b):
        a, b = _f32(a), _f32(b)
        out = np.empty_like(a)
        self._ok(self.lib.ref_add(_ptr(a), _ptr(b), C.c_int64(a.size), _ptr(out)), "add")
        return out

    def add_rms_norm(self, lhs, rhs, w, eps):
        lhs, rhs, w = _f32(lhs), _f32(rhs), _f32(w)
        h = lhs.shape[-1]
        res, nrm = np.empty_like(lhs), np.empty_like(lhs)
        self._ok(self.lib.ref_add_rms_norm(_ptr(lhs), _ptr(rhs), _ptr(w), C.c_float(eps), C.c_int64(lhs.size // h),
                                           C.c_int64(h), _ptr(res), _ptr(nrm)), "add_rms_norm")
        return res, nrm

    def time_add_rms_norm(self, lhs, rhs, w, eps, threads: int) -> float:
        lhs, rhs, w = _f32(lhs), _f32(rhs), _f32(w)
        h = lhs.shape[-1]
        res, nrm = np.empty_like(lhs), np.empty_like(lhs)
        dt = self.lib.ref_time_add_rms_norm(_ptr(lhs), _ptr(rhs), _ptr(w), C.c_float(eps), C.c_int64(lhs.size // h),
                                            C.c_int64(h), _ptr(res), _ptr(nrm), C.c_int(threads))
        if dt < 0:
            raise RuntimeError("reference add+rms_norm failed")
        return float(dt)

    def hardware_threads(self) -> int:
        return int(self.lib.ref_hardware_threads())

    def lm_head(self, hidden, table):
        hidden, table = _f32(hidden), _f32(table)
        out = np.empty((hidden.shape[0], table.shape[0]), np.float32)
        self._ok(self.lib.ref_lm_head(_ptr(hidden), _ptr(table), C.c_int64(hidden.shape[0]), C.c_int64(hidden.shape[1]),
                                      C.c_int64(table.shape[0]), _ptr(out)), "lm_head")
        return out

    def swiglu(self, gate, up):
        gate, up = _f32(gate), _f32(up)
        out = np.empty_like(gate)
        self._ok(self.lib.ref_swiglu(_ptr(gate), _ptr(up), C.c_int64(gate.size), _ptr(out)), "swiglu")
        return out

    def rope(self, x, positions, theta):
        x, positions = _f32(x), _i32(positions)
        t, h, d = x.shape
        out = np.empty_like(x)
        self._ok(self.lib.ref_rope(_ptr(x), _ptr(positions), C.c_float(theta), C.c_int64(t), C.c_int64(h),
                                   C.c_int64(d), _ptr(out)), "rope")
        return out

    def softmax(self, x):
        x = _f32(x)
        w = x.shape[-1]
        out = np.empty_like(x)
        self._ok(self.lib.ref_softmax(_ptr(x), C.c_int64(x.size // w), C.c_int64(w), _ptr(out)), "softmax")
        return out

    def embedding_lookup(self, table, ids):
        table, ids = _f32(table), _i32(ids)
        out = np.empty((ids.size, table.shape[1]), np.float32)
        self._ok(self.lib.ref_embedding_lookup(_ptr(table), C.c_int64(table.shape[0]), C.c_int64(table.shape[1]),
                                               _ptr(ids), C.c_int64(ids.size), _ptr(out)), "embedding_lookup")
        return out

    def decode_f16(self, h: int) -> float:
        return float(self.lib.ref_decode_f16(C.c_uint16(h)))

    def encode_f16(self, x: float) -> int:
        return int(self.lib.ref_encode_f16(C.c_float(x)))


_port = None
_ref = False


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref():
    """The reference-backed oracle, or None when oracle/_ref was not built."""
    global _ref
    if _ref is False:
        path = os.path.join(_HERE, "_ref", "liboracle_ref.so")
        _ref = Ref(path) if os.path.exists(path) else None
    return _ref


class RefCuda:
    """The reference's own CUDA operators (oracle/_ref/libref_cuda.so).  Arguments are device pointers
    (ints) or anything with ``data_ptr()``; dtype codes as elsewhere (F32 = 0, F16 = 1)."""

    def __init__(self, path: str):
        self.lib = L = C.CDLL(path)
        for name in ("refcu_time_add_rms_norm", "refcu_time_rms_norm", "refcu_time_binary", "refcu_time_rope_token_positions",
                     "refcu_time_embedding", "refcu_time_softmax", "refcu_time_argmax_last_row", "refcu_time_sample_row"):
            getattr(L, name).restype = C.c_float
        if hasattr(L, "refcu_time_decode_chain"):      # absent from a library built before this door existed
            L.refcu_time_decode_chain.restype = C.c_float

    @staticmethod
    def _p(t):
        return C.c_void_p(t if isinstance(t, int) else t.data_ptr())

    @staticmethod
    def _ok(rc, what):
        if rc:
            raise RuntimeError(f"reference CUDA operator {what} failed with {rc}")

    def rms_norm(self, x, w, out, rows, hidden, eps, dtype):
        self._ok(self.lib.refcu_rms_norm(self._p(x), self._p(w), self._p(out), C.c_int64(rows), C.c_int64(hidden),
                                         C.c_float(eps), C.c_int(dtype)), "rms_norm")

    def add_rms_norm(self, lhs, rhs, w, residual, normalized, rows, hidden, eps, dtype):
        self._ok(self.lib.refcu_add_rms_norm(self._p(lhs), self._p(rhs), self._p(w), self._p(residual), self._p(normalized),
                                             C.c_int64(rows), C.c_int64(hidden), C.c_float(eps), C.c_int(dtype)), "add_rms_norm")

    def add(self, a, b, out, n, dtype):
        self._ok(self.lib.refcu_add(self._p(a), self._p(b), self._p(out), C.c_int64(n), C.c_int(dtype)), "add")

    def swiglu(self, g, u, out, n, dtype):
        self._ok(self.lib.refcu_swiglu(self._p(g), self._p(u), self._p(out), C.c_int64(n), C.c_int(dtype)), "swiglu")

    def rope(self, x, positions_host, out, tokens, heads, head_dim, theta, dtype):
        pos = _i32(positions_host)
        self._ok(self.lib.refcu_rope(self._p(x), _ptr(pos), self._p(out), C.c_int64(tokens), C.c_int64(heads),
                                     C.c_int64(head_dim), C.c_float(theta), C.c_int(dtype)), "rope")

    def rope_token_positions(self, x, positions_device, out, tokens, heads, theta):
        self._ok(self.lib.refcu_rope_token_positions(self._p(x), self._p(positions_device), self._p(out), C.c_int64(tokens),
                                                     C.c_int64(heads), C.c_float(theta)), "rope_token_positions")

    def softmax(self, x, out, rows, width, dtype):
        self._ok(self.lib.refcu_softmax(self._p(x), self._p(out), C.c_int64(rows), C.c_int64(width), C.c_int(dtype)), "softmax")

    def embedding_lookup(self, table, ids_host, out, hidden, vocab, dtype):
        ids = _i32(ids_host)
        self._ok(self.lib.refcu_embedding_lookup(self._p(table), _ptr(ids), self._p(out), C.c_int64(ids.size), C.c_int64(hidden),
                                                 C.c_int64(vocab), C.c_int(dtype)), "embedding_lookup")

    def argmax_last_row(self, logits, rows, width, dtype) -> int:
        r = C.c_int32(-1)
        self._ok(self.lib.refcu_argmax_last_row(self._p(logits), C.c_int64(rows), C.c_int64(width), C.c_int(dtype), C.byref(r)),
                 "argmax_last_row")
        return int(r.value)

    def lm_head_argmax(self, hidden, table, rows, hidden_size, vocab, dtype, logits_out=None) -> int:
        """cuda_lm_head followed by cuda_argmax_last_row, as the reference's decode tail runs them."""
        r = C.c_int32(-1)
        self._ok(self.lib.refcu_lm_head_argmax(self._p(hidden), self._p(table), C.c_int64(rows), C.c_int64(hidden_size),
                                               C.c_int64(vocab), C.c_int(dtype),
                                               self._p(logits_out) if logits_out is not None else None, C.byref(r)),
                 "lm_head_argmax")
        return int(r.value)

    def sample_row(self, logits, rows, vocab, dtype, row, temperature, top_k, top_p, seed, draw_offset) -> int:
        """CudaSampler::sample_row of the reference: one token, one blocking call."""
        r = C.c_int32(-1)
        self._ok(self.lib.refcu_sample_row(self._p(logits), C.c_int64(rows), C.c_int64(vocab), C.c_int(dtype), C.c_int64(row),
                                           C.c_float(temperature), C.c_int32(top_k), C.c_float(top_p), C.c_uint64(seed),
                                           C.c_uint64(draw_offset), C.byref(r)), "sample_row")
        return int(r.value)

    def time_sample_row(self, logits, rows, vocab, dtype, temperature, top_k, top_p, reps):
        return float(self.lib.refcu_time_sample_row(self._p(logits), C.c_int64(rows), C.c_int64(vocab), C.c_int(dtype),
                                                    C.c_float(temperature), C.c_int32(top_k), C.c_float(top_p), C.c_int(reps)))

    # timings: milliseconds per call of the reference operator on device-resident tensors
    def time_add_rms_norm(self, lhs, rhs, w, rows, hidden, eps, dtype, reps):
        return float(self.lib.refcu_time_add_rms_norm(self._p(lhs), self._p(rhs), self._p(w), C.c_int64(rows), C.c_int64(hidden),
                                                      C.c_float(eps), C.c_int(dtype), C.c_int(reps)))

    def time_rms_norm(self, x, w, rows, hidden, eps, dtype, reps):
        return float(self.lib.refcu_time_rms_norm(self._p(x), self._p(w), C.c_int64(rows), C.c_int64(hidden), C.c_float(eps),
                                                  C.c_int(dtype), C.c_int(reps)))

    def time_binary(self, a, b, n, dtype, swiglu, reps):
        return float(self.lib.refcu_time_binary(self._p(a), self._p(b), C.c_int64(n), C.c_int(dtype), C.c_int(int(swiglu)),
                                                C.c_int(reps)))

    def time_rope_token_positions(self, x, positions_device, tokens, heads, theta, reps):
        return float(self.lib.refcu_time_rope_token_positions(self._p(x), self._p(positions_device), C.c_int64(tokens),
                                                              C.c_int64(heads), C.c_float(theta), C.c_int(reps)))

    def time_decode_chain(self, tokens, eps, theta, graph, reps):
        """ms per chain of the reference's in-scope operators of one decode layer (see refcu_time_decode_chain)."""
        return float(self.lib.refcu_time_decode_chain(C.c_int64(tokens), C.c_float(eps), C.c_float(theta), C.c_int(graph), C.c_int(reps)))

    def time_embedding(self, table, ids_device, count, hidden, vocab, dtype, reps):
        return float(self.lib.refcu_time_embedding(self._p(table), self._p(ids_device), C.c_int64(count), C.c_int64(hidden),
                                                   C.c_int64(vocab), C.c_int(dtype), C.c_int(reps)))

    def time_softmax(self, x, rows, width, dtype, reps):
        return float(self.lib.refcu_time_softmax(self._p(x), C.c_int64(rows), C.c_int64(width), C.c_int(dtype), C.c_int(reps)))

    def time_argmax_last_row(self, logits, rows, width, dtype, reps):
        return float(self.lib.refcu_time_argmax_last_row(self._p(logits), C.c_int64(rows), C.c_int64(width), C.c_int(dtype),
                                                         C.c_int(reps)))


    def time_lm_head_argmax(self, hidden, table, rows, hidden_size, vocab, dtype, reps):
        self.lib.refcu_time_lm_head_argmax.restype = C.c_float
        return float(self.lib.refcu_time_lm_head_argmax(self._p(hidden), self._p(table), C.c_int64(rows), C.c_int64(hidden_size),
                                                        C.c_int64(vocab), C.c_int(dtype), C.c_int(reps)))


_ref_cuda = False


def ref_cuda():
    """The reference's CUDA operators recompiled for sm_100a, or None when oracle/_ref/libref_cuda.so is absent."""
    global _ref_cuda
    if _ref_cuda is False:
        path = os.path.join(_HERE, "_ref", "libref_cuda.so")
        try:
            _ref_cuda = RefCuda(path) if os.path.exists(path) else None
        except OSError:
            _ref_cuda = None
    return _ref_cuda



# ---------------------------------------------------------------------------------------------
# The reference's own decoder-layer code, twice: with the reference's operators and with the in-scope
# operators replaced by this repository's (oracle/Makefile, target `layer`).
# ---------------------------------------------------------------------------------------------

LAYER_NODES = ("input_norm", "q_linear", "k_linear", "v_linear", "q_norm_output", "k_norm_output", "q_rope", "k_rope",
               "attention_output", "o_proj_output", "attention_residual", "post_attention_norm", "gate_proj_output",
               "up_proj_output", "swiglu_output", "down_proj_output", "layer_output")
LAYER_WEIGHTS = (("input_norm", (1024,)), ("q_proj", (2048, 1024)), ("k_proj", (1024, 1024)), ("v_proj", (1024, 1024)),
                 ("q_norm", (128,)), ("k_norm", (128,)), ("o_proj", (1024, 2048)), ("post_attention_norm", (1024,)),
                 ("gate_proj", (3072, 1024)), ("up_proj", (3072, 1024)), ("down_proj", (1024, 3072)))


class LayerLib:
    """qwen3_decoder_layer_cuda_trace / _trace_fp16 of the reference (src/qwen3_layer_cuda.cu:99-160) behind
    oracle/layer_wrapper.cu.  `replaced` tells whether RMSNorm, RoPE, add and SwiGLU are this repository's."""

    def __init__(self, path: str):
        self.lib = C.CDLL(path)
        self.lib.layer_trace.restype = C.c_int
        self.lib.layer_select_reductions.restype = C.c_int
        self.replaced = bool(self.lib.layer_select_reductions(0))

    def select_reductions(self, deterministic: bool) -> None:
        self.lib.layer_select_reductions(1 if deterministic else 0)

    def trace(self, hidden: np.ndarray, positions, weights: dict, eps: float, theta: float, half: bool) -> dict:
        seq = hidden.shape[0]
        x = _f32(hidden)
        pos = _i32(positions)
        ws = [_f32(weights[name]).reshape(shape) for name, shape in LAYER_WEIGHTS]
        wptr = (C.c_void_p * len(ws))(*[w.ctypes.data for w in ws])
        shapes = {"input_norm": 1024, "q_linear": 2048, "k_linear": 1024, "v_linear": 1024, "q_norm_output": 2048,
                  "k_norm_output": 1024, "q_rope": 2048, "k_rope": 1024, "attention_output": 2048, "o_proj_output": 1024,
                  "attention_residual": 1024, "post_attention_norm": 1024, "gate_proj_output": 3072, "up_proj_output": 3072,
                  "swiglu_output": 3072, "down_proj_output": 1024, "layer_output": 1024}
        outs = {n: np.empty((seq, shapes[n]), np.float32) for n in LAYER_NODES}
        optr = (C.c_void_p * len(LAYER_NODES))(*[outs[n].ctypes.data for n in LAYER_NODES])
        err = C.create_string_buffer(512)
        rc = self.lib.layer_trace(C.c_int(1 if half else 0), _ptr(x), C.c_int(seq), _ptr(pos), wptr, C.c_float(eps),
                                  C.c_float(theta), optr, err, C.c_int(512))
        if rc != 0:
            raise RuntimeError(err.value.decode(errors="replace"))
        return outs


def layer_libs():
    """(all-reference library, drop-in library), or None when they were not built."""
    paths = [os.path.join(_HERE, "_ref", n) for n in ("liblayer_ref.so", "liblayer_dropin.so")]
    if not all(os.path.exists(p) for p in paths):
        return None
    return LayerLib(paths[0]), LayerLib(paths[1])
