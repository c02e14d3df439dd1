"""Host-buffer forms of the row-independent operators: the data starts and ends in (pinned) host
memory, as it does for a caller of the reference's Tensor::to(CUDA) ... Tensor::to(CPU) round trip
(src/tensor_cuda.cu:56).  Rows are independent, so the batch is cut into row chunks and three
streams overlap the host->device copy of chunk i+1, the kernel on chunk i and the device->host copy
of chunk i-1: PCIe is full duplex, so the round trip costs about one direction's transfer time
instead of two.  The arithmetic is the same C ABI call as everywhere else, once per chunk.
"""
from __future__ import annotations

import torch

from . import lib as _lib


class AddRmsNormHostPipeline:
    """residual, normalized = add_rms_norm(x, res) for host tensors, chunked over rows."""

    def __init__(self, rows: int, hidden: int, device, chunks: int = 8, dtype=torch.float16):
        self.rows, self.hidden, self.dev = rows, hidden, torch.device(device)
        self.chunks = max(1, min(chunks, rows))
        self.bounds = [(rows * c // self.chunks, rows * (c + 1) // self.chunks) for c in range(self.chunks)]
        mk = lambda: torch.empty(rows, hidden, dtype=dtype, device=self.dev)
        self.x, self.r, self.res, self.nrm = mk(), mk(), mk(), mk()
        self.s_in, self.s_k, self.s_out = (torch.cuda.Stream(device=self.dev) for _ in range(3))
        self.done_out = [None] * self.chunks          # device->host copy of the previous call, per chunk
        self.code = _lib.F16 if dtype == torch.float16 else _lib.F32
        self.L = _lib.load()

    def __call__(self, hx, hr, gamma, h_res, h_nrm, eps=1e-6, mode=_lib.FAST, copies_only=False):
        """hx, hr, h_res, h_nrm: pinned host tensors [rows, hidden]; gamma: device tensor [hidden].
        Returns the event that marks the last device->host copy; nothing blocks the host.
        copies_only: the same copies in the same order without the kernel between them (what the host's
        PCIe and memory path alone allow: the ceiling of the end-to-end number)."""
        last = None
        for c, (lo, hi) in enumerate(self.bounds):
            with torch.cuda.stream(self.s_in):
                self.x[lo:hi].copy_(hx[lo:hi], non_blocking=True)
                self.r[lo:hi].copy_(hr[lo:hi], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(ready)
                if self.done_out[c] is not None:      # the previous call's results of this chunk have left the device
                    self.s_k.wait_event(self.done_out[c])
                n = hi - lo
                if not copies_only:
                    _lib.check(self.L.b2_add_rms_norm(self.x[lo:hi].data_ptr(), self.r[lo:hi].data_ptr(), gamma.data_ptr(),
                                                      self.res[lo:hi].data_ptr(), self.nrm[lo:hi].data_ptr(), n,
                                                      self.hidden, eps, self.code, mode, self.s_k.cuda_stream))
                computed = torch.cuda.Event()
                computed.record(self.s_k)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed)
                h_res[lo:hi].copy_(self.res[lo:hi], non_blocking=True)
                h_nrm[lo:hi].copy_(self.nrm[lo:hi], non_blocking=True)
                last = torch.cuda.Event()
                last.record(self.s_out)
                self.done_out[c] = last
        return last
