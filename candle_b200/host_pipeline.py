"""Norms over rows that live in pinned host memory.

A caller whose activations are on the host pays PCIe for every byte, in both directions; the only
thing to gain is to keep both directions and the kernel busy at once.  ``PinnedNormPipeline`` cuts
the rows into chunks and runs three stages on three streams: chunk i+1 is copied in while chunk i
is normalised and chunk i-1 is copied out.  Two sets of device buffers per stage; events order
the reuse of each.  The arithmetic is the one-launch kernels of ``ops`` on every chunk, so the
result is bit-identical to a single call on the whole tensor (rows are independent).
"""
from __future__ import annotations

import torch

from . import ops
from .errors import CandleError


class PinnedNormPipeline:
    """``rms_norm`` / ``layer_norm`` (optionally ``x + residual`` first) from pinned host tensors to
    a pinned host tensor, pipelined over row chunks."""

    def __init__(self, cols: int, dtype: torch.dtype, device, *, chunk_rows: int = 8192, with_residual: bool = True):
        self.cols, self.dtype, self.device, self.chunk_rows = cols, dtype, torch.device(device), int(chunk_rows)
        if self.chunk_rows < 1:
            raise CandleError("chunk_rows must be positive")
        mk = lambda: torch.empty(self.chunk_rows, cols, dtype=dtype, device=self.device)  # noqa: E731
        self.x = [mk(), mk()]
        self.r = [mk(), mk()] if with_residual else None
        self.y = [mk(), mk()]
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_comp = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]

    def _check_host(self, name: str, t: torch.Tensor, rows: int) -> None:
        if t.is_cuda or not t.is_pinned():
            raise CandleError(f"{name} must be a pinned host tensor")
        if t.dtype != self.dtype or t.dim() != 2 or t.shape[1] != self.cols or t.shape[0] != rows or not t.is_contiguous():
            raise CandleError(f"shape mismatch in pinned pipeline: {name} {list(t.shape)} for [{rows}, {self.cols}]")

    def run(self, x_host: torch.Tensor, y_host: torch.Tensor, alpha: torch.Tensor, eps: float, *,
            residual_host: torch.Tensor | None = None, beta: torch.Tensor | None = None, flags: int = 0) -> None:
        """``y_host = norm(x_host [+ residual_host])``; RMS norm, or layer norm when ``beta`` is given.
        Returns with the work queued: the caller's current stream waits for the last copy out, so a
        synchronize (or an event) on that stream tells when ``y_host`` is complete."""
        rows = x_host.shape[0]
        self._check_host("x", x_host, rows)
        self._check_host("y", y_host, rows)
        if (residual_host is None) != (self.r is None):
            raise CandleError("the pipeline was built with_residual=%s" % (self.r is not None))
        if residual_host is not None:
            self._check_host("residual", residual_host, rows)
        caller = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(caller)
        used = [False, False]
        for c, begin in enumerate(range(0, rows, self.chunk_rows)):
            n = min(self.chunk_rows, rows - begin)
            k = c & 1
            if used[k]:
                self.s_in.wait_event(self.ev_comp[k])   # the kernel that read this input set is done
            with torch.cuda.stream(self.s_in):
                self.x[k][:n].copy_(x_host[begin:begin + n], non_blocking=True)
                if self.r is not None:
                    self.r[k][:n].copy_(residual_host[begin:begin + n], non_blocking=True)
                self.ev_in[k].record(self.s_in)
            self.s_comp.wait_event(self.ev_in[k])
            if used[k]:
                self.s_comp.wait_event(self.ev_out[k])  # the copy out of this output set is done
            with torch.cuda.stream(self.s_comp):
                res = self.r[k][:n] if self.r is not None else None
                if beta is None:
                    y = ops.rms_norm(self.x[k][:n], alpha, eps, residual=res, flags=flags, out=self.y[k][:n])
                else:
                    y = ops.layer_norm(self.x[k][:n], alpha, beta, eps, residual=res, flags=flags, out=self.y[k][:n])
                assert y.data_ptr() == self.y[k].data_ptr()
                self.ev_comp[k].record(self.s_comp)
            self.s_out.wait_event(self.ev_comp[k])
            with torch.cuda.stream(self.s_out):
                y_host[begin:begin + n].copy_(self.y[k][:n], non_blocking=True)
                self.ev_out[k].record(self.s_out)
            used[k] = True
        caller.wait_stream(self.s_out)
        caller.wait_stream(self.s_comp)
        caller.wait_stream(self.s_in)
