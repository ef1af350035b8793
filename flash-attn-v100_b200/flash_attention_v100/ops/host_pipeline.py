"""Forward + backward with every operand in pinned host memory.

The reference keeps its tensors on the device and has no counterpart of this
module; its multi-GPU manager splits a call along the batch dimension
(interface.py:228-263), and the same split is used here in time instead of in
space: the batch is cut into chunks and three CUDA streams work on different
chunks at once,

    copy-in stream   q, k, v, d_o of chunk c        (host -> device)
    compute stream   fa_b200_fwd, fa_b200_bwd on c  (through the C ABI)
    copy-out stream  o, dq, dk, dv of chunk c       (device -> host)

so that PCIe carries data in both directions while the kernels run.  Chunks
are whole batch entries (contiguous in the (B, N, H, D) layout), the device
buffers are allocated once, and successive calls overlap too: the copy-in of a
call starts while the copy-out of the previous one drains.

Dropout: chunk c uses the stream (seed, offset + (c << 40)), so the mask of a
chunked call differs from the mask of one call over the whole batch but is a
pure function of (seed, offset, chunking).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import attention as _ops

_IN = ("q", "k", "v", "d_o")
_OUT = ("o", "dq", "dk", "dv")


def chunk_bounds(batch: int, chunks: int) -> List[Tuple[int, int]]:
    """[begin, end) batch ranges of `chunks` near-equal chunks (fewer if batch is smaller)."""
    if batch < 0 or chunks < 1:
        raise ValueError("batch must be non-negative and chunks positive")
    n = max(1, min(chunks, batch))
    base, extra = divmod(batch, n)
    out, b = [], 0
    for c in range(n):
        e = b + base + (1 if c < extra else 0)
        out.append((b, e))
        b = e
    return out


def chunk_dropout_offset(offset: int, chunk: int) -> int:
    """Dropout stream offset of chunk `chunk` of a call made with `offset`."""
    return (int(offset) + (int(chunk) << 40)) & 0xFFFFFFFFFFFFFFFF


class HostAttentionStep:
    """One attention forward + backward per call, operands and results in pinned host memory.

    step = HostAttentionStep(q.shape, k.shape, dtype, device, causal=True)
    step(host_in, host_out)          # dicts of pinned tensors; returns without blocking the host
    step.synchronize()               # host_out is complete

    host_in holds q, k, v, d_o and host_out holds o, dq, dk, dv, all (B, N, H, D).
    The caller's current stream waits for the results, so work queued on it afterwards
    (or an event recorded on it) is ordered after the last copy-out.
    """

    def __init__(self, q_shape: Sequence[int], k_shape: Sequence[int], dtype: torch.dtype,
                 device, causal: bool = False, scale: Optional[float] = None, dropout_p: float = 0.0,
                 chunks: Optional[int] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("HostAttentionStep needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        B, Nq, H, D = (int(x) for x in q_shape)
        Bk, Nk, Hkv, Dk = (int(x) for x in k_shape)
        if Bk != B or Dk != D:
            raise ValueError("q and k must agree in batch and head_dim")
        self.q_shape, self.k_shape, self.dtype = (B, Nq, H, D), (B, Nk, Hkv, D), dtype
        self.causal, self.dropout_p = bool(causal), float(dropout_p)
        self.scale = float(D ** -0.5 if scale is None else scale)
        self.bounds = chunk_bounds(B, B if chunks is None else int(chunks))
        dev = self.device
        with torch.cuda.device(dev):
            self._dev: Dict[str, torch.Tensor] = {}
            for n in _IN + _OUT:
                shape = self.k_shape if n in ("k", "v", "dk", "dv") else self.q_shape
                self._dev[n] = torch.empty(shape, dtype=dtype, device=dev)
            self._lse = torch.empty(B, H, Nq, dtype=torch.float32, device=dev)
            self._ws = [self._workspace(e - b) for b, e in self.bounds]
            self._s_in, self._s_run, self._s_out = (torch.cuda.Stream(dev) for _ in range(3))
            n = len(self.bounds)
            ev = lambda: [torch.cuda.Event() for _ in range(n)]
            self._ev_qkv, self._ev_do, self._ev_fwd, self._ev_bwd, self._ev_out = ev(), ev(), ev(), ev(), ev()
            self._ev_done = torch.cuda.Event()
        self._calls = 0

    def _workspace(self, batch: int) -> torch.Tensor:
        from .memory import backward_workspace_bytes
        _, Nq, H, D = self.q_shape
        _, Nk, Hkv, _ = self.k_shape
        n = backward_workspace_bytes(batch, Nq, Nk, H, D, self.dtype, num_heads_kv=Hkv) if batch else 0
        return torch.empty(max(n, 1), dtype=torch.uint8, device=self.device)

    @property
    def h2d_bytes(self) -> int:
        return sum(self._dev[n].numel() * self._dev[n].element_size() for n in _IN)

    @property
    def d2h_bytes(self) -> int:
        return sum(self._dev[n].numel() * self._dev[n].element_size() for n in _OUT)

    def _check(self, host: Dict[str, torch.Tensor], names) -> None:
        for n in names:
            t = host[n]
            want = self.k_shape if n in ("k", "v", "dk", "dv") else self.q_shape
            if tuple(t.shape) != want or t.dtype != self.dtype:
                raise ValueError(f"{n}: expected {want} {self.dtype}, got {tuple(t.shape)} {t.dtype}")
            if t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{n} must be a contiguous host tensor")
            if not t.is_pinned():
                raise ValueError(f"{n} must be in pinned host memory (asynchronous copies need it)")

    def __call__(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor],
                 seed: int = 0, offset: int = 0) -> None:
        self._check(host_in, _IN)
        self._check(host_out, _OUT)
        d = self._dev
        caller = torch.cuda.current_stream(self.device)
        self._s_in.wait_stream(caller)
        first = self._calls == 0
        for c, (b, e) in enumerate(self.bounds):
            if e == b:
                continue
            with torch.cuda.stream(self._s_in):
                if not first:
                    self._s_in.wait_event(self._ev_bwd[c])      # previous call still reads chunk c's inputs
                for n in ("q", "k", "v"):
                    d[n][b:e].copy_(host_in[n][b:e], non_blocking=True)
                self._ev_qkv[c].record(self._s_in)
                d["d_o"][b:e].copy_(host_in["d_o"][b:e], non_blocking=True)
                self._ev_do[c].record(self._s_in)
            with torch.cuda.stream(self._s_run):
                if not first:
                    self._s_run.wait_event(self._ev_out[c])     # previous results of chunk c copied out
                self._s_run.wait_event(self._ev_qkv[c])
                off = chunk_dropout_offset(offset, c) if self.dropout_p > 0 else 0
                sd = int(seed) if self.dropout_p > 0 else 0
                _ops.launch_forward(d["q"][b:e], d["k"][b:e], d["v"][b:e], self.scale, self.causal,
                                    self.dropout_p, sd, off, out=(d["o"][b:e], self._lse[b:e]))
                self._ev_fwd[c].record(self._s_run)
                self._s_run.wait_event(self._ev_do[c])
                _ops.launch_backward(d["d_o"][b:e], d["q"][b:e], d["k"][b:e], d["v"][b:e], d["o"][b:e],
                                     self._lse[b:e], self.scale, self.causal, self.dropout_p, sd, off,
                                     out=(d["dq"][b:e], d["dk"][b:e], d["dv"][b:e]), workspace=self._ws[c])
                self._ev_bwd[c].record(self._s_run)
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(self._ev_fwd[c])
                host_out["o"][b:e].copy_(d["o"][b:e], non_blocking=True)
                self._s_out.wait_event(self._ev_bwd[c])
                for n in ("dq", "dk", "dv"):
                    host_out[n][b:e].copy_(d[n][b:e], non_blocking=True)
                self._ev_out[c].record(self._s_out)
        self._ev_done.record(self._s_out)
        caller.wait_event(self._ev_done)
        self._calls += 1

    def synchronize(self) -> None:
        """Block the host until the results of the last call are in host memory."""
        self._ev_done.synchronize()
        _ops.check_status(self.device)


__all__ = ["HostAttentionStep", "chunk_bounds", "chunk_dropout_offset"]
