"""Forward + backward with every operand in pinned host memory.

The reference keeps its tensors on the device and has no counterpart of this
module; its multi-GPU manager splits a call over heads or batch entries
(interface.py:228-263, :382-434), and the same split is used here in time
instead of in space: the (batch x heads) grid is cut into chunks and three CUDA
streams work on different chunks at once,

    copy-in stream   q, k, v, d_o of chunk c        (host -> device)
    compute stream   fa_b200_fwd, fa_b200_bwd on c  (through the C ABI)
    copy-out stream  o, dq, dk, dv of chunk c       (device -> host)

so that PCIe carries data in both directions while the kernels run.  A chunk is
a range of heads of one batch entry (or whole batch entries): in the
(B, N, H, D) layout that is N rows of (h1 - h0) * D elements with a pitch of
H * D, which one strided copy per tensor moves (fa_b200_copy_rows), and which the
kernels consume in place as a strided view.  Small chunks shorten what cannot
overlap, the copy-in of the first chunk and the copy-out of the last one, and
let a batch of one overlap at all.  The device buffers are allocated once, and
successive calls overlap too: the copy-in of a call starts while the copy-out of
the previous one drains.

Dropout: every chunk uses the call's (seed, offset) and indexes the stream by
its columns' place in the whole problem, so a chunked call draws exactly the
mask of one call over the whole batch, however it is chunked.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import attention as _ops
from ..kernels import _cabi

_IN = ("q", "k", "v", "d_o")
_OUT = ("o", "dq", "dk", "dv")

Chunk = Tuple[int, int, int, int]     # (b0, b1, h0, h1): half-open batch and query-head ranges


def chunk_bounds(batch: int, chunks: int) -> List[Tuple[int, int]]:
    """[begin, end) ranges of `chunks` near-equal parts of `batch` items (fewer if batch is smaller)."""
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


def plan_chunks(batch: int, heads: int, heads_kv: int, chunks: Optional[int] = None,
                min_columns: int = 8, target: int = 16) -> List[Chunk]:
    """Cut the (batch x heads) grid into chunks, batch-major.

    `chunks=None` aims at `target` chunks of at least `min_columns` (batch, head) columns each (fewer
    columns leave SMs idle in the kernels; fewer chunks expose more of the first copy-in and the last
    copy-out).  Measured on B200 over PCIe, B4 N4096 H32 D128 bf16: 4 chunks 13.8 ms per step, 8 12.1,
    16 11.6, 32 12.8, 64 18.0; B1 N16384 H32: 2 chunks 16.9, 4 14.1, 8 14.2, 16 15.1: eight columns a chunk.  Up to `batch` chunks are whole batch entries; beyond that every batch entry is cut
    into head groups, at multiples of the K/V group size H / Hkv so that a chunk owns its K/V heads.
    """
    if batch <= 0:
        return [(0, 0, 0, heads)]
    if chunks is None:
        chunks = max(1, min(target, (batch * heads) // max(1, min_columns)))
    chunks = max(1, int(chunks))
    if chunks <= batch:
        return [(b, e, 0, heads) for b, e in chunk_bounds(batch, chunks)]
    group = heads // heads_kv
    per_entry = min(heads_kv, -(-chunks // batch))           # head groups per batch entry
    out = []
    for b in range(batch):
        for k0, k1 in chunk_bounds(heads_kv, per_entry):
            out.append((b, b + 1, k0 * group, k1 * group))
    return out


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
        # a chunk should also move enough bytes for a copy to run at PCIe speed: 8 MiB per tensor
        col_bytes = max(1, max(Nq, Nk) * D * torch.empty((), dtype=dtype).element_size())
        self.chunks: List[Chunk] = plan_chunks(B, H, Hkv, chunks, min_columns=max(8, -(-(8 << 20) // col_bytes)))
        self.bounds = self.chunks               # (b0, b1, h0, h1) per chunk
        self._group = H // Hkv
        dev = self.device
        with torch.cuda.device(dev):
            self._dev: Dict[str, torch.Tensor] = {}
            for n in _IN + _OUT:
                shape = self.k_shape if n in ("k", "v", "dk", "dv") else self.q_shape
                self._dev[n] = torch.empty(shape, dtype=dtype, device=dev)
            # what rounding the output to bf16 drops stays on the device for the backward (as in the autograd op)
            self._o_lo = torch.empty(self.q_shape, dtype=dtype, device=dev) if _ops.saves_output_residual(dtype) else None
            # the log-sum-exp stays on the device: one dense (b, h, Nq) buffer per chunk
            self._lse = [torch.empty(b1 - b0, h1 - h0, Nq, dtype=torch.float32, device=dev)
                         for b0, b1, h0, h1 in self.chunks]
            self._ws = [self._workspace(b1 - b0, h1 - h0) for b0, b1, h0, h1 in self.chunks]
            # dropout: one buffer for the keep bits of the chunk in flight (the kernels of all chunks run
            # on one stream): the chunk's forward fills it, its backward reads it
            self._bits = None
            if self.dropout_p > 0.0:
                cols = max(((b1 - b0) * (h1 - h0) for b0, b1, h0, h1 in self.chunks), default=0)
                pad = lambda n: -(-n // 128) * 128
                nbits = cols * pad(Nq) * pad(Nk) // 4
                if 0 < nbits <= _ops.KEEP_BITS_MAX_BYTES:          # beyond the cap the kernels draw their own bits
                    self._bits = torch.empty(nbits, dtype=torch.uint8, device=dev)
            self._s_in, self._s_run, self._s_out = (torch.cuda.Stream(dev) for _ in range(3))
            n = len(self.chunks)
            ev = lambda: [torch.cuda.Event() for _ in range(n)]
            self._ev_qkv, self._ev_do, self._ev_fwd, self._ev_bwd, self._ev_out = ev(), ev(), ev(), ev(), ev()
            self._ev_done = torch.cuda.Event()
        self._calls = 0

    def _workspace(self, batch: int, heads: int) -> torch.Tensor:
        from .memory import backward_workspace_bytes
        _, Nq, _, D = self.q_shape
        _, Nk, _, _ = self.k_shape
        n = backward_workspace_bytes(batch, Nq, Nk, heads, D, self.dtype,
                                     num_heads_kv=heads // self._group) if batch and heads else 0
        return torch.empty(max(n, 1), dtype=torch.uint8, device=self.device)

    def _copy(self, dst: torch.Tensor, src: torch.Tensor, stream: "torch.cuda.Stream") -> None:
        """dst <- src for two (b, N, h, D) views of the same shape (one in pinned host memory, one on
        the device), as one strided copy per batch entry on `stream`."""
        if dst.numel() == 0:
            return
        es = dst.element_size()
        b, n, h, d = dst.shape
        lib = _cabi.load()
        whole = all(t.stride(2) == d and t.stride(1) == h * d for t in (dst, src))
        if whole and dst.stride(0) == n * h * d and src.stride(0) == n * h * d:
            views = [(dst, src, 1, b * n * h * d * es)]                    # contiguous: one flat copy
        else:
            views = [(dst[i], src[i], n, h * d * es) for i in range(b)]    # N rows of h * D elements each
        for dv, sv, rows, row_bytes in views:
            dp = row_bytes if rows == 1 else dv.stride(0) * es
            sp = row_bytes if rows == 1 else sv.stride(0) * es
            rc = lib.fa_b200_copy_rows(dv.data_ptr(), dp, sv.data_ptr(), sp, row_bytes, rows,
                                       self.device.index or 0, stream.cuda_stream)
            _cabi.raise_for_status(rc, "fa_b200_copy_rows")

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
        g = self._group
        for c, (b, e, h0, h1) in enumerate(self.chunks):
            if e == b or h1 == h0:
                continue
            qs = (slice(b, e), slice(None), slice(h0, h1))               # the chunk's query heads
            ks = (slice(b, e), slice(None), slice(h0 // g, h1 // g))     # ... and its K/V heads
            sl = lambda n: ks if n in ("k", "v", "dk", "dv") else qs
            with torch.cuda.stream(self._s_in):
                if not first:
                    self._s_in.wait_event(self._ev_bwd[c])      # previous call still reads chunk c's inputs
                for n in ("q", "k", "v"):
                    self._copy(d[n][sl(n)], host_in[n][sl(n)], self._s_in)
                self._ev_qkv[c].record(self._s_in)
                self._copy(d["d_o"][qs], host_in["d_o"][qs], self._s_in)
                self._ev_do[c].record(self._s_in)
            with torch.cuda.stream(self._s_run):
                if not first:
                    self._s_run.wait_event(self._ev_out[c])     # previous results of chunk c copied out
                self._s_run.wait_event(self._ev_qkv[c])
                sd, off = (int(seed), int(offset)) if self.dropout_p > 0 else (0, 0)
                origin = (b, h0, self.q_shape[2])               # this chunk's place in the whole problem
                lse_c = self._lse[c]
                res = self._o_lo[qs] if self._o_lo is not None else None
                bits = (self._bits, False) if self._bits is not None else None
                _ops.launch_forward(d["q"][qs], d["k"][ks], d["v"][ks], self.scale, self.causal,
                                    self.dropout_p, sd, off, out=(d["o"][qs], lse_c), dropout_origin=origin,
                                    o_residual=res, keep_bits=bits, forward_only=False)
                self._ev_fwd[c].record(self._s_run)
                self._s_run.wait_event(self._ev_do[c])
                _ops.launch_backward(d["d_o"][qs], d["q"][qs], d["k"][ks], d["v"][ks], d["o"][qs],
                                     lse_c, self.scale, self.causal, self.dropout_p, sd, off,
                                     out=(d["dq"][qs], d["dk"][ks], d["dv"][ks]), workspace=self._ws[c],
                                     dropout_origin=origin, o_residual=res,
                                     keep_bits=(self._bits, True) if self._bits is not None else None)
                self._ev_bwd[c].record(self._s_run)
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(self._ev_fwd[c])
                self._copy(host_out["o"][qs], d["o"][qs], self._s_out)
                self._s_out.wait_event(self._ev_bwd[c])
                for n in ("dq", "dk", "dv"):
                    self._copy(host_out[n][sl(n)], d[n][sl(n)], self._s_out)
                self._ev_out[c].record(self._s_out)
        self._ev_done.record(self._s_out)
        caller.wait_event(self._ev_done)
        self._calls += 1

    def synchronize(self) -> None:
        """Block the host until the results of the last call are in host memory."""
        self._ev_done.synchronize()
        _ops.check_status(self.device, synchronize=False)      # the word is in host memory: no device sync


__all__ = ["HostAttentionStep", "chunk_bounds", "plan_chunks"]
