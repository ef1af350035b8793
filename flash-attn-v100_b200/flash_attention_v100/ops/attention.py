"""Autograd binding of the attention kernels.

Keeps the contract of the reference's EnhancedFlashAttentionV100Function
(ops/attention.py:36-333): the same 19 positional parameters of forward
(:50-72), a Tensor or (Tensor, Tensor) result (:229-232), and a backward that
returns one gradient slot per forward input (:313-333).  The Triton launches
inside are replaced by calls into libfa_b200.so.
"""
from __future__ import annotations

import contextlib
import ctypes
import threading
from typing import Any, Dict, Optional, Tuple, Union

import torch

from ..kernels import _cabi
from ..kernels.tile_table import dtype_enum
from ..utils import validate_inputs, _last_dim_contiguous

# --------------------------------------------------------------------------
# dropout stream state: (seed, offset) are host integers, never read back from
# the device (the reference draws them with two .item() syncs per call,
# kernels/forward_kernel.py:308-313, and does not keep them for backward).
# --------------------------------------------------------------------------
_rng_lock = threading.Lock()
_rng_state = {"seed": None, "offset": 0}


def set_dropout_seed(seed: int, offset: int = 0) -> None:
    """Fix the Philox key and the next call's counter word."""
    with _rng_lock:
        _rng_state["seed"] = int(seed) & 0xFFFFFFFFFFFFFFFF
        _rng_state["offset"] = int(offset) & 0xFFFFFFFFFFFFFFFF


def _next_dropout_stream() -> Tuple[int, int]:
    with _rng_lock:
        if _rng_state["seed"] is None:
            _rng_state["seed"] = torch.initial_seed() & 0xFFFFFFFFFFFFFFFF
        seed, offset = _rng_state["seed"], _rng_state["offset"]
        _rng_state["offset"] = (offset + 1) & 0xFFFFFFFFFFFFFFFF
    return seed, offset


_variant_override = threading.local()


@contextlib.contextmanager
def kernel_variant(name: str):
    """Force a kernel family ('auto', 'simt', 'tcgen05') inside the block."""
    table = {"auto": _cabi.VARIANT_AUTO, "simt": _cabi.VARIANT_SIMT, "tcgen05": _cabi.VARIANT_TCGEN05,
             "tcgen05_2pass": _cabi.VARIANT_TCGEN05_2PASS}
    old = getattr(_variant_override, "value", _cabi.VARIANT_AUTO)
    _variant_override.value = table[name]
    try:
        yield
    finally:
        _variant_override.value = old


# One int32 per device, in pinned host memory, that kernels set non-zero when a bounded device-side
# wait gives up (a protocol error, never expected).  The device writes it with a system-wide store;
# the host reads it without synchronising: the library on entry to every call (an earlier call's
# failure makes the next one return FA_ETIMEOUT), and check_status() below on request.  The
# reference's counterpart is the try/except around its launches (interface.py:331-348).
_status_words: Dict[int, torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _status_words[idx]


def check_status(device: Optional[torch.device] = None, synchronize: bool = True) -> None:
    """Raise if a kernel on `device` reported a timed-out wait.  `synchronize=True` waits for the
    device's queued work first, so that the answer covers it; False only looks at what has been
    reported so far (no synchronisation at all)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if synchronize:
        torch.cuda.synchronize(device)
    word = _status_word(device)
    code = int(word[0])
    if code != 0:
        word.zero_()
        raise RuntimeError(f"flash_attention_v100: a device-side wait timed out (status {code}); "
                           "results of the affected call are invalid")


def _tensor4(t: Optional[torch.Tensor]) -> _cabi.Tensor4:
    r = _cabi.Tensor4()
    if t is None or t.numel() == 0:
        r.ptr = None if t is None else (t.data_ptr() or None)
        if t is not None:
            r.stride_b, r.stride_n, r.stride_h = t.stride(0), t.stride(1), t.stride(2)
        return r
    assert t.stride(3) == 1
    r.ptr = t.data_ptr()
    r.stride_b, r.stride_n, r.stride_h = t.stride(0), t.stride(1), t.stride(2)
    return r


def _bias_operand(bias: Optional[torch.Tensor]):
    """(Tensor4, keep-alive tensor) for an additive bias: fp32, key index contiguous, size-1 batch /
    head / query dimensions passed as stride 0 (no expanded copy is made)."""
    if bias is None:
        return _cabi.Tensor4(), None
    bf = bias.detach()
    if bf.dtype != torch.float32:
        bf = bf.float()
    if bf.stride(3) != 1 and bf.shape[3] > 1:
        bf = bf.contiguous()
    r = _cabi.Tensor4()
    r.ptr = bf.data_ptr()
    r.stride_b = 0 if bf.shape[0] == 1 else bf.stride(0)
    r.stride_h = 0 if bf.shape[1] == 1 else bf.stride(1)
    r.stride_n = 0 if bf.shape[2] == 1 else bf.stride(2)
    return r, bf


def _lengths_operand(key_lengths: Optional[torch.Tensor], q: torch.Tensor):
    """(device pointer or None, keep-alive tensor) for per-batch key counts: int32, one per batch entry,
    on q's device."""
    if key_lengths is None:
        return None, None
    if key_lengths.dim() != 1 or key_lengths.shape[0] != q.shape[0]:
        raise ValueError(f"key_lengths must have shape ({q.shape[0]},), got {tuple(key_lengths.shape)}")
    kl = key_lengths.detach().to(device=q.device, dtype=torch.int32).contiguous()
    return kl.data_ptr(), kl


def _base_params(q, k, v, o, lse, scale, causal, dropout_p, seed, offset, causal_shift=0,
                 dropout_origin=None, variant=None) -> _cabi.Params:
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.q, p.k, p.v, p.o = _tensor4(q), _tensor4(k), _tensor4(v), _tensor4(o)
    p.lse = lse.data_ptr() or None
    p.B, p.Nq, p.H, p.D = q.shape
    p.Nk, p.Hkv = k.shape[1], k.shape[2]
    p.dtype = dtype_enum(q.dtype)
    p.causal = int(bool(causal))
    p.causal_shift = int(causal_shift) if causal else 0
    # an explicit kernel_variant() block wins; else the caller's choice (the autograd op's "speed" mode)
    override = getattr(_variant_override, "value", _cabi.VARIANT_AUTO)
    p.variant = override if override != _cabi.VARIANT_AUTO else (variant or _cabi.VARIANT_AUTO)
    p.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    p.scale = float(scale)
    p.dropout_p = float(dropout_p)
    p.seed, p.offset = int(seed), int(offset)
    p.stream = torch.cuda.current_stream(q.device).cuda_stream or None
    p.status_word = _status_word(q.device).data_ptr()
    if dropout_origin is not None:
        # the call is a slice of a larger problem: (batch offset, head offset, heads of the whole)
        p.rng_batch_offset, p.rng_head_offset, p.rng_heads = (int(x) for x in dropout_origin)
    return p


def _check_residual(o_residual: torch.Tensor, o: torch.Tensor) -> None:
    if o_residual.shape != o.shape or o_residual.dtype != o.dtype or o_residual.device != o.device or \
            (o_residual.numel() and o_residual.stride(3) != 1):
        raise ValueError("o_residual must match the output in shape, dtype and device, with a contiguous last dim")


def saves_output_residual(dtype: torch.dtype) -> bool:
    """Whether the autograd op keeps the output's rounding residual for its backward.  bf16 only: its 8
    significant bits make the saved output the largest error in dQ and dK of peaked attention rows."""
    return dtype == torch.bfloat16


# The keep bits of a call take Nq * Nk / 4 bytes per (batch, head) column (34 GB at B1 H32 N65536): beyond
# this size a buffer the caller did not supply is not allocated and the kernels draw their bits themselves.
KEEP_BITS_MAX_BYTES = 4 << 30


def _dropout_bits_operand(p, keep_bits, forward_only=False):
    """Point the call at a buffer for its dropout keep bits.  `keep_bits`: None (the kernels draw their
    bits themselves), "new" (allocate; returned for a later call to reuse), or (tensor, ready) with a
    uint8 tensor from an earlier call and whether that call has filled it."""
    if keep_bits is None:
        return None
    nbytes = int(_cabi.load().fa_b200_dropout_bits_bytes(ctypes.byref(p)))
    if nbytes == 0:
        return None                      # no dropout, or the CUDA-core kernels serve the call
    if isinstance(keep_bits, str):
        if nbytes > KEEP_BITS_MAX_BYTES:
            return None
        # a forward that no backward follows needs the query-major half only
        buf, ready = torch.empty(nbytes // 2 if forward_only else nbytes, dtype=torch.uint8, device="cuda:%d" % p.device), False
    else:
        buf, ready = keep_bits
        if buf.numel() < (nbytes // 2 if forward_only else nbytes):
            raise ValueError(f"keep-bit buffer holds {buf.numel()} bytes, the call needs {nbytes}")
    p.dropout_bits, p.dropout_bits_bytes, p.dropout_bits_ready = buf.data_ptr(), buf.numel(), int(bool(ready))
    return buf


def launch_forward(q, k, v, scale, causal, dropout_p=0.0, seed=0, offset=0, out=None, bias=None,
                   key_lengths=None, causal_shift=0, dropout_origin=None, o_residual=None, keep_bits=None,
                   forward_only=True):
    """o, lse <- fa_b200_fwd.  Counterpart of flash_attention_forward_triton_enhanced
    (kernels/forward_kernel.py:246-387); returns (o, lse).  `out=(o, lse)` writes into
    caller-owned buffers (o like q, lse (B, H, Nq) fp32 contiguous) instead of allocating.
    `o_residual` (a tensor like o) receives what rounding the output to its dtype dropped; handed
    to launch_backward it removes that rounding from the gradients.  `keep_bits="new"` (or a
    (uint8 tensor, ready) pair) has the call's dropout bits written to a buffer once instead of drawn
    inside the kernel; the call then returns (o, lse, buffer), and launch_backward given
    keep_bits=(buffer, True) reads the same bits (`forward_only=False` sizes the buffer for that)."""
    if out is not None:
        o, lse = out
    else:
        o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
    p = _base_params(q, k, v, o, lse, scale, causal, dropout_p, seed, offset, causal_shift, dropout_origin)
    p.bias, _keep = _bias_operand(bias)        # scores = scale * q.k + bias (CUDA-core kernels)
    p.kv_lengths, _keep_len = _lengths_operand(key_lengths, q)
    if o_residual is not None:
        _check_residual(o_residual, o)
        p.o_lo = _tensor4(o_residual)
    bits = _dropout_bits_operand(p, keep_bits, forward_only)
    rc = _cabi.load().fa_b200_fwd(ctypes.byref(p))
    _cabi.raise_for_status(rc, "fa_b200_fwd")
    if keep_bits is not None:
        return o, lse, bits
    return o, lse


def launch_backward(d_o, q, k, v, o, lse, scale, causal, dropout_p=0.0, seed=0, offset=0, out=None,
                    workspace=None, bias=None, d_scores=None, key_lengths=None, causal_shift=0,
                    dropout_origin=None, o_residual=None, fast=False, keep_bits=None):
    """dq, dk, dv <- fa_b200_bwd.  Counterpart of
    flash_attention_backward_triton_enhanced (kernels/backward_kernel.py:208-318).
    `out=(dq, dk, dv)` and `workspace` (uint8, at least fa_b200_bwd_workspace_bytes)
    use caller-owned buffers instead of allocating.  `fast`: allow the one-kernel backward where it
    is faster (D = 64); dQ is then summed in no fixed order and is not bit-reproducible.
    `keep_bits`: as in launch_forward; (buffer, True) reuses the bits the forward wrote."""
    d_o = _last_dim_contiguous(d_o)
    if out is not None:
        dq, dk, dv = out
    else:
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    p = _base_params(q, k, v, o, lse, scale, causal, dropout_p, seed, offset, causal_shift, dropout_origin,
                     variant=_cabi.VARIANT_TCGEN05 if fast else None)
    p.d_o, p.dq, p.dk, p.dv = _tensor4(d_o), _tensor4(dq), _tensor4(dk), _tensor4(dv)
    p.bias, _keep = _bias_operand(bias)
    p.kv_lengths, _keep_len = _lengths_operand(key_lengths, q)
    if o_residual is not None:
        _check_residual(o_residual, o)
        p.o_lo = _tensor4(o_residual)
    if d_scores is not None:
        # dense (B, H, Nq, Nk) fp32, zero-filled by the caller: receives d loss / d scores
        if d_scores.dtype != torch.float32 or not d_scores.is_contiguous() or \
                tuple(d_scores.shape) != (q.shape[0], q.shape[2], q.shape[1], k.shape[1]):
            raise ValueError("d_scores must be a contiguous fp32 (B, H, Nq, Nk) tensor")
        p.d_scores = d_scores.data_ptr()
    lib = _cabi.load()
    nbytes = int(lib.fa_b200_bwd_workspace_bytes(ctypes.byref(p)))
    if workspace is None:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    else:
        ws = workspace
        if ws.numel() < nbytes:
            raise ValueError(f"workspace holds {ws.numel()} bytes, the call needs {nbytes}")
    p.workspace, p.workspace_bytes = ws.data_ptr(), nbytes
    _bits = _dropout_bits_operand(p, keep_bits)
    rc = lib.fa_b200_bwd(ctypes.byref(p))
    _cabi.raise_for_status(rc, "fa_b200_bwd")
    return dq, dk, dv


def launch_combine(acc, part=None, lse_acc=None, lse_part=None, out=None, first=False):
    """fa_b200_combine: fold one block's partial result into the fp32 running total `acc` ((B, N, H, D)
    contiguous).  With lse_acc / lse_part ((B, H, N) fp32) the two are weighted by their log-sum-exps
    (attention outputs); without, they are added (gradients).  `first`: acc holds nothing yet.
    `out`: also write the new total there in out's dtype.  `part=None`: only that conversion."""
    like = part if part is not None else out
    if like is None:
        raise ValueError("launch_combine needs a partial, an output, or both")
    B, N, H, D = like.shape
    # acc may be a range of rows of a larger total: any batch stride, dense below it
    if acc.dtype != torch.float32 or acc.shape != like.shape or \
            (N > 0 and (acc.stride(3), acc.stride(2), acc.stride(1)) != (1, D, H * D)):
        raise ValueError("acc must be an fp32 tensor of the partial's shape, dense within a batch entry")
    if part is not None and out is not None and part.dtype != out.dtype:
        raise ValueError("part and out must have the same dtype")
    if lse_acc is not None and (lse_acc.dtype != torch.float32 or tuple(lse_acc.shape) != (B, H, N)
                                or (N > 1 and lse_acc.stride(2) != 1)):
        raise ValueError("lse_acc must be an fp32 (B, H, N) tensor with unit stride along N")
    if lse_part is not None and (lse_part.dtype != torch.float32 or not lse_part.is_contiguous()
                                 or tuple(lse_part.shape) != (B, H, N)):
        raise ValueError("lse_part must be a contiguous fp32 (B, H, N) tensor")
    p = _cabi.CombineParams()
    p.struct_bytes = ctypes.sizeof(_cabi.CombineParams)
    p.acc = acc.data_ptr()
    p.lse_acc = lse_acc.data_ptr() if lse_acc is not None else None
    p.lse_part = lse_part.data_ptr() if lse_part is not None else None
    p.part = _tensor4(_last_dim_contiguous(part)) if part is not None else _cabi.Tensor4()
    p.out = _tensor4(out) if out is not None else _cabi.Tensor4()
    p.B, p.N, p.H, p.D = acc.shape
    p.acc_stride_b = acc.stride(0)
    if lse_acc is not None:
        p.lse_stride_b, p.lse_stride_h = lse_acc.stride(0), lse_acc.stride(1)
    p.dtype = dtype_enum(like.dtype)
    p.first = int(bool(first))
    p.device = acc.device.index if acc.device.index is not None else torch.cuda.current_device()
    p.stream = torch.cuda.current_stream(acc.device).cuda_stream or None
    rc = _cabi.load().fa_b200_combine(ctypes.byref(p))
    _cabi.raise_for_status(rc, "fa_b200_combine")


class EnhancedFlashAttentionV100Function(torch.autograd.Function):
    """Attention as an autograd op; parameter list of reference ops/attention.py:50-72."""

    @staticmethod
    def forward(ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                causal: bool = False, dropout_p: float = 0.0, bias: Optional[torch.Tensor] = None,
                block_size_m: Optional[int] = None, block_size_n: Optional[int] = None,
                enable_autotuning: bool = True, return_softmax_lse: bool = False,
                enable_gradient_checkpointing: bool = False, enable_mixed_precision: bool = True,
                num_checkpoints: Optional[int] = None, memory_efficient: bool = True,
                performance_mode: str = "balanced", enable_multi_gpu: bool = False,
                world_size: int = 1, rank: int = 0, key_lengths: Optional[torch.Tensor] = None,
                causal_shift: int = 0, dropout_origin: Optional[Tuple[int, int, int]] = None,
                dropout_stream: Optional[Tuple[int, int]] = None
                ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        # block sizes, autotuning, checkpointing, mixed precision and the
        # multi-GPU arguments are accepted for source compatibility: tiles come
        # from the static table, the backward always recomputes P, and sharding
        # over GPUs happens above this op (interface.py).
        q, k, v, scale = validate_inputs(q, k, v, scale, bias, dropout_p)
        # dropout_origin / dropout_stream (after the reference's parameters): a call that is one shard of
        # a larger problem passes the shard's (batch offset, head offset, heads of the whole) and the
        # whole call's (seed, offset), and draws exactly the mask the whole call draws
        seed = offset = 0
        if dropout_p > 0.0:
            seed, offset = dropout_stream if dropout_stream is not None else _next_dropout_stream()
        # key_lengths (one int per batch entry, after the reference's 19 parameters): batch entry b
        # attends to its first key_lengths[b] keys only
        # causal_shift: key j is visible to query i iff j <= i + causal_shift (0: the reference's top-left
        # alignment; Nk - Nq: bottom-right)
        # the backward of a bf16 call also gets what rounding the output to bf16 dropped
        needs_grad = any(t.requires_grad for t in (q, k, v)) or (bias is not None and bias.requires_grad)
        o_lo = torch.empty_like(q) if (needs_grad and saves_output_residual(q.dtype)) else None
        # with dropout the call's keep bits are written to a buffer once; the backward reads the same bits
        res = launch_forward(q, k, v, scale, causal, dropout_p, seed, offset, bias=bias, key_lengths=key_lengths,
                             causal_shift=causal_shift, dropout_origin=dropout_origin, o_residual=o_lo,
                             keep_bits="new" if dropout_p > 0.0 else None, forward_only=not needs_grad)
        o, lse = res[0], res[1]
        ctx.keep_bits = res[2] if (len(res) > 2 and needs_grad) else None
        ctx.dropout_origin = dropout_origin
        ctx.has_bias, ctx.has_residual = bias is not None, o_lo is not None
        # performance_mode "speed" (the public entry's optimization_strategy) opts into the fastest
        # backward, whose dQ is not bit-reproducible at D = 64; every other mode is deterministic
        ctx.fast = performance_mode == "speed"
        ctx.save_for_backward(q, k, v, o, lse, *([bias] if bias is not None else []),
                              *([o_lo] if o_lo is not None else []))
        ctx.key_lengths = key_lengths
        ctx.causal_shift = int(causal_shift)
        ctx.scale, ctx.causal, ctx.dropout_p = scale, bool(causal), float(dropout_p)
        ctx.seed, ctx.offset = seed, offset
        ctx.return_softmax_lse = bool(return_softmax_lse)
        if return_softmax_lse:
            ctx.mark_non_differentiable(lse)
            return o, lse
        return o

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor, grad_softmax_lse: Optional[torch.Tensor] = None):
        q, k, v, o, lse, *rest = ctx.saved_tensors
        bias = rest[0] if ctx.has_bias else None
        o_lo = rest[-1] if ctx.has_residual else None
        d_scores = grad_bias = None
        if bias is not None and ctx.needs_input_grad[6]:
            # the reference returns zeros here (ops/attention.py:297-301); this is the real gradient:
            # d loss / d scores, dense, summed over the dimensions the bias broadcasts
            d_scores = torch.zeros(q.shape[0], q.shape[2], q.shape[1], k.shape[1], dtype=torch.float32,
                                   device=q.device)
        dq, dk, dv = launch_backward(grad_output, q, k, v, o, lse, ctx.scale, ctx.causal,
                                     ctx.dropout_p, ctx.seed, ctx.offset, bias=bias, d_scores=d_scores,
                                     key_lengths=ctx.key_lengths, causal_shift=ctx.causal_shift,
                                     dropout_origin=ctx.dropout_origin, o_residual=o_lo, fast=ctx.fast and bias is None,
                                     keep_bits=(ctx.keep_bits, True) if ctx.keep_bits is not None else None)
        if d_scores is not None:
            dims = [i for i in range(4) if bias.shape[i] == 1 and d_scores.shape[i] != 1]
            grad_bias = (d_scores.sum(dim=dims, keepdim=True) if dims else d_scores).to(bias.dtype)
        return (dq if ctx.needs_input_grad[0] else None,
                dk if ctx.needs_input_grad[1] else None,
                dv if ctx.needs_input_grad[2] else None, None, None, None, grad_bias) + (None,) * 16


def flash_attention_forward_enhanced(q, k, v, scale: Optional[float] = None, causal: bool = False,
                                     dropout_p: float = 0.0, bias: Optional[torch.Tensor] = None,
                                     enable_multi_gpu: bool = False, performance_mode: str = "balanced",
                                     **kwargs) -> torch.Tensor:
    """No-grad forward (reference ops/attention.py:464-533).  With
    return_softmax_lse=True in kwargs returns (o, lse)."""
    q, k, v, scale = validate_inputs(q, k, v, scale, bias, dropout_p)
    seed = offset = 0
    if dropout_p > 0.0:
        seed, offset = kwargs.get("dropout_stream") or _next_dropout_stream()
    with torch.no_grad():
        o, lse = launch_forward(q, k, v, scale, causal, dropout_p, seed, offset, bias=bias,
                                key_lengths=kwargs.get("key_lengths"), dropout_origin=kwargs.get("dropout_origin"),
                                o_residual=kwargs.get("output_residual"),
                                keep_bits="new" if dropout_p > 0.0 else None)[:2]
    return (o, lse) if kwargs.get("return_softmax_lse", False) else o


def flash_attention_backward_enhanced(grad_output, q, k, v, output, lse, max_vals=None,
                                      scale: Optional[float] = None, causal: bool = False,
                                      enable_multi_gpu: bool = False, **kwargs
                                      ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Explicit backward (reference ops/attention.py:536-600).  `max_vals` is
    accepted and ignored: the kernels recompute P from the log-sum-exp alone.
    kwargs: dropout_p and dropout_stream=(seed, offset) to replay a mask; output_residual (the tensor the
    forward filled when it was given one: removes the output's rounding from dQ and dK); bias (the
    forward's additive bias) and d_scores (zero-filled fp32 (B, H, Nq, Nk) that receives d loss / d scores)."""
    q, k, v, scale = validate_inputs(q, k, v, scale, kwargs.get("bias"), kwargs.get("dropout_p", 0.0))
    seed, offset = kwargs.get("dropout_stream", (0, 0))
    with torch.no_grad():
        return launch_backward(grad_output, q, k, v, _last_dim_contiguous(output), lse.contiguous(),
                               scale, causal, kwargs.get("dropout_p", 0.0), seed, offset,
                               bias=kwargs.get("bias"), d_scores=kwargs.get("d_scores"),
                               key_lengths=kwargs.get("key_lengths"), dropout_origin=kwargs.get("dropout_origin"),
                               o_residual=kwargs.get("output_residual"),
                               fast=kwargs.get("performance_mode") == "speed")


def compare_with_pytorch_attention_enhanced(q, k, v, causal: bool = False,
                                            bias: Optional[torch.Tensor] = None, dropout_p: float = 0.0,
                                            atol: float = 1e-4, rtol: float = 1e-4) -> Dict[str, Any]:
    """Compare the kernels with PyTorch's scaled_dot_product_attention on the
    GPU; same result keys as the reference (ops/attention.py:603-717)."""
    if dropout_p != 0.0:
        raise ValueError("comparison is only defined without dropout (different random streams)")
    import torch.nn.functional as F
    scale = q.shape[-1] ** -0.5
    flash = flash_attention_forward_enhanced(q, k, v, scale, causal, 0.0, bias)
    ref = F.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                         v.transpose(1, 2).float(), is_causal=causal,
                                         scale=scale).transpose(1, 2)
    diff = (flash.float() - ref).abs()
    denom = ref.abs().clamp_min(1e-6)
    cos = F.cosine_similarity(flash.float().flatten(), ref.flatten(), dim=0).item()
    stats = lambda t: {"mean": t.float().mean().item(), "std": t.float().std().item(),
                       "min": t.float().min().item(), "max": t.float().max().item()}
    return {
        "allclose": bool(torch.allclose(flash.float(), ref, atol=atol, rtol=rtol)),
        "max_absolute_difference": diff.max().item(),
        "mean_absolute_difference": diff.mean().item(),
        "max_relative_difference": (diff / denom).max().item(),
        "mean_relative_difference": (diff / denom).mean().item(),
        "cosine_similarity": cos, "atol": atol, "rtol": rtol,
        "flash_output_stats": stats(flash), "reference_output_stats": stats(ref),
        "input_shape": q.shape,
        "configuration": {"causal": causal, "dropout_p": dropout_p, "has_bias": bias is not None,
                          "dtype": str(q.dtype), "device": str(q.device)},
    }


@contextlib.contextmanager
def gradient_checkpointing_mode(enable: bool = True):
    """Placeholder kept from the reference (ops/attention.py:721-726): the
    backward already recomputes the probabilities, nothing is checkpointed."""
    yield


@contextlib.contextmanager
def mixed_precision_mode(enable: bool = True):
    """Reference ops/attention.py:729-736: run the block under autocast."""
    if enable and torch.cuda.is_available():
        with torch.autocast("cuda"):
            yield
    else:
        yield


FlashAttentionV100Function = EnhancedFlashAttentionV100Function
flash_attention_forward = flash_attention_forward_enhanced
flash_attention_backward = flash_attention_backward_enhanced
compare_with_pytorch_attention = compare_with_pytorch_attention_enhanced

def next_dropout_stream() -> Tuple[int, int]:
    """(seed, offset) the next dropout call would use; advances the counter.  A caller that splits one
    problem into several calls draws it once and hands it to every part (`dropout_stream=`)."""
    return _next_dropout_stream()


__all__ = [
    "EnhancedFlashAttentionV100Function", "next_dropout_stream", "flash_attention_forward_enhanced",
    "flash_attention_backward_enhanced", "compare_with_pytorch_attention_enhanced",
    "gradient_checkpointing_mode", "mixed_precision_mode", "FlashAttentionV100Function",
    "flash_attention_forward", "flash_attention_backward", "compare_with_pytorch_attention",
    "set_dropout_seed", "kernel_variant", "launch_forward", "launch_backward", "check_status",
]
