"""Host-side helpers: input validation and small integer utilities.

validate_inputs mirrors the reference's validate_inputs_enhanced
(utils.py:31-160): same checks in the same order, same exception types and
messages for the cheap checks.  The reference's full-tensor NaN/Inf/abs-max
scans (utils.py:227-254) are dropped: they synchronise the device on every
call.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .config import SUPPORTED_DTYPES


def cdiv(a: int, b: int) -> int:
    """Ceiling division (reference utils.py:606-623 helpers)."""
    return -(-a // b)


def _last_dim_contiguous(t: torch.Tensor) -> torch.Tensor:
    """Kernels need unit stride on the head dim and 16-byte aligned rows; head-
    or batch-sliced views pass through untouched, anything else is packed."""
    if t.numel() == 0:
        return t
    es = t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all((s * es) % 16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def validate_inputs(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    scale: Optional[float] = None, bias: Optional[torch.Tensor] = None,
                    dropout_p: float = 0.0, require_cuda: bool = True
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, float]:
    """Check (q, k, v) and return them kernel-ready together with the scale.

    Same rules as reference utils.py:56-153; raises TypeError/ValueError with
    the reference's messages.
    """
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        raise TypeError("q, k, v must be torch.Tensor instances")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("Input tensors must be 4-dimensional [batch, seq_len, num_heads, head_dim]")
    b, nq, hq, dq = q.shape
    bk, nk, hk, dk = k.shape
    bv, nv, hv, dv = v.shape
    if not (b == bk == bv):
        raise ValueError(f"Batch sizes must match across Q, K, V. Got Q: {b}, K: {bk}, V: {bv}")
    if nk != nv:
        raise ValueError(f"Sequence lengths of K and V must match. Got K: {nk}, V: {nv}")
    if not (dq == dk == dv):
        raise ValueError(f"Head dimensions must match across Q, K, V. Got Q: {dq}, K: {dk}, V: {dv}")
    if hk == 0 or hv == 0 or hq % hk != 0 or hq % hv != 0:
        raise ValueError(f"Number of query heads ({hq}) must be divisible by "
                         f"number of key heads ({hk}) and value heads ({hv})")
    if hk != hv:
        raise ValueError(f"Number of key heads ({hk}) must equal number of value heads ({hv})")
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError(f"All tensors must have the same dtype. Got Q: {q.dtype}, K: {k.dtype}, V: {v.dtype}")
    if q.dtype not in SUPPORTED_DTYPES:
        supported = ", ".join(str(dt) for dt in SUPPORTED_DTYPES)
        raise ValueError(f"Unsupported dtype {q.dtype}. Supported types: {supported}")
    if not (q.device == k.device == v.device):
        raise ValueError(f"All tensors must be on the same device. Got Q: {q.device}, K: {k.device}, V: {v.device}")
    if require_cuda and q.device.type != "cuda":
        # the reference warns and carries on when CUDA exists (utils.py:119-127);
        # there is no CPU path here, so this is always an error
        raise ValueError("Flash Attention V100 requires CUDA tensors")
    if bias is not None:
        # reference interface.py:505-525
        if not isinstance(bias, torch.Tensor):
            raise TypeError("bias must be a torch.Tensor")
        b, nq, h = q.shape[0], q.shape[1], q.shape[2]
        nk = k.shape[1]
        expected = [(b, h, nq, nk), (1, h, nq, nk), (b, 1, nq, nk), (1, 1, nq, nk),
                    (b, 1, 1, nk), (1, 1, 1, nk)]       # the last two: key-padding masks (broadcast over queries)
        if tuple(bias.shape) not in expected:
            raise ValueError(f"bias shape {tuple(bias.shape)} not compatible with attention shape. "
                             f"Expected one of: {expected}")
        if bias.device != q.device:
            raise ValueError("bias must be on the same device as input tensors")
    if not (0.0 <= dropout_p < 1.0):
        raise ValueError(f"dropout_p must be in [0.0, 1.0), got {dropout_p}")
    if dq > 128:
        raise ValueError(f"head_dim {dq} is not supported (maximum 128)")
    if scale is None:
        scale = dq ** -0.5                       # reference utils.py:148-149
    return _last_dim_contiguous(q), _last_dim_contiguous(k), _last_dim_contiguous(v), float(scale)


__all__ = ["cdiv", "validate_inputs"]
