"""Multi-head attention layer on top of flash_attention_v100.

Counterpart of the reference's EnhancedMultiHeadAttention
(examples/basic_usage.py:48-255): the same constructor arguments, the same
parameter names (q_proj, k_proj, v_proj, out_proj: state dicts are
interchangeable) and the same forward signature.  Differences that follow from
the kernels underneath:

* the projections' outputs are handed to the attention op as (B, N, H, D)
  views, no transposes or copies;
* a boolean key-padding mask on its own (no attn_mask, no causal mask) costs no bias at all:
  attention does not depend on the order of the keys, so the kept keys of every batch entry are
  moved to the front (one gather of K and V, undone for dK and dV by autograd) and the call runs
  on the tensor-core kernels with per-batch key counts;
* other masks become the smallest bias that expresses them - a key-padding mask is a
  (B, 1, 1, Nk) bias, a 2-D attn_mask a (1, 1, Nq, Nk) one - instead of a dense
  (B, H, Nq, Nk) tensor (reference :228-250); boolean masks hide where True,
  float masks are added to the scores;
* attention weights are never materialised: need_weights=True warns and
  returns None (the reference returns a tensor of zeros, :219-223).
"""
from __future__ import annotations

import warnings
from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn

from .interface import flash_attention_v100


def masks_to_bias(attn_mask: Optional[torch.Tensor], key_padding_mask: Optional[torch.Tensor],
                  batch: int, seq_q: int, seq_k: int) -> Optional[torch.Tensor]:
    """fp32 bias broadcastable to (B, H, Nq, Nk), or None.

    attn_mask: (Nq, Nk) or (B, Nq, Nk); key_padding_mask: (B, Nk).  Boolean
    masks hide the positions that are True; floating masks are added."""
    def as_additive(m: torch.Tensor) -> torch.Tensor:
        if m.dtype == torch.bool:
            return torch.zeros(m.shape, dtype=torch.float32, device=m.device).masked_fill_(m, float("-inf"))
        return m.float()

    bias = None
    if attn_mask is not None:
        if attn_mask.dim() == 2:
            if tuple(attn_mask.shape) != (seq_q, seq_k):
                raise ValueError(f"attn_mask shape {tuple(attn_mask.shape)}, expected {(seq_q, seq_k)}")
            bias = as_additive(attn_mask).view(1, 1, seq_q, seq_k)
        elif attn_mask.dim() == 3:
            if tuple(attn_mask.shape) != (batch, seq_q, seq_k):
                raise ValueError(f"attn_mask shape {tuple(attn_mask.shape)}, expected {(batch, seq_q, seq_k)}")
            bias = as_additive(attn_mask).view(batch, 1, seq_q, seq_k)
        else:
            raise ValueError("attn_mask must have 2 or 3 dimensions")
    if key_padding_mask is not None:
        if tuple(key_padding_mask.shape) != (batch, seq_k):
            raise ValueError(f"key_padding_mask shape {tuple(key_padding_mask.shape)}, expected {(batch, seq_k)}")
        pad = as_additive(key_padding_mask).view(batch, 1, 1, seq_k)
        bias = pad if bias is None else bias + pad          # broadcasts to (B, 1, Nq, Nk)
    return bias


def compact_keys(k: torch.Tensor, v: torch.Tensor, key_padding_mask: torch.Tensor
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Kept keys first: (k', v', counts) such that attention over the first counts[b] keys of k'[b], v'[b]
    equals attention over k[b], v[b] with the keys where key_padding_mask[b] is True hidden.

    k, v: (B, Nk, H, D); key_padding_mask: (B, Nk) bool.  The kept keys keep their order (a stable sort
    of the mask); nothing is read back to the host.  An entry whose keys are all hidden keeps a count
    of 1 (it attends to its first key) instead of producing the NaN a softmax over nothing gives."""
    if key_padding_mask.dtype != torch.bool or key_padding_mask.dim() != 2 or \
            tuple(key_padding_mask.shape) != (k.shape[0], k.shape[1]):
        raise ValueError("key_padding_mask must be a boolean (B, Nk) tensor")
    order = torch.argsort(key_padding_mask.to(torch.uint8), dim=1, stable=True)
    counts = (~key_padding_mask).sum(dim=1).clamp_(min=1).to(torch.int32)
    index = order.view(order.shape[0], order.shape[1], 1, 1).expand(-1, -1, k.shape[2], k.shape[3])
    return k.gather(1, index), v.gather(1, index), counts


class EnhancedMultiHeadAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 batch_first: bool = True, optimization_strategy: str = "balanced",
                 enable_multi_gpu: bool = True, enable_gradient_checkpointing: bool = False,
                 enable_performance_monitoring: bool = False):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.head_dim = embed_dim // num_heads
        self.dropout = dropout
        self.batch_first = batch_first
        self.optimization_strategy = optimization_strategy
        self.enable_multi_gpu = enable_multi_gpu
        # accepted for source compatibility: the backward always recomputes the probabilities
        self.enable_gradient_checkpointing = enable_gradient_checkpointing
        self.enable_performance_monitoring = enable_performance_monitoring
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=bias)
        self.forward_count = 0
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for proj in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            nn.init.xavier_uniform_(proj.weight)
            if proj.bias is not None:
                nn.init.zeros_(proj.bias)

    def forward(self, query: torch.Tensor, key: Optional[torch.Tensor] = None,
                value: Optional[torch.Tensor] = None, key_padding_mask: Optional[torch.Tensor] = None,
                attn_mask: Optional[torch.Tensor] = None, need_weights: bool = False,
                average_attn_weights: bool = True, is_causal: bool = False,
                key_lengths: Optional[torch.Tensor] = None
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Reference signature plus key_lengths (B,): for right-padded batches, the number of real keys
        of each batch entry; the call stays on the tensor-core kernels and skips the padding's key
        blocks.  A boolean key_padding_mask alone (no attn_mask, is_causal False) gets there too, by moving
        the kept keys to the front (compact_keys); combined with other masks, or as a float mask, it
        becomes a bias and runs on the CUDA-core kernels."""
        if not self.batch_first:
            query = query.transpose(0, 1)
            key = key.transpose(0, 1) if key is not None else None
            value = value.transpose(0, 1) if value is not None else None
        key = query if key is None else key
        value = key if value is None else value
        batch, seq_q, _ = query.shape
        seq_k = key.shape[1]
        # (B, N, E) -> (B, N, H, D): a view of the projection's output, which the kernels read in place
        q = self.q_proj(query).view(batch, seq_q, self.num_heads, self.head_dim)
        k = self.k_proj(key).view(batch, seq_k, self.num_heads, self.head_dim)
        v = self.v_proj(value).view(batch, seq_k, self.num_heads, self.head_dim)
        if key_padding_mask is not None and key_padding_mask.dtype == torch.bool and attn_mask is None \
                and not is_causal and key_lengths is None:
            if tuple(key_padding_mask.shape) != (batch, seq_k):
                raise ValueError(f"key_padding_mask shape {tuple(key_padding_mask.shape)}, expected {(batch, seq_k)}")
            k, v, key_lengths = compact_keys(k, v, key_padding_mask)
            key_padding_mask = None
        bias = masks_to_bias(attn_mask, key_padding_mask, batch, seq_q, seq_k)
        if need_weights:
            warnings.warn("need_weights=True: attention weights are never materialised by these kernels; "
                          "None is returned for them.", UserWarning)
        self.forward_count += 1
        out = flash_attention_v100(q, k, v, causal=is_causal, dropout_p=self.dropout if self.training else 0.0,
                                   bias=bias, optimization_strategy=self.optimization_strategy,
                                   enable_multi_gpu=self.enable_multi_gpu,
                                   enable_profiling=self.enable_performance_monitoring, key_lengths=key_lengths)
        out = self.out_proj(out.reshape(batch, seq_q, self.embed_dim))
        if not self.batch_first:
            out = out.transpose(0, 1)
        return out, None

    def get_performance_stats(self) -> Optional[Dict[str, Any]]:
        """Reference :252-256.  Only the call count is kept here; time the layer with CUDA events."""
        if not self.enable_performance_monitoring:
            return None
        return {"forward_count": self.forward_count}


__all__ = ["EnhancedMultiHeadAttention", "masks_to_bias", "compact_keys"]
