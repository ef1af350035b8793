"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference
legs may import this module; the shipped package never does.

What it restates: the reference's PyTorch math attention path,
`flash_attention_v100` in the reference's __init__.py:30-55 (twin with
dropout in tests/test_attention.py:30-87):

    q,k,v (B,N,H,D) -> transpose(1,2) -> matmul(q*scale, k^T)
      -> causal: masked_fill_(triu(ones(N,N), diagonal=1), -inf)
      -> softmax(-1) -> [dropout] -> matmul(P, v) -> transpose(1,2)

Pinned against the reference itself: tests/golden/make_golden.py imports the
reference package in the build container, runs that function (and autograd
through it) on seeded inputs and stores the outputs; tests/test_oracle.py
checks this restatement against those fixtures.

What it adds (the reference's math path has none of these; its LSE output is
a dummy zero tensor, tests/test_attention.py:81-85, interface.py:484-488):
  * lse = logsumexp over the same scaled, masked scores, (B,H,Nq) fp32;
  * gradients, by autograd through the restated forward and, independently,
    by closed-form flash-attention backward formulas;
  * dropout with an injected keep mask: P_drop = P * keep / (1 - p), applied
    after softmax normalisation as the reference twin does with F.dropout
    (tests/test_attention.py:69-73);
  * a precision rule: inputs are the dtype-rounded tensors up-cast to fp32
    (or fp64), so the oracle sees bit-identical values to the GPU kernels;
  * chunking over (batch, head) so large configs do not materialise
    B*H*N*N scores at once (exact: heads are independent).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def _scores(q, k, scale, causal, bias=None, causal_shift=0):
    """(B,H,Nq,Nk) scaled, masked scores; reference __init__.py:36-48.  `bias`
    (broadcastable to (B,H,Nq,Nk)) is added after the scaling and before the
    causal mask, as the reference's test twin does (tests/test_attention.py:48-58)
    and its forward kernel intends (kernels/forward_kernel.py:171-176).
    `causal_shift` moves the mask's diagonal: key j is hidden iff j > i + shift.
    0 is the reference's mask; the reference has no other (Nk - Nq gives the
    bottom-right alignment, which has no counterpart there)."""
    qt = q.transpose(1, 2)
    kt = k.transpose(1, 2)
    hq, hk = qt.shape[1], kt.shape[1]
    if hq != hk:  # grouped K/V heads: query head h reads kv head h // (H/Hkv)
        kt = kt.repeat_interleave(hq // hk, dim=1)
    s = torch.matmul(qt * scale, kt.transpose(-2, -1))
    if bias is not None:
        s = s + bias.to(s.dtype)
    if causal:
        nq, nk = s.shape[-2], s.shape[-1]
        # reference: triu(ones(seq, seq), diagonal=1) -> key j masked iff j > i
        mask = torch.triu(torch.ones(nq, nk, device=s.device), diagonal=1 + int(causal_shift)).bool()
        s = s.masked_fill(mask, float("-inf"))
    return s


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *,
                      causal: bool = False, scale: Optional[float] = None,
                      dropout_p: float = 0.0, keep_mask: Optional[torch.Tensor] = None,
                      compute_dtype: torch.dtype = torch.float32, bias: Optional[torch.Tensor] = None,
                      causal_shift: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense attention, returns (O (B,Nq,H,D), LSE (B,H,Nq)) in compute_dtype.

    Follows reference __init__.py:30-55 step by step; `keep_mask` (B,H,Nq,Nk)
    of {0,1} with `dropout_p` follows tests/test_attention.py:69-73
    (probabilities are dropped after normalisation and scaled by 1/(1-p)).
    """
    q = q.to(compute_dtype)
    k = k.to(compute_dtype)
    v = v.to(compute_dtype)
    if scale is None:
        scale = q.shape[-1] ** -0.5          # reference __init__.py:32
    s = _scores(q, k, scale, causal, bias, causal_shift)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)             # reference __init__.py:50
    if keep_mask is not None:
        p = p * keep_mask.to(p.dtype) / (1.0 - dropout_p)
    vt = v.transpose(1, 2)
    if vt.shape[1] != p.shape[1]:
        vt = vt.repeat_interleave(p.shape[1] // vt.shape[1], dim=1)
    o = torch.matmul(p, vt).transpose(1, 2)  # reference __init__.py:51-54
    return o.contiguous(), lse


def attention_forward_backward(q, k, v, d_o, *, causal=False, scale=None, dropout_p=0.0,
                               keep_mask=None, compute_dtype=torch.float32, bias=None, causal_shift=0):
    """(O, LSE, dQ, dK, dV) with gradients from autograd through the restated
    forward (the same route a user of the reference's math path takes).  With a
    `bias` that requires grad, its gradient is left in bias.grad."""
    q = q.detach().to(compute_dtype).requires_grad_(True)
    k = k.detach().to(compute_dtype).requires_grad_(True)
    v = v.detach().to(compute_dtype).requires_grad_(True)
    o, lse = attention_forward(q, k, v, causal=causal, scale=scale, dropout_p=dropout_p,
                               keep_mask=keep_mask, compute_dtype=compute_dtype, bias=bias,
                               causal_shift=causal_shift)
    o.backward(d_o.to(compute_dtype))
    return o.detach(), lse.detach(), q.grad, k.grad, v.grad


def attention_backward_closed_form(q, k, v, o, lse, d_o, *, causal=False, scale=None,
                                   dropout_p=0.0, keep_mask=None, compute_dtype=torch.float64):
    """Closed-form backward (no autograd): the recomputation the kernels do.

        P = exp(S - lse);  Z = keep/(1-p);  delta = rowsum(dO o O)
        dV = (P o Z)^T dO;  dP = dO V^T;  dS = P o (dP o Z - delta)
        dQ = scale * dS K;  dK = scale * dS^T Q
    Used to cross-check the autograd route and the C restatement.
    """
    cd = compute_dtype
    q, k, v, o, d_o = (t.to(cd) for t in (q, k, v, o, d_o))
    if scale is None:
        scale = q.shape[-1] ** -0.5
    g = q.shape[2] // k.shape[2]
    s = _scores(q, k, scale, causal)
    p = torch.exp(s - lse.to(cd).unsqueeze(-1))
    z = torch.ones_like(p) if keep_mask is None else keep_mask.to(cd) / (1.0 - dropout_p)
    dot = d_o.transpose(1, 2)                      # (B,H,Nq,D)
    delta = (dot * o.transpose(1, 2)).sum(-1, keepdim=True)
    vt = v.transpose(1, 2).repeat_interleave(g, dim=1)
    kt = k.transpose(1, 2).repeat_interleave(g, dim=1)
    dv = torch.matmul((p * z).transpose(-2, -1), dot)
    dp = torch.matmul(dot, vt.transpose(-2, -1))
    ds = p * (dp * z - delta)
    dq = scale * torch.matmul(ds, kt)
    dk = scale * torch.matmul(ds.transpose(-2, -1), q.transpose(1, 2))
    if g > 1:
        b, h, nk, d = dk.shape
        dk = dk.view(b, h // g, g, nk, d).sum(2)
        dv = dv.view(b, h // g, g, nk, d).sum(2)
    return dq.transpose(1, 2).contiguous(), dk.transpose(1, 2).contiguous(), dv.transpose(1, 2).contiguous()


def chunked(fn, q, k, v, *rest, heads_per_chunk=1, **kw):
    """Run `fn` over (batch, head-group) chunks and stitch the results.

    `fn` is attention_forward or attention_forward_backward; tensors in `rest`
    (dO) share q's layout.  keep_mask, if given in kw, is sliced alike.  Only
    for equal q/kv head counts.
    """
    b_, _, h_, _ = q.shape
    keep = kw.pop("keep_mask", None)
    outs = None
    for b in range(b_):
        for h0 in range(0, h_, heads_per_chunk):
            sl = (slice(b, b + 1), slice(None), slice(h0, h0 + heads_per_chunk))
            km = None if keep is None else keep[b:b + 1, h0:h0 + heads_per_chunk]
            res = fn(q[sl], k[sl], v[sl], *[r[sl] for r in rest], keep_mask=km, **kw)
            if outs is None:
                outs = []
                for i, r in enumerate(res):
                    if i == 1:   # lse (B,H,Nq)
                        outs.append(torch.empty(b_, h_, q.shape[1], dtype=r.dtype))
                    else:
                        ref = q if i in (0, 2) else k
                        outs.append(torch.empty(ref.shape, dtype=r.dtype))
            for i, r in enumerate(res):
                if i == 1:
                    outs[i][b:b + 1, h0:h0 + heads_per_chunk] = r
                else:
                    outs[i][sl] = r
    return tuple(outs)


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    """||x - ref||_2 / ||ref||_2 in float64."""
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = ref.norm().item()
    num = (x - ref).norm().item()
    if den == 0.0:
        return 0.0 if num == 0.0 else math.inf
    return num / den
