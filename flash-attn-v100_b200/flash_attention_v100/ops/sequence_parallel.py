"""Sequence-parallel (ring) attention: every rank holds one slice of the sequence.

The reference names this strategy but does not implement it: its
_execute_sequence_parallel warns and runs on one GPU (interface.py:437-450;
the strategy table is config.py:153-157).  Here rank r keeps its queries
q_r (B, n, H, D) and the key/value blocks travel around the ring
r -> r + 1: at step t rank r holds block (r - t) mod G, runs one ordinary
forward (or backward) call on (q_r, block) and folds the result into a running
total with fa_b200_combine:

    forward   O_r, LSE_r = merge over blocks of (O_part, LSE_part)
    backward  dQ_r = sum over blocks of dQ_part;  dK_b, dV_b = sum over ranks,
              accumulated in fp32 buffers that travel with their block and are
              back home after G hops

The block calls use the final O_r and LSE_r (P = exp(S - LSE) and
delta = rowsum(dO * O) are then those of the whole row), so the backward needs
no second softmax pass.  Under a causal mask block b is hidden from rank r when
b > r, takes the diagonal mask when b == r and none when b < r; hidden blocks
are neither computed nor sent on.  With contiguous slices rank r then computes
r + 1 of the G blocks, so the last rank sets the pace.  layout="zigzag" evens that
out: the sequence is cut into 2 G chunks and rank r holds chunks r and
2 G - 1 - r (zigzag_split / zigzag_merge), so that every (rank, block) pair has
the same visible area: the whole slice under the diagonal mask for the rank's
own block, all queries against the block's first chunk when the block comes from
a lower rank, the second chunk's queries against the whole block when it comes
from a higher one.

The next block's transfer is posted before the current block's kernels are
launched, into the other half of a double buffer in this GPU's own memory:
kernels only ever read local memory.  Every transfer is a batch of one send
and one receive, so the ring cannot deadlock on a single communication stream.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import attention as _ops


LAYOUTS = ("contiguous", "zigzag")


def ring_schedule(rank: int, world: int, causal: bool, layout: str = "contiguous") -> List[Tuple[int, str]]:
    """[(block, mode)] for steps 0 .. world - 1 of `rank`.  mode: 'full' (no mask), 'causal' (diagonal
    mask), 'skip' (nothing visible), and for the zigzag layout 'lower' (all queries, the block's first
    chunk of keys) and 'upper' (the second chunk's queries, all of the block's keys)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a ring of {world}")
    if layout not in LAYOUTS:
        raise ValueError(f"layout must be one of {LAYOUTS}")
    steps = []
    for t in range(world):
        block = (rank - t) % world
        if not causal:
            mode = "full"
        elif block == rank:
            mode = "causal"
        elif layout == "zigzag":
            mode = "lower" if block < rank else "upper"
        else:
            mode = "full" if block < rank else "skip"
        steps.append((block, mode))
    return steps


def _step_ranges(mode: str, n: int) -> Tuple[slice, slice]:
    """(query rows, key rows) of the local slice / the visiting block that a step's call covers."""
    if mode == "lower":
        return slice(None), slice(0, n // 2)
    if mode == "upper":
        return slice(n // 2, None), slice(None)
    return slice(None), slice(None)


def zigzag_split(x: torch.Tensor, world: int, rank: int, dim: int = 1) -> torch.Tensor:
    """This rank's slice of a whole-sequence tensor under the zigzag layout: chunks rank and
    2 world - 1 - rank of 2 world equal chunks along `dim`."""
    if x.shape[dim] % (2 * world) != 0:
        raise ValueError(f"the sequence length {x.shape[dim]} must be a multiple of {2 * world}")
    chunks = x.chunk(2 * world, dim=dim)
    return torch.cat((chunks[rank], chunks[2 * world - 1 - rank]), dim=dim)


def zigzag_merge(slices, dim: int = 1) -> torch.Tensor:
    """Inverse of zigzag_split over the slices of ranks 0 .. world - 1 (in that order)."""
    world = len(slices)
    chunks = [None] * (2 * world)
    for r, s in enumerate(slices):
        chunks[r], chunks[2 * world - 1 - r] = s.chunk(2, dim=dim)
    return torch.cat(chunks, dim=dim)


def kv_transfer(rank: int, world: int, causal: bool, step: int, layout: str = "contiguous") -> Tuple[bool, bool]:
    """(send, receive): does `rank` pass its current block on after `step`, and does it get one?
    Without a mask every block visits every rank.  Under a causal mask block b is only of use to
    ranks above b, so it stops at the last rank and blocks that wrapped around are never sent."""
    if step >= world - 1:
        return False, False
    if not causal or layout == "zigzag":
        return True, True
    send = rank - step >= 0 and rank + 1 < world
    recv = rank >= 1 and rank - 1 - step >= 0
    return send, recv


class DistributedRing:
    """The ring over a torch.distributed process group (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, group=None):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("sequence-parallel attention needs an initialised torch.distributed")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        to_global = (lambda r: r) if group is None else (lambda r: dist.get_global_rank(group, r))
        self.next = to_global((self.rank + 1) % self.world)
        self.prev = to_global((self.rank - 1) % self.world)

    def exchange(self, send: Optional[torch.Tensor], recv: Optional[torch.Tensor]):
        """Post `send` to the next rank and `recv` from the previous one as one batch."""
        if self.world == 1:                      # a ring of one: the message goes to this rank itself
            if send is not None and recv is not None:
                recv.copy_(send)
            return []
        ops = []
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send, self.next, self.group))
        if recv is not None:
            ops.append(dist.P2POp(dist.irecv, recv, self.prev, self.group))
        return dist.batch_isend_irecv(ops) if ops else []

    @staticmethod
    def wait(pending) -> None:
        for req in pending:
            req.wait()


class CudaBlockKernels:
    """The per-block work through the C ABI (fa_b200_fwd, fa_b200_bwd, fa_b200_combine)."""

    @staticmethod
    def forward_block(q, k, v, scale, causal):
        return _ops.launch_forward(q, k, v, scale, causal)

    @staticmethod
    def backward_block(d_o, q, k, v, o, lse, scale, causal):
        """(dq, dkv): dK and dV share one (2, B, Nk, Hkv, D) tensor, which one combine launch folds in."""
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dkv = torch.empty((2,) + tuple(k.shape), dtype=k.dtype, device=k.device)
        _ops.launch_backward(d_o, q, k, v, o, lse, scale, causal, out=(dq, dkv[0], dkv[1]))
        return dq, dkv

    combine = staticmethod(_ops.launch_combine)


def ring_forward(q, k, v, scale: float, causal: bool, ring, kernels=CudaBlockKernels, layout: str = "contiguous"):
    """(o, lse) of this rank's queries against the keys of every rank."""
    rank, world = ring.rank, ring.world
    sched = ring_schedule(rank, world, causal, layout)
    B, n, H, D = q.shape
    if causal and layout == "zigzag" and n % 2 != 0:
        raise ValueError("the zigzag layout needs an even number of positions per rank")
    whole = [t for t, (_, mode) in enumerate(sched) if mode in ("full", "causal", "lower")]
    last = max(t for t, (_, mode) in enumerate(sched) if mode != "skip")
    kv = [torch.stack((k, v)), None]                      # (2, B, n, Hkv, D): one message per hop
    kv[1] = torch.empty_like(kv[0])
    acc = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    lse = torch.empty(B, H, n, dtype=torch.float32, device=q.device)
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    written = False
    for t, (_, mode) in enumerate(sched):
        cur, nxt = kv[t % 2], kv[(t + 1) % 2]
        send, recv = kv_transfer(rank, world, causal, t, layout)
        pending = ring.exchange(cur if send else None, nxt if recv else None)
        if mode != "skip":
            rows, keys = _step_ranges(mode, n)
            o_part, lse_part = kernels.forward_block(q[:, rows], cur[0][:, keys], cur[1][:, keys], scale,
                                                     mode == "causal")
            final = t == last and t in whole              # the last partial, and it covers every row
            kernels.combine(acc[:, rows], o_part, lse[:, :, rows], lse_part, out=o if final else None,
                            first=(t == 0))
            written = written or final
        ring.wait(pending)
    if not written:
        kernels.combine(acc, None, out=o)
    return o, lse


def ring_backward(d_o, q, k, v, o, lse, scale: float, causal: bool, ring, kernels=CudaBlockKernels,
                  layout: str = "contiguous"):
    """(dq, dk, dv) of this rank's slices; o and lse are ring_forward's results."""
    rank, world = ring.rank, ring.world
    sched = ring_schedule(rank, world, causal, layout)
    n = q.shape[1]
    whole = [t for t, (_, mode) in enumerate(sched) if mode in ("full", "causal", "lower")]
    last = max(t for t, (_, mode) in enumerate(sched) if mode != "skip")
    kv = [torch.stack((k, v)), None]
    kv[1] = torch.empty_like(kv[0])
    # fp32 totals of dK and dV of the block this rank holds: they travel with the block
    dkv = [torch.empty(kv[0].shape, dtype=torch.float32, device=q.device) for _ in range(2)]
    dq_acc = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    dq = torch.empty_like(q)
    lse_upper = None                                       # the kernels want a dense log-sum-exp
    written = False
    coming = []                                            # the transfer that fills dkv[t % 2]
    for t, (_, mode) in enumerate(sched):
        cur, nxt = kv[t % 2], kv[(t + 1) % 2]
        send, recv = kv_transfer(rank, world, causal, t, layout)
        pending = ring.exchange(cur if send else None, nxt if recv else None)
        if mode != "skip":
            rows, keys = _step_ranges(mode, n)
            if mode == "upper":
                if lse_upper is None:
                    lse_upper = lse[:, :, rows].contiguous()
                lse_rows = lse_upper
            else:
                lse_rows = lse
            dq_p, dkv_p = kernels.backward_block(d_o[:, rows], q[:, rows], cur[0][:, keys], cur[1][:, keys],
                                                 o[:, rows], lse_rows, scale, mode == "causal")
            final = t == last and t in whole
            kernels.combine(dq_acc[:, rows], dq_p, out=dq if final else None, first=(t == 0))
            written = written or final
        ring.wait(coming)
        if mode != "skip":
            # dK and dV in one launch: (2, B, n, Hkv, D) seen as 2 B batch entries
            kernels.combine(dkv[t % 2].flatten(0, 1)[:, keys], dkv_p.flatten(0, 1), first=(t == 0))
        coming = ring.exchange(dkv[t % 2], dkv[(t + 1) % 2])   # after the last step: the way home
        ring.wait(pending)
    if not written:
        kernels.combine(dq_acc, None, out=dq)
    ring.wait(coming)
    home = dkv[world % 2]
    dkv_out = torch.empty(home.shape, dtype=k.dtype, device=k.device)
    kernels.combine(home.flatten(0, 1), None, out=dkv_out.flatten(0, 1))
    return dq, dkv_out[0], dkv_out[1]


class RingAttentionFunction(torch.autograd.Function):
    """autograd wrapper: apply(q, k, v, scale, causal, ring, kernels, layout) -> (o, lse)."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, ring, kernels, layout):
        o, lse = ring_forward(q, k, v, scale, causal, ring, kernels, layout)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.causal, ctx.ring, ctx.kernels, ctx.layout = scale, causal, ring, kernels, layout
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, grad_o, grad_lse=None):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ring_backward(grad_o, q, k, v, o, lse, ctx.scale, ctx.causal, ctx.ring, ctx.kernels,
                                   ctx.layout)
        return dq, dk, dv, None, None, None, None, None


def flash_attention_v100_sequence_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                           causal: bool = False, scale: Optional[float] = None,
                                           group=None, return_softmax_lse: bool = False,
                                           layout: str = "contiguous", ring=None, kernels=None):
    """Attention over a sequence that is split across the ranks of `group`.

    q, k, v are this rank's slices, (B, n, H, D) / (B, n, Hkv, D), the same n on every rank.
    layout="contiguous": rank r holds positions [r n, (r + 1) n).  layout="zigzag": rank r holds chunks
    r and 2 G - 1 - r of 2 G equal chunks (zigzag_split), which balances the work under a causal mask.
    Returns this rank's slice of the output (and of the log-sum-exp, (B, H, n) fp32, with
    return_softmax_lse).  Differentiable: the backward is a second trip around the ring.  Every rank of
    the group must make the call.  Dropout and bias are not offered on this path."""
    if q.dim() != 4 or k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3]:
        raise ValueError("expected q (B, n, H, D) and k, v (B, n, Hkv, D)")
    if q.shape[1] != k.shape[1]:
        raise ValueError("sequence-parallel attention splits one sequence: q and k must have the same length")
    if layout not in LAYOUTS:
        raise ValueError(f"layout must be one of {LAYOUTS}")
    if ring is None:
        ring = DistributedRing(group)
    if kernels is None:
        if not q.is_cuda:
            raise RuntimeError("flash_attention_v100 has no CPU path: q, k and v must be CUDA tensors")
        kernels = CudaBlockKernels
    scale = float(q.shape[3] ** -0.5 if scale is None else scale)
    o, lse = RingAttentionFunction.apply(q, k.contiguous(), v.contiguous(), scale, bool(causal), ring, kernels,
                                         layout)
    return (o, lse) if return_softmax_lse else o


__all__ = ["ring_schedule", "kv_transfer", "zigzag_split", "zigzag_merge", "LAYOUTS", "DistributedRing", "CudaBlockKernels", "ring_forward", "ring_backward",
           "RingAttentionFunction", "flash_attention_v100_sequence_parallel"]
