"""Test doubles for sequence-parallel attention.

ThreadRing runs the ranks of a ring as threads of one process (messages are
copies handed over through queues), so the ring logic can be exercised without
process groups, on CPU tensors or on one GPU.  OracleBlockKernels does the
per-block work with the CPU oracle instead of the CUDA library; it exists only
so that the ring's scheduling and merging arithmetic can be tested where there
is no GPU.
"""
import queue
import threading

import torch

from oracle import attention_oracle as orc


class ThreadRing:
    def __init__(self, rank, world, boxes):
        self.rank, self.world, self._boxes = rank, world, boxes

    def exchange(self, send, recv):
        if send is not None:
            self._boxes[(self.rank + 1) % self.world].put(send.clone())
        return [recv] if recv is not None else []

    def wait(self, pending):
        for recv in pending:
            recv.copy_(self._boxes[self.rank].get(timeout=30))


def run_ring(world, fn):
    """fn(ring) on `world` threads; returns the results in rank order, re-raises the first failure."""
    boxes = [queue.Queue() for _ in range(world)]
    out, err = [None] * world, []

    def body(r):
        try:
            out[r] = fn(ThreadRing(r, world, boxes))
        except BaseException as e:      # noqa: BLE001 - reported to the caller below
            err.append(e)

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    if err:
        raise err[0]
    assert all(not t.is_alive() for t in threads), "a ring thread did not finish"
    return out


class OracleBlockKernels:
    """forward_block / backward_block / combine with the semantics of the CUDA library's entry points."""

    @staticmethod
    def forward_block(q, k, v, scale, causal):
        o, lse = orc.attention_forward(q, k, v, causal=causal, scale=scale)
        return o.to(q.dtype), lse.float()

    @staticmethod
    def backward_block(d_o, q, k, v, o, lse, scale, causal):
        dq, dk, dv = orc.attention_backward_closed_form(q, k, v, o, lse, d_o, causal=causal, scale=scale)
        return dq.to(q.dtype), torch.stack((dk.to(k.dtype), dv.to(v.dtype)))

    @staticmethod
    def combine(acc, part=None, lse_acc=None, lse_part=None, out=None, first=False):
        if part is not None:
            p = part.float()
            if lse_acc is not None:
                la = torch.full_like(lse_part, float("-inf")) if first else lse_acc.clone()
                ln = torch.logaddexp(la, lse_part)
                seen = ln > float("-inf")
                wa = torch.where(seen, torch.exp(la - ln), torch.zeros_like(ln)).transpose(1, 2).unsqueeze(-1)
                wp = torch.where(seen, torch.exp(lse_part - ln), torch.zeros_like(ln)).transpose(1, 2).unsqueeze(-1)
                acc.copy_(p * wp if first else acc * wa + p * wp)
                lse_acc.copy_(ln)
            else:
                acc.copy_(p if first else acc + p)
        if out is not None:
            out.copy_(acc.to(out.dtype))
