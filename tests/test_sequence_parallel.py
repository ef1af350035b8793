"""Sequence-parallel (ring) attention: schedule, merging arithmetic and the exchange pattern on CPU.

The per-block kernels are replaced by the oracle here (tests only); the GPU
tests run the same ring code over the CUDA library."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attention_v100.ops import sequence_parallel as sp
from oracle import attention_oracle as orc
from ring_helpers import OracleBlockKernels, run_ring


@pytest.mark.parametrize("world", [1, 2, 3, 5])
@pytest.mark.parametrize("causal", [False, True])
def test_schedule_delivers_every_visible_block(world, causal):
    held = list(range(world))                      # block each rank holds at step 0: its own
    for t in range(world):
        for r in range(world):
            block, mode = sp.ring_schedule(r, world, causal)[t]
            assert block == (r - t) % world
            visible = (not causal) or block <= r
            assert (mode != "skip") == visible
            assert mode == ("causal" if causal and block == r else "full" if visible else "skip")
            if visible:
                assert held[r] == block, "a block that is needed was not delivered"
        nxt = list(held)
        for r in range(world):
            send, _ = sp.kv_transfer(r, world, causal, t)
            _, recv = sp.kv_transfer((r + 1) % world, world, causal, t)
            assert send == recv, "a send without its receive would hang the ring"
            nxt[(r + 1) % world] = held[r] if send else None
        held = nxt


def test_schedule_rejects_bad_rank():
    with pytest.raises(ValueError):
        sp.ring_schedule(2, 2, False)


def _whole(B, N, H, Hkv, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, N, H, D, generator=g)
    k = torch.randn(B, N, Hkv, D, generator=g)
    v = torch.randn(B, N, Hkv, D, generator=g)
    d_o = torch.randn(B, N, H, D, generator=g)
    return q, k, v, d_o


def _shard(t, ring, layout, dim=1):
    if layout == "zigzag":
        return sp.zigzag_split(t, ring.world, ring.rank, dim)
    return t.chunk(ring.world, dim=dim)[ring.rank]


def _unshard(parts, layout, dim=1):
    return sp.zigzag_merge(parts, dim) if layout == "zigzag" else torch.cat(parts, dim=dim)


def _rank_call(ring, q, k, v, d_o, causal, kernels, layout="contiguous"):
    ql, kl, vl = (_shard(t, ring, layout).clone().requires_grad_(True) for t in (q, k, v))
    o, lse = sp.flash_attention_v100_sequence_parallel(ql, kl, vl, causal=causal, return_softmax_lse=True,
                                                       layout=layout, ring=ring, kernels=kernels)
    o.backward(_shard(d_o, ring, layout))
    return o.detach(), lse, ql.grad, kl.grad, vl.grad


def _gathered(res, layout):
    o, dq, dk, dv = (_unshard([r[i] for r in res], layout) for i in (0, 2, 3, 4))
    return o, _unshard([r[1] for r in res], layout, dim=2), dq, dk, dv


@pytest.mark.parametrize("world,causal,Hkv,layout", [
    (2, True, 4, "contiguous"), (3, False, 4, "contiguous"), (4, True, 2, "contiguous"), (1, True, 4, "contiguous"),
    (2, True, 4, "zigzag"), (3, True, 2, "zigzag"), (4, True, 4, "zigzag"), (2, False, 4, "zigzag"),
    (1, True, 4, "zigzag")])
def test_thread_ring_with_oracle_blocks_equals_whole_sequence(world, causal, Hkv, layout):
    q, k, v, d_o = _whole(2, 24 * world, 4, Hkv, 16)
    ref = orc.attention_forward_backward(q, k, v, d_o, causal=causal)
    res = run_ring(world, lambda ring: _rank_call(ring, q, k, v, d_o, causal, OracleBlockKernels, layout))
    for got, want in zip(_gathered(res, layout), ref):
        assert orc.rel_l2(got, want) < 2e-6


def test_zigzag_split_and_merge_are_inverse():
    x = torch.arange(24).reshape(1, 24, 1).repeat(2, 1, 3)
    parts = [sp.zigzag_split(x, 4, r) for r in range(4)]
    assert parts[1][0, :, 0].tolist() == [3, 4, 5, 18, 19, 20]            # chunks 1 and 6 of 8
    assert torch.equal(sp.zigzag_merge(parts), x)
    with pytest.raises(ValueError):
        sp.zigzag_split(x, 5, 0)


@pytest.mark.parametrize("world", [1, 2, 3, 5])
def test_zigzag_schedule_is_balanced(world):
    # visible (query chunk, key chunk) pairs per step, in units of half a chunk pair: the same for every rank
    for r in range(world):
        sched = sp.ring_schedule(r, world, True, "zigzag")
        assert [m for _, m in sched][0] == "causal"
        for t, (block, mode) in enumerate(sched):
            assert mode == ("causal" if block == r else "lower" if block < r else "upper")
            assert sp.kv_transfer(r, world, True, t, "zigzag") == ((True, True) if t < world - 1 else (False, False))
            # check the visible area against the definition: chunk ids of the rows and keys
            qc, kc = (r, 2 * world - 1 - r), (block, 2 * world - 1 - block)
            rows, keys = sp._step_ranges(mode, 2)
            seen = {(a, b) for a in qc[rows] for b in kc[keys]}
            want = {(a, b) for a in qc for b in kc if b <= a}
            if mode == "causal":                   # the call covers all four pairs; its mask hides (r, 2G-1-r)
                assert len(seen) == 4 and len(want) == 3
            else:                                  # two whole chunk pairs, none on the diagonal
                assert seen == want and len(seen) == 2
    with pytest.raises(ValueError):
        sp.ring_schedule(0, 2, True, "striped")


def test_needs_distributed_or_a_ring():
    q = torch.zeros(1, 8, 1, 16)
    with pytest.raises(RuntimeError, match="initialised torch.distributed"):
        sp.flash_attention_v100_sequence_parallel(q, q, q)
    with pytest.raises(ValueError, match="same length"):
        sp.flash_attention_v100_sequence_parallel(q, q[:, :4], q[:, :4], ring=object(), kernels=OracleBlockKernels)


def test_no_cpu_path_for_the_blocks():
    class OneRank:
        rank, world = 0, 1
    q = torch.zeros(1, 8, 1, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        sp.flash_attention_v100_sequence_parallel(q, q, q, ring=OneRank())


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_rank(rank, world, port, causal, layout, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, d_o = _whole(1, 16 * world, 2, 2, 16)
        ring = sp.DistributedRing()
        assert (ring.rank, ring.world) == (rank, world)
        out = _rank_call(ring, q, k, v, d_o, causal, OracleBlockKernels, layout)
        ret[rank] = [t.clone() for t in out]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,causal,layout", [(2, False, "contiguous"), (2, True, "contiguous"),
                                                 (2, True, "zigzag"), (3, True, "zigzag")])
def test_distributed_ring_gloo(world, causal, layout):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_gloo_rank, args=(r, world, port, causal, layout, ret))
                 for port in [_free_port()] for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        res = [ret[r] for r in range(world)]
    q, k, v, d_o = _whole(1, 16 * world, 2, 2, 16)
    ref = orc.attention_forward_backward(q, k, v, d_o, causal=causal)
    for got, want in zip(_gathered(res, layout), ref):
        assert orc.rel_l2(got, want) < 2e-6


def test_distributed_ring_of_one_delivers_to_itself():
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        q, k, v, d_o = _whole(1, 16, 2, 1, 16)
        out = _rank_call(sp.DistributedRing(), q, k, v, d_o, True, OracleBlockKernels)
    finally:
        dist.destroy_process_group()
    ref = orc.attention_forward_backward(q, k, v, d_o, causal=True)
    for got, want in zip(out, ref):
        assert orc.rel_l2(got, want) < 2e-6
