"""Shard planning and the scatter/gather plumbing of the one-process-per-GPU
mode, exercised with gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attention_v100.interface import FlashAttentionV100Manager, plan_shards, _slice, _kv_shard


def _covers(shards, B, H):
    seen = torch.zeros(B, H, dtype=torch.int32)
    for b0, b1, h0, h1 in shards:
        seen[b0:b1, h0:h1] += 1
    return bool((seen == 1).all())


@pytest.mark.parametrize("B,H,G", [(4, 32, 8), (4, 32, 2), (32, 16, 8), (1, 32, 8), (3, 5, 4), (8, 3, 8),
                                   (2, 2, 8), (1, 1, 4), (5, 7, 3)])
def test_plan_covers_grid_exactly_once(B, H, G):
    kind, shards = plan_shards(B, H, G)
    assert len(shards) == G and kind in ("head_parallel", "batch_parallel")
    assert _covers(shards, B, H)


def test_plan_prefers_heads_then_batch():
    assert plan_shards(4, 32, 8)[0] == "head_parallel"          # cfg3: 4 heads per GPU
    assert plan_shards(4, 32, 8)[1][1] == (0, 4, 4, 8)
    assert plan_shards(32, 12, 8)[0] == "batch_parallel"        # heads do not divide, batch does
    kind, shards = plan_shards(2, 8, 4, num_heads_kv=2)         # GQA: split only at kv-head boundaries
    assert all(h0 % 4 == 0 and h1 % 4 == 0 for _, _, h0, h1 in shards)
    assert _covers(shards, 2, 8)
    assert _kv_shard((0, 2, 4, 8), 4) == (0, 2, 1, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fail_rank, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=__import__("datetime").timedelta(seconds=20))
    try:
        B, N, H, D = 3, 16, 5, 8
        _, shards = plan_shards(B, H, world)
        g = torch.Generator().manual_seed(0)
        full = torch.randn(B, N, H, D, generator=g)
        lse_full = torch.randn(B, H, N, generator=g)
        like = torch.empty(B, N, H, D)
        local = FlashAttentionV100Manager.scatter_shards(full if rank == 0 else None, shards, like, src=0)
        assert torch.equal(local, _slice(full, shards[rank]))
        lse_local = FlashAttentionV100Manager.scatter_shards(lse_full if rank == 0 else None, shards,
                                                             torch.empty(B, H, N), src=0, lse=True)
        if fail_rank == rank:
            raise RuntimeError("injected failure on rank %d" % rank)
        # per-rank "compute": something rank-local and shard-shaped
        out = FlashAttentionV100Manager.gather_shards(local * 2, shards, full.shape, dst=0)
        lse_out = FlashAttentionV100Manager.gather_shards(lse_local + 1, shards, lse_full.shape, dst=0, lse=True)
        if rank == 0:
            assert torch.equal(out, full * 2)
            assert torch.equal(lse_out, lse_full + 1)
        ret[rank] = "ok"
    except Exception as e:   # noqa: BLE001
        ret[rank] = "error: %s" % e
    finally:
        try:
            dist.destroy_process_group()
        except Exception:   # noqa: BLE001
            pass


def _run(world, fail_rank=None):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive()
    return dict(ret)


def test_scatter_gather_world2_gloo():
    assert _run(2) == {0: "ok", 1: "ok"}


def test_scatter_gather_uneven_world3_gloo():
    assert _run(3) == {0: "ok", 1: "ok", 2: "ok"}


def test_rank_that_raises_is_reported_not_hung():
    res = _run(2, fail_rank=1)
    assert res[1].startswith("error: injected failure")
    assert res[0] != "ok"      # rank 0 sees the missing peer as an error, within the group timeout
