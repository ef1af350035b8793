"""Multi-GPU paths on real devices (skipped with fewer than two GPUs).

Per-(batch, head) work is identical whichever GPU runs it, so a sharded run must
equal the single-GPU run bit for bit."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import flash_attention_v100 as fa
from flash_attention_v100.interface import FlashAttentionV100Manager, plan_shards, _slice
from flash_attention_v100.ops import sequence_parallel
from flash_attention_v100.testing import dq_is_bit_reproducible, assert_same_dq, rel_l2

pytestmark = pytest.mark.gpu


def _need_gpus(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _inputs(B, N, H, D, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, N, H, D, generator=g).to(dtype) for _ in range(4)]


@pytest.mark.parametrize("dropout_p", [0.0, 0.2], ids=["nodrop", "dropout"])
@pytest.mark.parametrize("B,H", [(2, 8), (4, 3)], ids=["heads", "batch"])
def test_single_process_sharding_equals_single_gpu(B, H, dropout_p):
    """Also under dropout: every shard indexes the stream by its columns' place in the whole problem."""
    _need_gpus(2)
    dev = torch.device("cuda:0")
    qc, kc, vc, gc = _inputs(B, 384, H, 128, torch.bfloat16)
    q1, k1, v1 = (t.to(dev).requires_grad_(True) for t in (qc, kc, vc))
    fa.set_dropout_seed(0xABCD, 5)
    o1, lse1 = fa.flash_attention_v100(q1, k1, v1, causal=True, return_softmax_lse=True, enable_multi_gpu=False,
                                       dropout_p=dropout_p)
    o1.backward(gc.to(dev))
    with FlashAttentionV100Manager(enable_multi_gpu=True) as mgr:
        assert len(mgr.devices) >= 2
        q2, k2, v2 = (t.to(dev).requires_grad_(True) for t in (qc, kc, vc))
        fa.set_dropout_seed(0xABCD, 5)
        o2, lse2 = fa.flash_attention_v100(q2, k2, v2, causal=True, return_softmax_lse=True, enable_multi_gpu=True,
                                           dropout_p=dropout_p)
        o2.backward(gc.to(dev))
    torch.cuda.synchronize()
    assert o2.device == dev and torch.equal(o1, o2) and torch.equal(lse1, lse2)
    assert torch.equal(k1.grad, k2.grad) and torch.equal(v1.grad, v2.grad)
    assert_same_dq(q1.grad, q2.grad, dq_is_bit_reproducible("auto", torch.bfloat16, 128))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


# A rank that is alone in a collective gives up after this long instead of waiting for ever.
_GROUP_TIMEOUT = datetime.timedelta(seconds=60)


def _run_ranks(target, world, *args):
    """Run `target(rank, world, port, *args, ret)` in `world` child processes and return what they
    reported.  The children are daemons and any that is still alive after the join (a rank whose peer
    raised stays blocked in its collective) is terminated, then killed, before the test asserts: no
    child, and no kernel of a child, outlives the test."""
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port) + args + (ret,), daemon=True) for r in range(world)]
    stuck = []
    try:
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
    finally:
        for r, p in enumerate(procs):
            if p.is_alive():
                stuck.append(r)
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(10)
    assert not stuck, f"ranks {stuck} did not finish (reports: {dict(ret)})"
    return dict(ret)


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=_GROUP_TIMEOUT)
    try:
        B, N, H, D = 2, 512, 8, 64
        qc, kc, vc, gc = _inputs(B, N, H, D, torch.float16, seed=3)
        _, shards = plan_shards(B, H, world)
        like = torch.empty(B, N, H, D, dtype=torch.float16, device=dev)
        full = [t.to(dev) if rank == 0 else None for t in (qc, kc, vc, gc)]
        ql, kl, vl, gl = (FlashAttentionV100Manager.scatter_shards(t, shards, like) for t in full)
        ql, kl, vl = (t.requires_grad_(True) for t in (ql, kl, vl))
        # the shard's origin in the whole problem and the whole call's stream: the mask of the whole call
        sh = shards[rank]
        o = fa.flash_attention_v100(ql, kl, vl, causal=True, enable_multi_gpu=False, dropout_p=0.2,
                                    dropout_origin=(sh[0], sh[2], H), dropout_stream=(0x77, 1))
        o.backward(gl)
        outs = [FlashAttentionV100Manager.gather_shards(t, shards, (B, N, H, D)) for t in
                (o.detach(), ql.grad, kl.grad, vl.grad)]
        if rank == 0:
            q1, k1, v1 = (t.to(dev).requires_grad_(True) for t in (qc, kc, vc))
            o1 = fa.flash_attention_v100(q1, k1, v1, causal=True, enable_multi_gpu=False, dropout_p=0.2,
                                         dropout_stream=(0x77, 1))
            o1.backward(gc.to(dev))
            same = all(torch.equal(outs[i], x) for i, x in ((0, o1.detach()), (2, k1.grad), (3, v1.grad)))
            same = same and rel_l2(outs[1], q1.grad) <= 1e-3     # dQ: unordered fp32 sums, then rounding
            ret[0] = "ok" if same else "mismatch"
        torch.cuda.synchronize()
    except Exception as e:   # noqa: BLE001
        ret[rank] = f"error: {e}"
    finally:
        dist.destroy_process_group()


def test_nccl_scatter_compute_gather_equals_single_gpu():
    _need_gpus(2)
    ret = _run_ranks(_rank_main, 2)
    assert ret.get(0) == "ok", ret


def _ring_rank_main(rank, world, port, layout, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=_GROUP_TIMEOUT)
    try:
        B, n, H, D = 2, 384, 4, 128
        qc, kc, vc, gc = _inputs(B, n * world, H, D, torch.bfloat16, seed=5)
        if layout == "zigzag":
            cut = lambda t, dim=1: sequence_parallel.zigzag_split(t, world, rank, dim)
        else:
            cut = lambda t, dim=1: t.chunk(world, dim=dim)[rank]
        ql, kl, vl = (cut(t).to(dev).requires_grad_(True) for t in (qc, kc, vc))
        o, lse = fa.flash_attention_v100_sequence_parallel(ql, kl, vl, causal=True, return_softmax_lse=True,
                                                           layout=layout)
        o.backward(cut(gc).to(dev))
        # one call over the whole sequence on this rank's own GPU, sliced, is the reference
        q1, k1, v1 = (t.to(dev).requires_grad_(True) for t in (qc, kc, vc))
        o1, lse1 = fa.flash_attention_v100(q1, k1, v1, causal=True, return_softmax_lse=True, enable_multi_gpu=False)
        o1.backward(gc.to(dev))
        torch.cuda.synchronize()
        errs = {"o": rel_l2(o.detach(), cut(o1.detach())), "lse": rel_l2(lse, cut(lse1, 2)),
                "dq": rel_l2(ql.grad, cut(q1.grad)), "dk": rel_l2(kl.grad, cut(k1.grad)),
                "dv": rel_l2(vl.grad, cut(v1.grad))}
        bad = {k: v for k, v in errs.items() if not v < (1e-5 if k == "lse" else 4e-3)}
        ret[rank] = "ok" if not bad else f"mismatch: {bad}"
    except Exception as e:   # noqa: BLE001
        ret[rank] = f"error: {e}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_nccl_ring_attention_equals_whole_sequence(layout):
    _need_gpus(2)
    ret = _run_ranks(_ring_rank_main, 2, layout)
    assert ret == {0: "ok", 1: "ok"}, ret
