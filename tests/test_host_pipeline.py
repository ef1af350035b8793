"""Host-operand step: chunk planning on the CPU, results against single calls on the GPU."""
import pytest
import torch

import flash_attention_v100 as fa
from flash_attention_v100.ops import host_pipeline as hp
from flash_attention_v100.ops import attention as ops
from flash_attention_v100.testing import dq_is_bit_reproducible, assert_same_dq


def test_chunk_bounds_cover_the_batch():
    for batch in (0, 1, 3, 4, 7, 32):
        for chunks in (1, 2, 4, 5, 64):
            b = hp.chunk_bounds(batch, chunks)
            assert b[0][0] == 0 and b[-1][1] == batch
            assert all(x[1] == y[0] for x, y in zip(b, b[1:]))
            sizes = [e - s for s, e in b]
            assert max(sizes) - min(sizes) <= 1
            assert len(b) == max(1, min(chunks, batch))
    with pytest.raises(ValueError):
        hp.chunk_bounds(4, 0)


def test_plan_chunks_cover_the_grid_once():
    for batch, heads, hkv in ((4, 32, 32), (1, 32, 8), (3, 4, 2), (32, 16, 16), (2, 6, 3), (1, 1, 1)):
        group = heads // hkv
        for chunks in (None, 1, 2, 3, 8, 16, 64):
            plan = hp.plan_chunks(batch, heads, hkv, chunks)
            seen = set()
            for b0, b1, h0, h1 in plan:
                assert 0 <= b0 < b1 <= batch and 0 <= h0 < h1 <= heads
                assert h0 % group == 0 and h1 % group == 0          # a chunk owns whole K/V heads
                cols = {(b, h) for b in range(b0, b1) for h in range(h0, h1)}
                assert not (cols & seen)
                seen |= cols
            assert len(seen) == batch * heads
            if chunks is not None and chunks <= batch:
                assert len(plan) == chunks
    # a batch of one is cut along heads, so its copies can overlap its kernels
    assert len(hp.plan_chunks(1, 32, 32)) > 1
    # the default keeps at least 8 columns per chunk
    assert all((b1 - b0) * (h1 - h0) >= 8 for b0, b1, h0, h1 in hp.plan_chunks(4, 32, 32))
    assert len(hp.plan_chunks(4, 32, 32)) == 16 and len(hp.plan_chunks(1, 32, 32)) == 4


def test_needs_cuda():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        fa.HostAttentionStep((2, 128, 2, 64), (2, 128, 2, 64), torch.float16, "cuda:0")


def _pinned(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * 0.5).to(dtype).pin_memory()


@pytest.mark.gpu
@pytest.mark.parametrize("chunks", [None, 2, 1, 6])
@pytest.mark.parametrize("dropout_p", [0.0, 0.25])
def test_host_step_matches_one_call_over_the_whole_problem(chunks, dropout_p):
    """However the step is chunked (whole batch entries, or head groups of a batch entry), its results
    equal one forward and one backward call over the whole problem, dropout mask included."""
    dev = torch.device("cuda", 0)
    B, N, H, Hkv, D, dt = 3, 320, 4, 2, 128, torch.bfloat16
    host = {"q": _pinned((B, N, H, D), dt, 1), "k": _pinned((B, N, Hkv, D), dt, 2),
            "v": _pinned((B, N, Hkv, D), dt, 3), "d_o": _pinned((B, N, H, D), dt, 4)}
    out = {n: torch.empty(host["k" if n in ("dk", "dv") else "q"].shape, dtype=dt).pin_memory()
           for n in ("o", "dq", "dk", "dv")}
    step = fa.HostAttentionStep(host["q"].shape, host["k"].shape, dt, dev, causal=True, dropout_p=dropout_p,
                                chunks=chunks)
    if chunks == 6:
        assert len(step.chunks) == 6 and step.chunks[0] == (0, 1, 0, 2)
    seed, offset = (0x5EED, 3) if dropout_p > 0 else (0, 0)
    d = {n: t.to(dev) for n, t in host.items()}
    res = torch.empty_like(d["q"])            # bf16: the step keeps the output residual for its backward
    o, lse = ops.launch_forward(d["q"], d["k"], d["v"], step.scale, True, dropout_p, seed, offset, o_residual=res)
    dq, dk, dv = ops.launch_backward(d["d_o"], d["q"], d["k"], d["v"], o, lse, step.scale, True, dropout_p,
                                     seed, offset, o_residual=res)
    for rep in range(2):                       # the second call reuses buffers while the first drains
        for t in out.values():
            t.fill_(float("nan"))
        step(host, out, seed, offset)
        step.synchronize()
        for name, ref in (("o", o), ("dk", dk), ("dv", dv)):
            assert torch.equal(out[name], ref.cpu()), (name, rep)
        assert_same_dq(out["dq"], dq.cpu(), dq_is_bit_reproducible("auto", dt, D, dropout_p))


@pytest.mark.gpu
def test_host_step_rejects_pageable_and_wrong_shapes():
    dev = torch.device("cuda", 0)
    shape, dt = (2, 128, 2, 64), torch.float16
    step = fa.HostAttentionStep(shape, shape, dt, dev)
    good = {n: torch.zeros(shape, dtype=dt).pin_memory() for n in ("q", "k", "v", "d_o")}
    out = {n: torch.zeros(shape, dtype=dt).pin_memory() for n in ("o", "dq", "dk", "dv")}
    with pytest.raises(ValueError, match="pinned"):
        step({**good, "q": torch.zeros(shape, dtype=dt)}, out)
    with pytest.raises(ValueError, match="expected"):
        step({**good, "k": torch.zeros((2, 64, 2, 64), dtype=dt).pin_memory()}, out)
