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


def test_chunk_dropout_offsets_are_distinct_streams():
    offs = {hp.chunk_dropout_offset(7, c) for c in range(16)}
    assert len(offs) == 16
    assert hp.chunk_dropout_offset(7, 0) == 7
    assert all((o >> 32) != 0 for o in offs if o != 7)      # the chunk index lands in the key word


def test_needs_cuda():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        fa.HostAttentionStep((2, 128, 2, 64), (2, 128, 2, 64), torch.float16, "cuda:0")


def _pinned(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * 0.5).to(dtype).pin_memory()


@pytest.mark.gpu
@pytest.mark.parametrize("chunks", [None, 2, 1])
@pytest.mark.parametrize("dropout_p", [0.0, 0.25])
def test_host_step_matches_single_calls(chunks, dropout_p):
    dev = torch.device("cuda", 0)
    B, N, H, Hkv, D, dt = 3, 320, 4, 2, 128, torch.bfloat16
    host = {"q": _pinned((B, N, H, D), dt, 1), "k": _pinned((B, N, Hkv, D), dt, 2),
            "v": _pinned((B, N, Hkv, D), dt, 3), "d_o": _pinned((B, N, H, D), dt, 4)}
    out = {n: torch.empty(host["k" if n in ("dk", "dv") else "q"].shape, dtype=dt).pin_memory()
           for n in ("o", "dq", "dk", "dv")}
    step = fa.HostAttentionStep(host["q"].shape, host["k"].shape, dt, dev, causal=True, dropout_p=dropout_p,
                                chunks=chunks)
    seed, offset = 0x5EED, 3
    for rep in range(2):                       # the second call reuses buffers while the first drains
        for t in out.values():
            t.fill_(float("nan"))
        step(host, out, seed, offset)
        step.synchronize()
        for c, (b, e) in enumerate(step.bounds):
            d = {n: t[b:e].to(dev) for n, t in host.items()}
            off = hp.chunk_dropout_offset(offset, c) if dropout_p > 0 else 0
            sd = seed if dropout_p > 0 else 0
            o, lse = ops.launch_forward(d["q"], d["k"], d["v"], step.scale, True, dropout_p, sd, off)
            dq, dk, dv = ops.launch_backward(d["d_o"], d["q"], d["k"], d["v"], o, lse, step.scale, True,
                                             dropout_p, sd, off)
            for name, ref in (("o", o), ("dk", dk), ("dv", dv)):
                assert torch.equal(out[name][b:e], ref.cpu()), (name, c, rep)
            assert_same_dq(out["dq"][b:e], dq.cpu(), dq_is_bit_reproducible("auto", dt, D, dropout_p))


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
