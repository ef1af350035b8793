"""Benchmark workloads at reduced batch/heads against the oracle, and at full
size through size-independent properties (shards == whole, determinism,
oracle on a sampled subset of heads)."""
import os

import numpy as np
import pytest
import torch

import flash_attention_v100 as fa
from flash_attention_v100.kernels import _cabi
from flash_attention_v100.ops.attention import launch_forward, launch_backward, saves_output_residual
from flash_attention_v100.testing import (WORKLOADS, tolerance, DROPOUT_SEED, DROPOUT_OFFSET, make_inputs, rel_l2,
                                          dq_is_bit_reproducible, assert_same_dq)
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu


def _oracle_subset(w, t, b, heads, keep=None, p_eff=0.0):
    sl = (slice(b, b + 1), slice(None), heads)
    return ao.attention_forward_backward(*(t[n][sl].float() for n in ("q", "k", "v", "d_o")),
                                         causal=w.causal, scale=w.scale, dropout_p=p_eff, keep_mask=keep)


@pytest.mark.parametrize("name,shrink", [
    ("cfg2", dict(B=1, H=2)), ("cfg3", dict(B=1, H=2)), ("cfg4", dict(N=8192, H=1)), ("cfg5", dict(B=1, H=2)),
])
def test_workload_shapes_reduced_vs_oracle(device, name, shrink):
    w = WORKLOADS[name].shrink(**shrink)
    t = make_inputs(w)
    keep, p_eff, stream = None, 0.0, (0, 0)
    if w.dropout_p > 0:
        stream = (DROPOUT_SEED, DROPOUT_OFFSET)
        lib = _cabi.load()
        keep_np = np.empty((w.B, w.H, w.N, w.N), np.uint8)
        assert lib.fa_b200_dropout_mask_host(*stream, w.dropout_p, w.B, w.H, w.N, w.N, keep_np.ctypes.data) == 0
        keep, p_eff = torch.from_numpy(keep_np), float(lib.fa_b200_dropout_effective_p(w.dropout_p))
    ref = ao.attention_forward_backward(*(t[n].float() for n in ("q", "k", "v", "d_o")), causal=w.causal,
                                        scale=w.scale, dropout_p=p_eff, keep_mask=keep)
    d = {n: x.to(device) for n, x in t.items()}
    # bf16: with the output residual, as the autograd op runs it (peaked rows, cfg4's outliers, amplify
    # the rounding of a bf16 O in dQ/dK otherwise: test_softmax_range_stress_rows)
    res = torch.empty_like(d["q"]) if saves_output_residual(w.dtype) else None
    o, lse = launch_forward(d["q"], d["k"], d["v"], w.scale, w.causal, w.dropout_p, *stream, o_residual=res)
    dq, dk, dv = launch_backward(d["d_o"], d["q"], d["k"], d["v"], o, lse, w.scale, w.causal, w.dropout_p, *stream,
                                 o_residual=res)
    tol = tolerance(w.dtype, "auto", w.D)
    for nm, got, r in zip(("o", "lse", "dq", "dk", "dv"), (o, lse, dq, dk, dv), ref):
        err = rel_l2(got, r)
        assert err <= tol, f"{name}:{nm} rel-L2 {err:.3e}"


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg4", "cfg5"])
def test_full_size_properties(device, name):
    """Full benchmark size: (1) two runs agree bit for bit, (2) a head shard and a batch shard equal
    the whole, dropout mask included, (3) two sampled (b, h) columns match the oracle."""
    w = WORKLOADS[name]
    if "tcgen05" not in os.environ.get("FA_B200_TEST_VARIANTS", "simt,tcgen05").split(","):
        pytest.skip("full-size runs are only practical on the tensor-core kernels")
    t = make_inputs(w)
    stream = (DROPOUT_SEED, DROPOUT_OFFSET) if w.dropout_p > 0 else (0, 0)
    d = {n: x.to(device) for n, x in t.items()}

    def run(q, k, v, g, origin=None):
        res = torch.empty_like(q) if saves_output_residual(w.dtype) else None
        o, lse = launch_forward(q, k, v, w.scale, w.causal, w.dropout_p, *stream, dropout_origin=origin,
                                o_residual=res)
        return (o, lse) + launch_backward(g, q, k, v, o, lse, w.scale, w.causal, w.dropout_p, *stream,
                                          dropout_origin=origin, o_residual=res)

    a = run(d["q"], d["k"], d["v"], d["d_o"])
    b = run(d["q"], d["k"], d["v"], d["d_o"])
    exact_dq = dq_is_bit_reproducible("auto", w.dtype, w.D, w.dropout_p)
    assert all(torch.equal(a[i], b[i]) for i in (0, 1, 3, 4))
    assert_same_dq(a[2], b[2], exact_dq)
    del b
    # a shard passes its origin in the whole problem, so it draws the whole call's dropout mask
    h0, h1 = w.H // 2, w.H // 2 + 2
    b0, b1 = (w.B // 2, w.B // 2 + 1) if w.B > 1 else (0, 1)
    for (bs, hs, origin) in ((slice(None), slice(h0, h1), (0, h0, w.H)), (slice(b0, b1), slice(None), (b0, 0, w.H))):
        s = run(*(d[n][bs, :, hs] for n in ("q", "k", "v", "d_o")), origin=origin)
        assert torch.equal(s[0], a[0][bs, :, hs]) and torch.equal(s[1], a[1][bs, hs])
        assert all(torch.equal(s[i], a[i][bs, :, hs]) for i in (3, 4))
        assert_same_dq(s[2], a[2][bs, :, hs], exact_dq)
        del s
    tol = tolerance(w.dtype, "auto", w.D)
    # dropout: the stream is indexed by b*H + h, so sample low (b, h) columns whose
    # host mask is cheap to generate; otherwise sample the first and the last column
    samples = ((0, 0), (0, 1)) if w.dropout_p > 0 else ((0, 0), (w.B - 1, w.H - 1))
    for bb, hh in samples:
        keep, p_eff = None, 0.0
        if w.dropout_p > 0:
            lib = _cabi.load()
            bh = bb * w.H + hh
            tmp = np.empty((1, bh + 1, w.N, w.N), np.uint8)
            assert lib.fa_b200_dropout_mask_host(*stream, w.dropout_p, 1, bh + 1, w.N, w.N, tmp.ctypes.data) == 0
            keep = torch.from_numpy(tmp[:, bh:bh + 1])
            p_eff = float(lib.fa_b200_dropout_effective_p(w.dropout_p))
        ref = _oracle_subset(w, t, bb, slice(hh, hh + 1), keep, p_eff)
        got = (a[0][bb:bb + 1, :, hh:hh + 1], a[1][bb:bb + 1, hh:hh + 1], a[2][bb:bb + 1, :, hh:hh + 1],
               a[3][bb:bb + 1, :, hh:hh + 1], a[4][bb:bb + 1, :, hh:hh + 1])
        for nm, g_, r in zip(("o", "lse", "dq", "dk", "dv"), got, ref):
            err = rel_l2(g_, r)
            assert err <= tol, f"{name}[b{bb},h{hh}]:{nm} rel-L2 {err:.3e}"
