"""The oracle itself: pinned against the reference's golden vectors, its two
restatements against each other, and the dropout stream against the published
Philox known answers.  CPU only."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from oracle import c_oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = sorted(p for p in glob.glob(os.path.join(GOLDEN, "math_path_*.npz")) if "cfg1" not in p)


def _load(path):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in ("q", "k", "v", "d_o", "o", "dq", "dk", "dv")}
    return t, bool(z["causal"]), float(z["scale"])


def test_golden_fixtures_present():
    assert len(CASES) >= 5


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[10:-4] for p in CASES])
def test_python_oracle_matches_reference_math_path(path):
    t, causal, scale = _load(path)
    o, lse, dq, dk, dv = ao.attention_forward_backward(t["q"], t["k"], t["v"], t["d_o"],
                                                       causal=causal, scale=scale)
    # same ops in the same order as the reference: fp32 round-off only
    assert ao.rel_l2(o, t["o"]) < 1e-6
    assert ao.rel_l2(dq, t["dq"]) < 1e-6
    assert ao.rel_l2(dk, t["dk"]) < 1e-6
    assert ao.rel_l2(dv, t["dv"]) < 1e-6
    # lse is the oracle's addition: it must normalise the scores it was built from
    s = ao._scores(t["q"].double(), t["k"].double(), scale, causal)
    assert torch.allclose(torch.exp(s - lse.double().unsqueeze(-1)).sum(-1),
                          torch.ones_like(lse, dtype=torch.float64), atol=1e-5)


BIAS_CASES = sorted(glob.glob(os.path.join(GOLDEN, "test_twin_bias_*.npz")))


@pytest.mark.parametrize("path", BIAS_CASES, ids=[os.path.basename(p)[15:-4] for p in BIAS_CASES])
def test_python_oracle_matches_reference_test_twin_with_bias(path):
    """Additive bias: the fixtures come from the dense twin in the reference's own tests
    (tests/test_attention.py:30-87), gradients by autograd through it, dBias included."""
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in ("q", "k", "v", "d_o", "bias", "o", "dq", "dk", "dv", "dbias")}
    bias = t["bias"].clone().requires_grad_(True)
    o, lse, dq, dk, dv = ao.attention_forward_backward(t["q"], t["k"], t["v"], t["d_o"], causal=bool(z["causal"]),
                                                       scale=float(z["scale"]), bias=bias)
    for name, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv), ("dbias", bias.grad)):
        assert ao.rel_l2(got, t[name]) < 2e-6, name


def test_bias_fixtures_present():
    assert len(BIAS_CASES) == 3


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[10:-4] for p in CASES])
def test_c_oracle_matches_reference_math_path(path):
    t, causal, scale = _load(path)
    o, lse = c_oracle.forward(t["q"].numpy(), t["k"].numpy(), t["v"].numpy(), causal, scale)
    dq, dk, dv = c_oracle.backward(t["q"].numpy(), t["k"].numpy(), t["v"].numpy(), o, lse,
                                   t["d_o"].numpy(), causal, scale)
    assert ao.rel_l2(torch.from_numpy(o), t["o"]) < 1e-6
    assert ao.rel_l2(torch.from_numpy(dq), t["dq"]) < 2e-6
    assert ao.rel_l2(torch.from_numpy(dk), t["dk"]) < 2e-6
    assert ao.rel_l2(torch.from_numpy(dv), t["dv"]) < 2e-6


def test_cfg1_rows_match_reference():
    from flash_attention_v100.testing import WORKLOADS, make_inputs
    z = np.load(os.path.join(GOLDEN, "math_path_cfg1_rows.npz"))
    w = WORKLOADS["cfg1"]
    t = make_inputs(w)
    # the seeded generator reproduces the inputs the fixture was made from
    assert abs(t["q"].double().sum().item() - float(z["q_sum"])) < 1e-6
    assert abs(t["k"].double().sum().item() - float(z["k_sum"])) < 1e-6
    step = int(z["row_step"])
    o, _ = ao.chunked(ao.attention_forward, t["q"], t["k"], t["v"], heads_per_chunk=4,
                      causal=True, scale=w.scale)
    assert ao.rel_l2(o[:, ::step], torch.from_numpy(z["o_rows"])) < 1e-6


def test_closed_form_backward_matches_autograd_with_dropout_and_gqa():
    g = torch.Generator().manual_seed(7)
    q = torch.randn(2, 40, 4, 16, generator=g)
    k = torch.randn(2, 56, 2, 16, generator=g)
    v = torch.randn(2, 56, 2, 16, generator=g)
    d_o = torch.randn(2, 40, 4, 16, generator=g)
    keep = (torch.rand(2, 4, 40, 56, generator=g) > 0.25).to(torch.uint8)
    o, lse, dq, dk, dv = ao.attention_forward_backward(q, k, v, d_o, causal=True, dropout_p=0.25,
                                                       keep_mask=keep, compute_dtype=torch.float64)
    dq2, dk2, dv2 = ao.attention_backward_closed_form(q, k, v, o, lse, d_o, causal=True,
                                                      dropout_p=0.25, keep_mask=keep)
    for a, b in ((dq, dq2), (dk, dk2), (dv, dv2)):
        assert ao.rel_l2(b, a) < 1e-12
    oc, lsec = c_oracle.forward(q.numpy(), k.numpy(), v.numpy(), True, None, keep.numpy(), 0.25)
    dqc, dkc, dvc = c_oracle.backward(q.numpy(), k.numpy(), v.numpy(), oc, lsec, d_o.numpy(), True, None,
                                      keep.numpy(), 0.25)
    assert ao.rel_l2(torch.from_numpy(oc), o) < 1e-6
    assert ao.rel_l2(torch.from_numpy(lsec), lse) < 1e-6
    for a, b in ((dq, dqc), (dk, dkc), (dv, dvc)):
        assert ao.rel_l2(torch.from_numpy(b), a) < 1e-6


# Philox4x32-10 known answers published with the Random123 library
# (counter, key) -> output
PHILOX_KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
     (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


@pytest.mark.parametrize("ctr,key,expect", PHILOX_KAT)
def test_philox_known_answers(ctr, key, expect):
    from flash_attention_v100.kernels import _cabi
    assert c_oracle.philox4x32_10(ctr, key) == expect
    assert _cabi.philox4x32_10(ctr, key) == expect


def test_library_and_oracle_philox_agree_on_random_blocks():
    from flash_attention_v100.kernels import _cabi
    rng = np.random.default_rng(3)
    for _ in range(200):
        ctr = tuple(int(x) for x in rng.integers(0, 2 ** 32, 4))
        key = tuple(int(x) for x in rng.integers(0, 2 ** 32, 2))
        assert c_oracle.philox4x32_10(ctr, key) == _cabi.philox4x32_10(ctr, key)


@pytest.mark.parametrize("p", [0.0, 0.1, 0.5, 0.9])
def test_host_dropout_mask_matches_oracle_definition(p):
    import ctypes
    from flash_attention_v100.kernels import _cabi
    lib = _cabi.load()
    B, H, Nq, Nk = 2, 3, 37, 53
    seed, offset = 0x1234_5678_9ABC_DEF0, 0x1_0000_0005
    out = np.empty((B, H, Nq, Nk), np.uint8)
    rc = lib.fa_b200_dropout_mask_host(seed, offset, p, B, H, Nq, Nk, out.ctypes.data)
    assert rc == 0
    ref = c_oracle.dropout_mask(seed, offset, p, B, H, Nq, Nk)
    assert np.array_equal(out, ref)
    eff = lib.fa_b200_dropout_effective_p(p)
    assert abs(eff - round(p * 256) / 256) < 1e-7
    if p > 0:
        assert abs((1 - out.mean()) - eff) < 0.03
    else:
        assert out.all()


@pytest.mark.parametrize("nq,nk", [(5, 12), (7, 7), (1, 9)])
def test_causal_shift_equals_the_same_mask_given_as_a_bias(nq, nk):
    """The shifted diagonal (bottom-right alignment at shift = Nk - Nq) against the reference's own
    mechanism for arbitrary masks, a 0 / -inf bias; shift 0 is the reference's mask."""
    import torch
    from oracle import attention_oracle as ao
    g = torch.Generator().manual_seed(11)
    q, d_o = torch.randn(2, nq, 3, 8, generator=g), torch.randn(2, nq, 3, 8, generator=g)
    k, v = torch.randn(2, nk, 3, 8, generator=g), torch.randn(2, nk, 3, 8, generator=g)
    shift = nk - nq
    i, j = torch.arange(nq)[:, None], torch.arange(nk)[None, :]
    mask = torch.zeros(1, 1, nq, nk).masked_fill_((j > i + shift)[None, None], float("-inf"))
    a = ao.attention_forward_backward(q, k, v, d_o, causal=True, causal_shift=shift)
    b = ao.attention_forward_backward(q, k, v, d_o, causal=False, bias=mask)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-6, atol=1e-6)
    if shift == 0:
        c = ao.attention_forward_backward(q, k, v, d_o, causal=True)
        for x, y in zip(a, c):
            assert torch.equal(x, y)


@pytest.mark.parametrize("nq,nk", [(5, 12), (6, 6)])
def test_c_oracle_causal_shift_equals_the_torch_restatement(nq, nk):
    g = torch.Generator().manual_seed(12)
    q, d_o = torch.randn(1, nq, 2, 8, generator=g), torch.randn(1, nq, 2, 8, generator=g)
    k, v = torch.randn(1, nk, 1, 8, generator=g), torch.randn(1, nk, 1, 8, generator=g)
    shift = nk - nq
    ro, rlse, rdq, rdk, rdv = ao.attention_forward_backward(q, k, v, d_o, causal=True, causal_shift=shift)
    o, lse = c_oracle.forward(q.numpy(), k.numpy(), v.numpy(), causal=True, causal_shift=shift)
    dq, dk, dv = c_oracle.backward(q.numpy(), k.numpy(), v.numpy(), o, lse, d_o.numpy(), causal=True,
                                   causal_shift=shift)
    for got, want in ((o, ro), (lse, rlse), (dq, rdq), (dk, rdk), (dv, rdv)):
        assert np.allclose(got, want.numpy(), rtol=2e-5, atol=2e-5)
