"""The workspace-free backward entry point (fa_b200_bwd_static).

It serves callers that cannot allocate device memory for the library (hosts that
own all GPU memory, paths where cudaMalloc is off limits): its scratch is a fixed
array inside the library.  Checked here through the C ABI against the regular
entry point, twice in a row (the array keeps the first call's contents), and for
its size limit.  Collected last so a failure here cannot hide other tests.
"""
import ctypes

import pytest
import torch

from flash_attention_v100.kernels import _cabi
from flash_attention_v100.ops import attention as ops
from flash_attention_v100.testing import tolerance, rel_l2

pytestmark = pytest.mark.gpu


def _problem(device, B, N, H, D, dtype, seed, causal=True):
    g = torch.Generator().manual_seed(seed)
    q, k, v, d_o = (torch.randn(B, N, H, D, generator=g).to(dtype).to(device) for _ in range(4))
    scale = D ** -0.5
    o, lse = ops.launch_forward(q, k, v, scale, causal)
    return q, k, v, d_o, o, lse, scale, causal


def _bwd_static(q, k, v, d_o, o, lse, scale, causal):
    """Call fa_b200_bwd_static directly: no workspace pointer is passed."""
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = ops._base_params(q, k, v, o, lse, scale, causal, 0.0, 0, 0)
    p.d_o, p.dq, p.dk, p.dv = ops._tensor4(d_o), ops._tensor4(dq), ops._tensor4(dk), ops._tensor4(dv)
    p.workspace, p.workspace_bytes = None, 0
    rc = _cabi.load().fa_b200_bwd_static(ctypes.byref(p))
    _cabi.raise_for_status(rc, "fa_b200_bwd_static")
    return dq, dk, dv


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float32, 32)],
                         ids=["bf16-d128", "fp16-d64", "fp32-d32"])
def test_static_backward_matches_regular_entry_point_twice(device, dtype, D):
    # two different problems back to back: the second call finds the first one's
    # delta / lse values in the shared array and must not be affected by them
    for call, (B, N, H) in enumerate([(2, 300, 3), (1, 520, 2)]):
        args = _problem(device, B, N, H, D, dtype, seed=100 + call)
        q, k, v, d_o, o, lse, scale, causal = args
        # the static entry serves tensor-core calls with the two-pass backward: ask the regular
        # entry for the same kernels
        with ops.kernel_variant("tcgen05_2pass" if dtype != torch.float32 else "auto"):
            ref = ops.launch_backward(d_o, q, k, v, o, lse, scale, causal)
        got = _bwd_static(*args)
        torch.cuda.synchronize()
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert rel_l2(a, b) <= tolerance(dtype), f"call {call}: {name}"
            if dtype == torch.bfloat16:
                # fa_b200_bwd streams fp16 copies of Q, dO and K from its workspace; without one the
                # same kernels convert the bf16 tiles themselves and normalise dO per column instead
                # of per row: the same arithmetic up to roundings far below bf16's last place
                assert rel_l2(a, b) <= 2e-4, f"call {call}: {name}: {rel_l2(a, b):.2e}"
            else:
                assert torch.equal(a, b), f"call {call}: {name} differs from fa_b200_bwd (same kernels, same order)"


def test_static_backward_against_the_oracle(device):
    """The workspace-free entry compared with the CPU oracle directly, not only with fa_b200_bwd."""
    from oracle import attention_oracle as ao
    B, N, H, D = 1, 260, 2, 64
    g = torch.Generator().manual_seed(7)
    qc, kc, vc, gc = (torch.randn(B, N, H, D, generator=g).to(torch.float16) for _ in range(4))
    q, k, v, d_o = (t.to(device) for t in (qc, kc, vc, gc))
    o, lse = ops.launch_forward(q, k, v, D ** -0.5, True)
    got = _bwd_static(q, k, v, d_o, o, lse, D ** -0.5, True)
    torch.cuda.synchronize()
    ref = ao.attention_forward_backward(qc.float(), kc.float(), vc.float(), gc.float(), causal=True)[2:]
    for name, a, r in zip(("dq", "dk", "dv"), got, ref):
        assert rel_l2(a, r) <= tolerance(torch.float16), name


def test_static_backward_without_queries_zero_fills_like_the_regular_entry(device):
    B, Nk, H, D = 2, 40, 2, 64
    k = torch.randn(B, Nk, H, D, device=device).to(torch.float16)
    q = torch.empty(B, 0, H, D, dtype=torch.float16, device=device)
    lse = torch.empty(B, H, 0, dtype=torch.float32, device=device)
    dk, dv = torch.ones_like(k), torch.ones_like(k)
    p = ops._base_params(q, k, k, q, lse, 0.125, False, 0.0, 0, 0)
    p.lse = dk.data_ptr()          # any non-null pointer: an empty lse has none and is never read
    p.d_o, p.dq, p.dk, p.dv = ops._tensor4(q), ops._tensor4(q), ops._tensor4(dk), ops._tensor4(dv)
    for t in ("q", "o", "d_o", "dq"):
        getattr(p, t).ptr = dk.data_ptr()      # empty tensors: never dereferenced
    rc = _cabi.load().fa_b200_bwd_static(ctypes.byref(p))
    _cabi.raise_for_status(rc, "fa_b200_bwd_static")
    torch.cuda.synchronize()
    assert not dk.any() and not dv.any()


@pytest.mark.parametrize("dtype,D", [(_cabi.FA_B200_BF16, 64), (_cabi.FA_B200_F32, 32)], ids=["tensor-core", "cuda-core"])
def test_static_backward_refuses_problems_beyond_its_array(dtype, D):
    """One row limit for every kernel family, checked before anything else.  The call carries NO
    pointers at all: should the size check ever be skipped, the null-pointer check refuses the call
    too, so this test can never reach a kernel launch."""
    lib = _cabi.load()
    B, N, H = 16, 4096, 40                 # 16*40*4096 = 2621440 rows > 1048576
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = B, N, N, H, H, D
    p.dtype, p.scale, p.device = dtype, 0.125, 0
    assert lib.fa_b200_bwd_static(ctypes.byref(p)) == _cabi.FA_EWORKSPACE
    assert b"1048576" in lib.fa_b200_last_error()
    p.B = 1                                # within the limit: now the missing pointers are what is refused
    assert lib.fa_b200_bwd_static(ctypes.byref(p)) == _cabi.FA_EINVAL
