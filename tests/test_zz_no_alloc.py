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
            assert torch.equal(a, b), f"call {call}: {name} differs from fa_b200_bwd (same kernels, same order)"


def test_static_backward_refuses_problems_beyond_its_array(device):
    lib = _cabi.load()
    B, N, H, D = 8, 4096, 40, 64          # 8*40*4096 = 1310720 rows > 1048576
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = B, N, N, H, H, D
    p.dtype, p.scale, p.device = _cabi.FA_B200_BF16, 0.125, device.index or 0
    fake = 4096                            # never dereferenced: the size check comes first
    for t in ("q", "k", "v", "o", "d_o", "dq", "dk", "dv"):
        getattr(p, t).ptr = fake
        getattr(p, t).stride_b, getattr(p, t).stride_n, getattr(p, t).stride_h = N * H * D, H * D, D
    p.lse = fake
    assert lib.fa_b200_bwd_static(ctypes.byref(p)) == _cabi.FA_EWORKSPACE
    assert b"1048576" in lib.fa_b200_last_error()
