"""Sequence-parallel attention on the GPU: the combination kernel, and the ring over the CUDA library.

The ring's ranks run as threads of this process on one device (no kernel waits
for another: ranks hand messages over on the host), so these tests need one GPU;
the NCCL ring over two GPUs is in test_gpu_multi.py."""
import pytest
import torch

import flash_attention_v100 as fa
from flash_attention_v100.ops import attention as ops
from flash_attention_v100.ops import sequence_parallel as sp
from oracle import attention_oracle as orc
from ring_helpers import OracleBlockKernels, run_ring

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [64, 40, 8, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_combine_merge_matches_formula(device, dtype, D):
    B, N, H = 2, 70, 3
    g = torch.Generator().manual_seed(1)
    wide = torch.randn(3, B, N, H, 2 * D, generator=g).to(dtype).to(device)
    parts = [wide[i, ..., :D] for i in range(3)]                     # strided views: row pitch 2 D
    lses = [torch.randn(B, H, N, generator=g).to(device) for _ in range(3)]
    lses[1][0, 0, :5] = float("-inf")                                 # rows that saw no key in one block
    lses[0][1, 2, 7] = lses[1][1, 2, 7] = lses[2][1, 2, 7] = float("-inf")   # ... and in no block
    acc = torch.full((B, N, H, D), float("nan"), device=device)      # `first` must not read it
    lse = torch.full((B, H, N), float("nan"), device=device)
    out_wide = torch.zeros(B, N, H, 2 * D, dtype=dtype, device=device)
    out = out_wide[..., D:]
    acc_ref = torch.empty(B, N, H, D)
    lse_ref = torch.empty(B, H, N)
    out_ref = torch.empty(B, N, H, D, dtype=dtype)
    for i in range(3):
        ops.launch_combine(acc, parts[i], lse, lses[i], out=out if i == 2 else None, first=(i == 0))
        OracleBlockKernels.combine(acc_ref, parts[i].cpu(), lse_ref, lses[i].cpu(),
                                   out=out_ref if i == 2 else None, first=(i == 0))
    torch.cuda.synchronize()
    assert torch.equal(torch.isinf(lse.cpu()), torch.isinf(lse_ref))
    fin = ~torch.isinf(lse_ref)
    assert torch.allclose(lse.cpu()[fin], lse_ref[fin], rtol=0, atol=5e-6)
    assert not torch.isnan(acc).any()
    assert torch.allclose(acc.cpu(), acc_ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(out.float().cpu(), out_ref.float(), rtol=1e-2 if dtype != torch.float32 else 1e-5, atol=1e-5)
    assert torch.all(out_wide[..., :D] == 0), "the output view's neighbours were written"
    assert torch.all(acc[1, 7, 2] == 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_combine_sum_and_convert_only(device, dtype):
    B, N, H, D = 1, 33, 2, 128
    g = torch.Generator().manual_seed(2)
    parts = [torch.randn(B, N, H, D, generator=g).to(dtype).to(device) for _ in range(4)]
    acc = torch.full((B, N, H, D), float("nan"), device=device)
    for i, p in enumerate(parts):
        ops.launch_combine(acc, p, first=(i == 0))
    out = torch.empty(B, N, H, D, dtype=dtype, device=device)
    ops.launch_combine(acc, None, out=out)
    want = parts[0].float() + parts[1].float() + parts[2].float() + parts[3].float()
    assert torch.equal(acc, want)                                    # same order of fp32 additions
    assert torch.equal(out, want.to(dtype))


def test_combine_on_a_range_of_rows(device):
    """acc and lse_acc may be a range of rows of a larger total (the zigzag layout's second chunk)."""
    B, N, H, D, c = 2, 40, 3, 64, 24
    g = torch.Generator().manual_seed(5)
    acc = torch.randn(B, N, H, D, generator=g).to(device)
    lse = torch.randn(B, H, N, generator=g).to(device)
    part = torch.randn(B, N - c, H, D, generator=g).to(torch.bfloat16).to(device)
    lse_part = torch.randn(B, H, N - c, generator=g).to(device)
    acc_ref, lse_ref = acc.cpu().clone(), lse.cpu().clone()
    ops.launch_combine(acc[:, c:], part, lse[:, :, c:], lse_part)
    OracleBlockKernels.combine(acc_ref[:, c:], part.cpu(), lse_ref[:, :, c:], lse_part.cpu())
    assert torch.equal(acc[:, :c].cpu(), acc_ref[:, :c]) and torch.equal(lse[:, :, :c].cpu(), lse_ref[:, :, :c])
    assert torch.allclose(acc.cpu(), acc_ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(lse.cpu(), lse_ref, rtol=0, atol=5e-6)
    with pytest.raises(ValueError):
        ops.launch_combine(acc[:, :, :2], part[:, :, :2])            # rows of a batch entry not dense


def test_combine_rejects_bad_operands(device):
    acc = torch.zeros(1, 8, 1, 64, device=device)
    part = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16, device=device)
    with pytest.raises(ValueError):
        ops.launch_combine(acc.half(), part)
    with pytest.raises(ValueError):
        ops.launch_combine(acc, None)
    with pytest.raises(ValueError):
        ops.launch_combine(torch.zeros(1, 8, 1, 60, device=device), torch.zeros(1, 8, 1, 60, device=device))
    with pytest.raises(ValueError):
        ops.launch_combine(acc, part, lse_acc=torch.zeros(1, 8, 1, device=device))


def _rank_call(ring, q, k, v, d_o, causal, layout="contiguous"):
    # ring_forward / ring_backward are called directly: autograd would run every rank's backward on
    # the one worker thread it keeps per device, where the ranks of a thread ring would wait for each
    # other for ever.  The autograd wrapper is covered below with one rank and, over NCCL, with two GPUs.
    if layout == "zigzag":
        ql, kl, vl, gl = (sp.zigzag_split(t, ring.world, ring.rank) for t in (q, k, v, d_o))
    else:
        ql, kl, vl, gl = (t.chunk(ring.world, dim=1)[ring.rank].contiguous() for t in (q, k, v, d_o))
    scale = q.shape[3] ** -0.5
    o, lse = sp.ring_forward(ql, kl, vl, scale, causal, ring, layout=layout)
    dq, dk, dv = sp.ring_backward(gl, ql, kl, vl, o, lse, scale, causal, ring, layout=layout)
    return o, lse, dq, dk, dv


@pytest.mark.parametrize("world,causal,dtype,H,Hkv,D,n,layout", [
    (2, True, torch.bfloat16, 4, 4, 128, 256, "contiguous"),
    (4, True, torch.bfloat16, 4, 2, 128, 192, "contiguous"),   # ragged slices (not a multiple of 128), GQA
    (3, False, torch.float16, 2, 2, 64, 128, "contiguous"),
    (2, True, torch.float32, 2, 2, 64, 96, "contiguous"),      # CUDA-core kernels
    (2, True, torch.bfloat16, 4, 4, 128, 256, "zigzag"),
    (4, True, torch.bfloat16, 4, 2, 128, 176, "zigzag"),       # chunks of 88 rows, GQA
    (3, True, torch.float16, 2, 2, 64, 256, "zigzag"),
    (2, True, torch.float32, 2, 1, 64, 96, "zigzag"),
])
def test_ring_on_one_device_equals_whole_sequence(device, world, causal, dtype, H, Hkv, D, n, layout):
    B, N = 2, n * world
    g = torch.Generator().manual_seed(3)
    qc = (0.5 * torch.randn(B, N, H, D, generator=g)).to(dtype)
    kc = (0.5 * torch.randn(B, N, Hkv, D, generator=g)).to(dtype)
    vc = (0.5 * torch.randn(B, N, Hkv, D, generator=g)).to(dtype)
    gc = torch.randn(B, N, H, D, generator=g).to(dtype)
    q, k, v, d_o = (t.to(device) for t in (qc, kc, vc, gc))
    res = run_ring(world, lambda ring: _rank_call(ring, q, k, v, d_o, causal, layout))
    torch.cuda.synchronize()
    ops.check_status(device)
    join = (lambda parts, dim: sp.zigzag_merge(parts, dim)) if layout == "zigzag" else \
        (lambda parts, dim: torch.cat(parts, dim=dim))
    o, dq, dk, dv = (join([r[i] for r in res], 1) for i in (0, 2, 3, 4))
    lse = join([r[1] for r in res], 2)
    # against the oracle on the dtype-rounded inputs ...
    ref = orc.attention_forward_backward(qc.float(), kc.float(), vc.float(), gc.float(), causal=causal)
    # ... and against one call over the whole sequence on the same device
    q1, k1, v1 = (t.clone().requires_grad_(True) for t in (q, k, v))
    o1, lse1 = fa.flash_attention_v100(q1, k1, v1, causal=causal, return_softmax_lse=True)
    o1.backward(d_o)
    one = (o1.detach(), lse1, q1.grad, k1.grad, v1.grad)
    # tolerance: 2e-3 for one call in 16-bit types; each block's partial is rounded to the dtype before it
    # is folded in, which adds up to one more rounding per block
    tol = 1e-5 if dtype == torch.float32 else 4e-3
    for name, got, want, single in zip(("o", "lse", "dq", "dk", "dv"), (o, lse, dq, dk, dv), ref, one):
        assert orc.rel_l2(got, want) < (1e-5 if name == "lse" else tol), name
        assert orc.rel_l2(got, single) < (1e-5 if name == "lse" else tol), name


def test_autograd_wrapper_one_rank_equals_plain_call(device):
    class OneRank:
        rank, world = 0, 1

        @staticmethod
        def exchange(send, recv):
            if send is not None and recv is not None:
                recv.copy_(send)
            return []

        @staticmethod
        def wait(pending):
            pass

    g = torch.Generator().manual_seed(4)
    qc, kc, vc, gc = (torch.randn(1, 300, 2, 64, generator=g).to(torch.float16) for _ in range(4))
    a = [t.to(device).requires_grad_(True) for t in (qc, kc, vc)]
    b = [t.to(device).requires_grad_(True) for t in (qc, kc, vc)]
    o, lse = fa.flash_attention_v100_sequence_parallel(*a, causal=True, return_softmax_lse=True, ring=OneRank())
    o.backward(gc.to(device))
    o1, lse1 = fa.flash_attention_v100(*b, causal=True, return_softmax_lse=True)
    o1.backward(gc.to(device))
    assert not lse.requires_grad
    assert torch.equal(lse, lse1)
    assert torch.equal(o, o1)                      # one block: the fp32 round trip is exact
    for x, y in zip(a, b):
        assert orc.rel_l2(x.grad, y.grad) < 1e-3
