"""Generate golden vectors from the reference's own math attention path.

Run in the build container (where the reference tree is mounted):

    python tests/golden/make_golden.py /path/to/parent/of/reference

It imports the reference package (whose top-level `flash_attention_v100` is the
PyTorch math path, reference __init__.py:30-55), runs it and autograd through
it on small seeded fp32 inputs, and stores inputs and outputs in
tests/golden/math_path_*.npz.  The fixtures are committed; tests never import
the reference.
"""
import io
import os
import sys
from contextlib import redirect_stdout

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "flash-attn-v100_b200"))

CASES = [
    # name, B, N, H, D, causal, scale
    ("b2n64h3d32_full", 2, 64, 3, 32, False, None),
    ("b1n128h2d64_causal", 1, 128, 2, 64, True, None),
    ("b2n96h2d64_causal", 2, 96, 2, 64, True, None),
    ("b1n200h2d128_full_scale0p1", 1, 200, 2, 128, False, 0.1),
    ("b1n130h1d16_causal", 1, 130, 1, 16, True, 0.3),
]


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_golden.py <directory that holds the reference checkout as 'reference/'>")
    parent = sys.argv[1]
    sys.path.insert(0, parent)
    with redirect_stdout(io.StringIO()):      # the reference prints a no-CUDA warning on import
        import reference
    fn = reference.flash_attention_v100
    assert fn.__doc__ == "Simple fallback implementation", "expected the reference's math path"
    torch.manual_seed(0)
    for name, b, n, h, d, causal, scale in CASES:
        g = torch.Generator().manual_seed(1234 + n)
        q, k, v, d_o = (torch.randn(b, n, h, d, generator=g) for _ in range(4))
        qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
        kw = {"causal": causal}
        if scale is not None:
            kw["scale"] = scale
        o = fn(qa, ka, va, **kw)
        o.backward(d_o)
        np.savez_compressed(
            os.path.join(HERE, f"math_path_{name}.npz"),
            q=q.numpy(), k=k.numpy(), v=v.numpy(), d_o=d_o.numpy(), o=o.detach().numpy(),
            dq=qa.grad.numpy(), dk=ka.grad.numpy(), dv=va.grad.numpy(),
            causal=np.array(causal), scale=np.array(d ** -0.5 if scale is None else scale, np.float64))
        print("wrote", name, tuple(o.shape))

    # Additive bias: the top-level math path takes none, so these come from the dense twin the
    # reference's own tests compare against (tests/test_attention.py:30-87: scores * scale + bias,
    # then the causal mask, softmax, P V), with autograd through it for dQ, dK, dV and dBias.
    with redirect_stdout(io.StringIO()):
        import reference.tests.test_attention as ref_tests
    twin = ref_tests.flash_attention_v100
    assert twin.__doc__ == "Simple flash attention implementation for testing"
    for name, b, n, h, d, causal, bias_shape in [
            ("bias_full_b2n80h3d32", 2, 80, 3, 32, False, (2, 3, 80, 80)),
            ("bias_heads_bcast_b2n96h2d64_causal", 2, 96, 2, 64, True, (2, 1, 96, 96)),
            ("bias_both_bcast_b1n70h2d16", 1, 70, 2, 16, False, (1, 1, 70, 70))]:
        g = torch.Generator().manual_seed(4321 + n)
        q, k, v, d_o = (torch.randn(b, n, h, d, generator=g) for _ in range(4))
        bias = torch.randn(bias_shape, generator=g)
        qa, ka, va, ba = (t.clone().requires_grad_(True) for t in (q, k, v, bias))
        o = twin(qa, ka, va, causal=causal, bias=ba)
        o.backward(d_o)
        np.savez_compressed(
            os.path.join(HERE, f"test_twin_{name}.npz"),
            q=q.numpy(), k=k.numpy(), v=v.numpy(), d_o=d_o.numpy(), bias=bias.numpy(), o=o.detach().numpy(),
            dq=qa.grad.numpy(), dk=ka.grad.numpy(), dv=va.grad.numpy(), dbias=ba.grad.numpy(),
            causal=np.array(causal), scale=np.array(d ** -0.5, np.float64))
        print("wrote", name, tuple(o.shape))

    # README quick-start shape (B2 N1024 H12 D64 fp32 causal, seed 0): inputs come from
    # the package's seeded generator; every 37th query row of O is stored.
    from flash_attention_v100.testing import WORKLOADS, make_inputs
    w = WORKLOADS["cfg1"]
    t = make_inputs(w)
    o = fn(t["q"], t["k"], t["v"], causal=True, scale=w.scale)
    np.savez_compressed(os.path.join(HERE, "math_path_cfg1_rows.npz"),
                        o_rows=o[:, ::37].numpy(), row_step=np.array(37),
                        q_sum=np.array(t["q"].double().sum().item()),
                        k_sum=np.array(t["k"].double().sum().item()),
                        v_sum=np.array(t["v"].double().sum().item()))
    print("wrote cfg1 rows", tuple(o[:, ::37].shape))


if __name__ == "__main__":
    main()
