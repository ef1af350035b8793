"""Seeded synthetic workloads and error metrics shared by tests and bench.

The five workloads are the benchmark configurations of this build (shapes,
dtypes and value distributions).  Inputs are drawn on the CPU from a seeded
generator in the order q, k, v, dO, scaled, then rounded to the workload's
dtype, so a CPU checker and the GPU kernels see bit-identical values.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, Optional

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    N: int
    H: int
    D: int
    dtype: torch.dtype
    causal: bool
    dropout_p: float = 0.0
    qkv_std: float = 1.0        # q, k, v ~ N(0, qkv_std^2)
    outlier_rows: float = 0.0   # fraction of q/k rows scaled x8
    backward: bool = True
    seed: int = 0

    @property
    def scale(self) -> float:
        return self.D ** -0.5

    def fwd_flops(self) -> float:
        return 4.0 * self.B * self.H * self.N * self.N * self.D * (0.5 if self.causal else 1.0)

    def bwd_flops(self) -> float:
        return 2.5 * self.fwd_flops()

    def tensor_bytes(self) -> int:
        return self.B * self.N * self.H * self.D * torch.empty((), dtype=self.dtype).element_size()

    def shrink(self, **kw) -> "Workload":
        return replace(self, **kw)


WORKLOADS: Dict[str, Workload] = {
    "cfg1": Workload("cfg1 B2 N1024 H12 D64 fp32 causal (forward)", 2, 1024, 12, 64, torch.float32, True,
                     backward=False),
    "cfg2": Workload("cfg2 B8 N2048 H16 D64 fp16 full", 8, 2048, 16, 64, torch.float16, False),
    "cfg3": Workload("cfg3 B4 N4096 H32 D128 bf16 causal", 4, 4096, 32, 128, torch.bfloat16, True,
                     qkv_std=0.5),
    "cfg4": Workload("cfg4 B1 N16384 H32 D128 bf16 causal long-context", 1, 16384, 32, 128,
                     torch.bfloat16, True, outlier_rows=0.01),
    "cfg5": Workload("cfg5 B32 N2048 H16 D64 bf16 causal dropout 0.1", 32, 2048, 16, 64, torch.bfloat16,
                     True, dropout_p=0.1),
}
DROPOUT_SEED, DROPOUT_OFFSET = 0x5EED, 0


def make_inputs(w: Workload, device: Optional[torch.device] = None, seed: Optional[int] = None,
                pin: bool = False) -> Dict[str, torch.Tensor]:
    """q, k, v, d_o of shape (B, N, H, D) in w.dtype."""
    g = torch.Generator().manual_seed(w.seed if seed is None else seed)
    shape = (w.B, w.N, w.H, w.D)
    out = {}
    for name in ("q", "k", "v", "d_o"):
        t = torch.randn(shape, generator=g, dtype=torch.float32)
        if name != "d_o":
            t *= w.qkv_std
        out[name] = t
    if w.outlier_rows > 0:
        for name in ("q", "k"):
            pick = torch.rand((w.B, w.N, w.H, 1), generator=g) < w.outlier_rows
            out[name] = torch.where(pick, out[name] * 8.0, out[name])
    for name in out:
        t = out[name].to(w.dtype)
        if pin and torch.cuda.is_available():
            t = t.pin_memory()
        if device is not None:
            t = t.to(device)
        out[name] = t
    return out


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    """||x - ref||_2 / ||ref||_2, accumulated in float64."""
    x = x.detach().double().cpu()
    ref = ref.detach().double().cpu()
    den = ref.norm().item()
    num = (x - ref).norm().item()
    if den == 0.0:
        return 0.0 if num == 0.0 else math.inf
    return num / den


# Relative-L2 tolerance per dtype: outputs and gradients vs the fp32 math path evaluated on the
# dtype-rounded inputs: 2e-3 for fp16 and bf16, 1e-5 for fp32.  Measured on B200: fp32 1e-6, fp16
# 3e-4, bf16 O 1.6e-3, dV 1.7e-3, dQ / dK 1.8e-3.  Rounding an exact result to bf16 (8 significant
# bits) alone costs 1.6e-3, so bf16 has room for little else: the tensor-core kernels round P and
# dS to fp16, not bf16 (bf16 operand tiles are converted to fp16 for the MMAs), because a bf16
# rounding of P or dS reaches the result at full size (with zero-mean V / K / Q / dO the products
# add like a random walk) and put O at 2.2e-3 and dQ / dK at 2.5e-3.
TOLERANCE = {torch.float16: 2e-3, torch.bfloat16: 2e-3, torch.float32: 1e-5}
TOLERANCE_TARGET = dict(TOLERANCE)


def tolerance(dtype: torch.dtype, variant: str = "auto", head_dim: int = 128) -> float:
    return TOLERANCE[dtype]


def dq_is_bit_reproducible(variant: str, dtype: torch.dtype, head_dim: int, dropout_p: float = 0.0) -> bool:
    """Whether two backward calls on the same inputs return the same dQ bit for bit.
    dK, dV, O and LSE always do, and so does dQ by default ("auto").  Only the opt-in
    fast variant ("tcgen05": optimization_strategy="speed") sums dQ tiles with
    unordered fp32 additions, for fp16/bf16 with D = 64."""
    if variant != "tcgen05":
        return True
    return not (dtype in (torch.float16, torch.bfloat16) and head_dim == 64)


def assert_same_dq(a: torch.Tensor, b: torch.Tensor, exact: bool, what: str = "dQ") -> None:
    """Bitwise when `exact`; otherwise equal up to the reordering of fp32 sums
    before the final rounding (a few last-place flips of the 16-bit result)."""
    if exact:
        assert torch.equal(a, b), f"{what} differs bitwise"
    else:
        err = rel_l2(a, b)
        assert err <= 1e-3, f"{what}: rel-L2 {err:.2e} between two summation orders"
