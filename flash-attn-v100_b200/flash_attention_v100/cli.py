"""Command-line benchmark (`flash-attn-benchmark`).

Counterpart of the reference's console script (pyproject.toml:63-64, which runs
examples/basic_usage.py:818-873): prints what the machine offers, then times
the attention forward and backward on one device.  Times come from CUDA events
on the launching stream, not from the host clock (the reference uses
time.time() around a synchronize, examples/basic_usage.py:640-700).
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def get_device_info() -> Dict[str, Any]:
    """Same keys as the reference's utils.get_device_info (utils.py:563-602), with
    `b200_compatible` where the reference reports `v100_compatible`."""
    info: Dict[str, Any] = {
        "cuda_available": torch.cuda.is_available(),
        "cuda_device_count": torch.cuda.device_count() if torch.cuda.is_available() else 0,
        "pytorch_version": torch.__version__,
        "distributed_available": dist.is_available(),
        "distributed_initialized": dist.is_available() and dist.is_initialized(),
        "system": {"cpu_count": os.cpu_count()},
    }
    if info["cuda_available"]:
        devices = []
        for i in range(torch.cuda.device_count()):
            props = torch.cuda.get_device_properties(i)
            cap = torch.cuda.get_device_capability(i)
            devices.append({"device_id": i, "name": props.name, "compute_capability": cap,
                            "total_memory_gb": props.total_memory / 2 ** 30,
                            "multi_processor_count": props.multi_processor_count,
                            "b200_compatible": cap[0] == 10, "tensor_core_support": cap[0] == 10})
        info["devices"] = devices
        info["current_device"] = torch.cuda.current_device()
    return info


def attention_flops(batch: int, seq_q: int, seq_k: int, heads: int, head_dim: int, causal: bool) -> Dict[str, float]:
    """Counted FLOPs: forward 4 B H Nq Nk D (the reference's figure, kernels/autotuning.py:763),
    backward 2.5 times that, both halved under a causal mask."""
    fwd = 4.0 * batch * heads * seq_q * seq_k * head_dim * (0.5 if causal else 1.0)
    return {"fwd": fwd, "bwd": 2.5 * fwd}


def run_benchmark(batch: int, seq_len: int, heads: int, head_dim: int, dtype: torch.dtype, causal: bool,
                  dropout_p: float = 0.0, steps: int = 20, warmup: int = 5, device: int = 0,
                  heads_kv: Optional[int] = None) -> Dict[str, Any]:
    """Median forward and backward times over `steps` launches, inputs resident on the device."""
    from . import flash_attention_v100
    if not torch.cuda.is_available():
        raise RuntimeError("flash-attn-benchmark needs a CUDA device: there is no CPU path")
    dev = torch.device("cuda", device)
    gen = torch.Generator().manual_seed(0)
    hkv = heads if heads_kv is None else heads_kv
    mk = lambda h: torch.randn(batch, seq_len, h, head_dim, generator=gen).to(dtype).to(dev).requires_grad_(True)
    q, k, v = mk(heads), mk(hkv), mk(hkv)
    d_o = torch.randn(batch, seq_len, heads, head_dim, generator=gen).to(dtype).to(dev)
    fwd_ms: List[float] = []
    bwd_ms: List[float] = []
    for it in range(warmup + steps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        o = flash_attention_v100(q, k, v, causal=causal, dropout_p=dropout_p)
        e[1].record()
        o.backward(d_o)
        e[2].record()
        e[2].synchronize()
        q.grad = k.grad = v.grad = None
        if it >= warmup:
            fwd_ms.append(e[0].elapsed_time(e[1]))
            bwd_ms.append(e[1].elapsed_time(e[2]))
    med = lambda x: sorted(x)[len(x) // 2]
    fl = attention_flops(batch, seq_len, seq_len, heads, head_dim, causal)
    f, b = med(fwd_ms), med(bwd_ms)
    return {"shape": [batch, seq_len, heads, head_dim], "heads_kv": hkv, "dtype": str(dtype).replace("torch.", ""),
            "causal": causal, "dropout_p": dropout_p, "steps": steps, "warmup": warmup,
            "fwd_ms": f, "bwd_ms": b, "fwd_tflops": fl["fwd"] / f * 1e-9, "bwd_tflops": fl["bwd"] / b * 1e-9,
            "fwd_bwd_tflops": (fl["fwd"] + fl["bwd"]) / (f + b) * 1e-9}


def run_sequence_parallel_benchmark(batch: int, seq_len: int, heads: int, head_dim: int, dtype: torch.dtype,
                                    causal: bool, layout: str, steps: int = 5, warmup: int = 3,
                                    heads_kv: Optional[int] = None) -> Dict[str, Any]:
    """Forward + backward of one sequence of `seq_len` positions split over the ranks of a torchrun
    launch (one process per GPU, NCCL).  Time: CUDA events around `steps` steps, the maximum over
    ranks; TFLOP/s of the whole job."""
    from . import flash_attention_v100_sequence_parallel
    if not torch.cuda.is_available():
        raise RuntimeError("flash-attn-benchmark needs a CUDA device: there is no CPU path")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    started = not dist.is_initialized()
    if started:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        if seq_len % (2 * world) != 0:
            raise ValueError(f"--seq-len must be a multiple of {2 * world}")
        n, hkv = seq_len // world, heads if heads_kv is None else heads_kv
        gen = torch.Generator().manual_seed(rank)
        mk = lambda h: torch.randn(batch, n, h, head_dim, generator=gen).to(dtype).to(dev).requires_grad_(True)
        q, k, v = mk(heads), mk(hkv), mk(hkv)
        d_o = torch.randn(batch, n, heads, head_dim, generator=gen).to(dtype).to(dev)

        def step():
            o = flash_attention_v100_sequence_parallel(q, k, v, causal=causal, layout=layout)
            o.backward(d_o)
            q.grad = k.grad = v.grad = None

        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        fl = attention_flops(batch, seq_len, seq_len, heads, head_dim, causal)
        return {"rank": rank, "n_gpus": world, "shape": [batch, seq_len, heads, head_dim], "per_rank": n,
                "heads_kv": hkv, "dtype": str(dtype).replace("torch.", ""), "causal": causal, "layout": layout,
                "steps": steps, "warmup": warmup, "ms_per_step": ms.item(),
                "fwd_bwd_tflops": (fl["fwd"] + fl["bwd"]) / ms.item() * 1e-9}
    finally:
        if started:
            dist.destroy_process_group()


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="flash-attn-benchmark", description=__doc__.split("\n\n")[0])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--heads-kv", type=int, default=None)
    ap.add_argument("--head-dim", type=int, default=128, choices=(64, 128))
    ap.add_argument("--dtype", default="bf16", choices=sorted(_DTYPES))
    ap.add_argument("--causal", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--dropout", type=float, default=0.0)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--json", action="store_true", help="print one JSON line instead of text")
    ap.add_argument("--sequence-parallel", choices=("contiguous", "zigzag"), default=None,
                    help="under torchrun: split one sequence of --seq-len over the ranks (ring attention)")
    args = ap.parse_args(argv)
    if args.sequence_parallel:
        if not torch.cuda.is_available():
            print("CUDA not available: nothing to time (there is no CPU path).")
            return 1
        res = run_sequence_parallel_benchmark(args.batch, args.seq_len, args.heads, args.head_dim,
                                              _DTYPES[args.dtype], args.causal, args.sequence_parallel,
                                              args.steps, args.warmup, args.heads_kv)
        if res["rank"] == 0:
            print(json.dumps(res) if args.json else
                  f"{res['n_gpus']} GPUs, (B, N, H, D) = {tuple(res['shape'])}, {res['per_rank']} positions per "
                  f"rank, causal={res['causal']}, {res['layout']}: {res['ms_per_step']:.3f} ms per forward + "
                  f"backward, {res['fwd_bwd_tflops']:.1f} TFLOP/s")
        return 0

    info = get_device_info()
    if not args.json:
        print(f"PyTorch {info['pytorch_version']}, CUDA available: {info['cuda_available']}, "
              f"GPUs: {info['cuda_device_count']}, distributed available: {info['distributed_available']}")
        for d in info.get("devices", []):
            print(f"  GPU {d['device_id']}: {d['name']} (CC {d['compute_capability']}, "
                  f"{d['total_memory_gb']:.1f} GB, {d['multi_processor_count']} SMs)")
    if not info["cuda_available"]:
        print("CUDA not available: nothing to time (there is no CPU path).")
        return 1
    res = run_benchmark(args.batch, args.seq_len, args.heads, args.head_dim, _DTYPES[args.dtype], args.causal,
                        args.dropout, args.steps, args.warmup, args.device, args.heads_kv)
    if args.json:
        print(json.dumps(res))
    else:
        print(f"shape (B, N, H, D) = {tuple(res['shape'])}, {res['dtype']}, causal={res['causal']}, "
              f"dropout={res['dropout_p']}")
        print(f"  forward   {res['fwd_ms']:.3f} ms  {res['fwd_tflops']:.1f} TFLOP/s")
        print(f"  backward  {res['bwd_ms']:.3f} ms  {res['bwd_tflops']:.1f} TFLOP/s")
        print(f"  together  {res['fwd_ms'] + res['bwd_ms']:.3f} ms  {res['fwd_bwd_tflops']:.1f} TFLOP/s")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
