"""Public API: flash_attention_v100(), FlashAttentionV100Manager and wrappers.

Same names, parameters, defaults and return values as the reference's
interface.py (flash_attention_v100 :199-348, FlashAttentionV100Manager :25-185,
get_flash_attention_manager :188-196, wrappers and context managers :612-661).
The bodies differ: tiles come from a static table, validation is O(1) host
work, there is no PyTorch/CPU fallback, and the multi-GPU path shards the
(batch x heads) grid over the GPUs of one box with no collective inside
attention.
"""
from __future__ import annotations

import contextlib
import logging
import os
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from .config import get_enhanced_config
from .ops.attention import FlashAttentionV100Function
from .utils import validate_inputs as _validate_inputs

log = logging.getLogger("flash_attention_v100")

Shard = Tuple[int, int, int, int]   # (b0, b1, h0, h1): half-open batch and head ranges


def plan_shards(batch_size: int, num_heads: int, num_parts: int, num_heads_kv: Optional[int] = None
                ) -> Tuple[str, List[Shard]]:
    """Split the (batch x heads) grid into `num_parts` independent shards.

    Heads are preferred when they divide evenly (the reference's head-parallel
    rule, interface.py:361 and :170-185), then batch; otherwise heads (or, with
    too few heads, batches) are split unevenly and trailing parts may be empty.
    K/V heads must split along with the query heads, so head splits are only
    taken at multiples of the group size H/Hkv.
    """
    hkv = num_heads if num_heads_kv is None else num_heads_kv
    group = num_heads // hkv
    g = max(1, int(num_parts))

    def even(total, parts, unit=1):
        per = total // parts
        return [(i * per, (i + 1) * per) for i in range(parts)]

    def uneven(total, parts, unit=1):
        units = total // unit
        out, start = [], 0
        for i in range(parts):
            n = units // parts + (1 if i < units % parts else 0)
            out.append((start * unit, (start + n) * unit))
            start += n
        return out

    if hkv % g == 0:
        return "head_parallel", [(0, batch_size, h0, h1) for h0, h1 in even(num_heads, g)]
    if batch_size % g == 0:
        return "batch_parallel", [(b0, b1, 0, num_heads) for b0, b1 in even(batch_size, g)]
    if hkv >= g or hkv >= batch_size:
        return "head_parallel", [(0, batch_size, h0, h1) for h0, h1 in uneven(num_heads, g, group)]
    return "batch_parallel", [(b0, b1, 0, num_heads) for b0, b1 in uneven(batch_size, g)]


def _kv_shard(shard: Shard, group: int) -> Shard:
    b0, b1, h0, h1 = shard
    return (b0, b1, h0 // group, h1 // group)


def _slice(t: torch.Tensor, shard: Shard) -> torch.Tensor:
    b0, b1, h0, h1 = shard
    return t[b0:b1, :, h0:h1, :]


class FlashAttentionV100Manager:
    """Device discovery, tile lookup and the (batch x heads) shard planner.

    Constructor and attributes follow reference interface.py:36-74
    (enable_multi_gpu auto-detect, .devices, .primary_device,
    .performance_history, .config_cache, .error_recovery_count).  Also a
    context manager, as the reference's README usage (`with manager:`) needs.
    """

    def __init__(self, enable_multi_gpu: Optional[bool] = None,
                 optimization_strategy: str = "balanced", enable_profiling: bool = False):
        self.optimization_strategy = optimization_strategy
        self.enable_profiling = enable_profiling
        cuda = torch.cuda.is_available()
        launcher = "RANK" in os.environ and "WORLD_SIZE" in os.environ
        if enable_multi_gpu is None:
            # one process per GPU under a distributed launcher: the process
            # drives its own device only
            self.enable_multi_gpu = cuda and torch.cuda.device_count() > 1 and not launcher
        else:
            self.enable_multi_gpu = bool(enable_multi_gpu) and cuda
        self.devices = self._get_available_devices()
        self.primary_device = self.devices[0] if self.devices else torch.device("cpu")
        self.performance_history: List[Dict[str, Any]] = []
        self.config_cache: Dict[str, Dict[str, Any]] = {}
        self.error_recovery_count = 0
        self._streams: Dict[int, torch.cuda.Stream] = {}
        log.info("Flash Attention manager: %d device(s), multi-GPU %s, strategy %s, profiling %s",
                 len(self.devices), self.enable_multi_gpu, optimization_strategy, enable_profiling)

    # -- reference interface.py:75-91 -------------------------------------
    def _get_available_devices(self) -> List[torch.device]:
        if not torch.cuda.is_available():
            return [torch.device("cpu")]
        devs = [torch.device(f"cuda:{i}") for i in range(torch.cuda.device_count())
                if torch.cuda.get_device_capability(i)[0] == 10]
        return devs or [torch.device(f"cuda:{i}") for i in range(torch.cuda.device_count())]

    # -- reference interface.py:108-148 -----------------------------------
    def get_optimal_config(self, seq_len_q: int, seq_len_k: int, num_heads: int, head_dim: int,
                           force_recompute: bool = False, dtype: torch.dtype = torch.bfloat16,
                           causal: bool = False) -> Dict[str, Any]:
        key = f"{seq_len_q}_{seq_len_k}_{num_heads}_{head_dim}_{len(self.devices)}_{dtype}_{causal}"
        if not force_recompute and key in self.config_cache:
            return self.config_cache[key]
        n_dev = len(self.devices) if self.enable_multi_gpu else 1
        cfg = get_enhanced_config(max(seq_len_q, seq_len_k), head_dim, n_dev,
                                  self.optimization_strategy, dtype=dtype, causal=causal)
        if self.enable_multi_gpu and len(self.devices) > 1:
            # reference interface.py:170-185
            if num_heads % len(self.devices) == 0:
                cfg["PARALLELIZATION_STRATEGY"] = "head_parallel"
                cfg["HEADS_PER_GPU"] = num_heads // len(self.devices)
            else:
                cfg["PARALLELIZATION_STRATEGY"] = "batch_parallel"
        self.config_cache[key] = cfg
        return cfg

    def plan_shards(self, batch_size: int, num_heads: int, num_heads_kv: Optional[int] = None,
                    num_parts: Optional[int] = None) -> Tuple[str, List[Shard]]:
        return plan_shards(batch_size, num_heads, num_parts or len(self.devices), num_heads_kv)

    def stream(self, device: torch.device) -> "torch.cuda.Stream":
        idx = device.index
        if idx not in self._streams:
            self._streams[idx] = torch.cuda.Stream(device=device)
        return self._streams[idx]

    def __enter__(self):
        global _global_manager
        self._previous_manager = _global_manager
        _global_manager = self
        return self

    def __exit__(self, *exc):
        global _global_manager
        _global_manager = self._previous_manager
        return False

    # -- one process per GPU (torch.distributed) ---------------------------
    # Attention over (b, h) has no exchange step, so the only communication is
    # moving shards: scatter q/k/v (and dO) from a source rank, gather O/LSE
    # (and dQ/dK/dV) back.  The reference does 3 all_gathers forward and 3
    # full-size all_reduces backward (ops/attention.py:380-382,
    # kernels/backward_kernel.py:395-398).
    @staticmethod
    def scatter_shards(full: Optional[torch.Tensor], shards: Sequence[Shard], like: torch.Tensor,
                       src: int = 0, group=None, lse: bool = False) -> torch.Tensor:
        """Rank `src` holds `full`; every rank gets its shard, packed contiguous.
        `like` supplies dtype/device; for lse=True the tensor is (B, H, N)."""
        rank = dist.get_rank(group)
        b0, b1, h0, h1 = shards[rank]
        if lse:
            shape = (b1 - b0, h1 - h0, like.shape[-1])
        else:
            shape = (b1 - b0, like.shape[1], h1 - h0, like.shape[3])
        out = torch.empty(shape, dtype=like.dtype, device=like.device)
        pieces = None
        if rank == src:
            pieces = [(full[s[0]:s[1], s[2]:s[3]] if lse else _slice(full, s)).contiguous() for s in shards]
        _scatter_uneven(out, pieces, src, group)
        return out

    @staticmethod
    def gather_shards(local: torch.Tensor, shards: Sequence[Shard], full_shape: Sequence[int],
                      dst: int = 0, group=None, lse: bool = False) -> Optional[torch.Tensor]:
        """Inverse of scatter_shards; returns the full tensor on `dst`, None elsewhere."""
        rank = dist.get_rank(group)
        pieces = None
        if rank == dst:
            pieces = []
            for b0, b1, h0, h1 in shards:
                shape = (b1 - b0, h1 - h0, full_shape[-1]) if lse else (b1 - b0, full_shape[1], h1 - h0, full_shape[3])
                pieces.append(torch.empty(shape, dtype=local.dtype, device=local.device))
        _gather_uneven(local.contiguous(), pieces, dst, group)
        if rank != dst:
            return None
        full = torch.empty(tuple(full_shape), dtype=local.dtype, device=local.device)
        for s, piece in zip(shards, pieces):
            if lse:
                full[s[0]:s[1], s[2]:s[3]] = piece
            else:
                _slice(full, s).copy_(piece)
        return full


def _scatter_uneven(out, pieces, src, group):
    """dist.scatter needs equal sizes; shards may differ, so use point-to-point."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if rank == src:
        reqs = []
        for r in range(world):
            if r == src:
                out.copy_(pieces[r])
            elif pieces[r].numel():
                reqs.append(dist.isend(pieces[r], dst=r, group=group))
        for q in reqs:
            q.wait()
    elif out.numel():
        dist.recv(out, src=src, group=group)


def _gather_uneven(local, pieces, dst, group):
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if rank == dst:
        reqs = []
        for r in range(world):
            if r == dst:
                pieces[r].copy_(local)
            elif pieces[r].numel():
                reqs.append(dist.irecv(pieces[r], src=r, group=group))
        for q in reqs:
            q.wait()
    elif local.numel():
        dist.send(local, dst=dst, group=group)


_global_manager: Optional[FlashAttentionV100Manager] = None


def get_flash_attention_manager(**kwargs) -> FlashAttentionV100Manager:
    """Global manager instance (reference interface.py:188-196: created on first
    use; later kwargs do not replace it)."""
    global _global_manager
    if _global_manager is None:
        _global_manager = FlashAttentionV100Manager(**kwargs)
    return _global_manager


def flash_attention_v100(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    causal: bool = False,
    scale: Optional[float] = None,
    dropout_p: float = 0.0,
    bias: Optional[torch.Tensor] = None,
    block_size_m: Optional[int] = None,
    block_size_n: Optional[int] = None,
    enable_autotuning: bool = True,
    return_softmax_lse: bool = False,
    optimization_strategy: str = "balanced",
    enable_multi_gpu: Optional[bool] = None,
    enable_profiling: bool = False,
    fallback_on_error: bool = True,
    validate_inputs: bool = True,
    key_lengths: Optional[torch.Tensor] = None,
    causal_alignment: str = "top_left",
    dropout_origin: Optional[Tuple[int, int, int]] = None,
    dropout_stream: Optional[Tuple[int, int]] = None,
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """Exact attention on (B, N, H, D) tensors; signature of reference interface.py:199-217.

    Args:
        q: [batch, seq_len_q, num_heads, head_dim]; k, v: [batch, seq_len_k, num_heads_kv, head_dim]
        causal: key j is visible to query i iff j <= i
        scale: defaults to 1/sqrt(head_dim)
        dropout_p: drop probability of the attention weights (quantised to 1/256)
        bias: additive score bias, (B|1, H|1, Nq|1, Nk): scores = scale * q.k + bias before the causal mask;
            -inf entries mask keys.  Served by the CUDA-core kernels; its gradient is returned
        key_lengths: (not in the reference) int tensor (B,): batch entry b attends to its first
            key_lengths[b] keys only (right-padded batches); key blocks beyond are skipped on every
            kernel family, dK / dV of the padding are zero
        causal_alignment: (not in the reference) "top_left" (the reference's mask: key j visible to
            query i iff j <= i) or "bottom_right" (j <= i + Nk - Nq: the last query sees every key;
            needs Nk >= Nq); the same for Nq == Nk
        dropout_origin, dropout_stream: (not in the reference) for a call that is one shard of a larger
            problem, e.g. a rank that received its shard from `scatter_shards`: the shard's (batch offset,
            head offset, heads of the whole problem) and the whole problem's (seed, offset).  The shard
            then draws exactly the dropout mask the whole call would draw for its columns
        block_size_m, block_size_n, enable_autotuning:
            accepted for source compatibility; tiles come from the static table
        optimization_strategy: "speed" lets the backward use its fastest kernels even where they sum dQ
            in no fixed order (D = 64: one kernel for dK, dV and dQ); any other value ("balanced",
            "memory") keeps every gradient bit-reproducible
        return_softmax_lse: also return the (B, H, Nq) fp32 log-sum-exp
        enable_multi_gpu: shard (batch x heads) over the visible GPUs (auto if None)
        enable_profiling: record CUDA-event timings in manager.performance_history
        fallback_on_error: accepted; there is no PyTorch/CPU fallback, errors raise
        validate_inputs: run the shape/dtype/device checks (always O(1), no tensor scans)

    Returns: O [batch, seq_len_q, num_heads, head_dim], or (O, LSE).
    """
    manager = get_flash_attention_manager(enable_multi_gpu=enable_multi_gpu,
                                          optimization_strategy=optimization_strategy,
                                          enable_profiling=enable_profiling)
    if validate_inputs:
        q, k, v, scale = _validate_inputs(q, k, v, scale, bias, dropout_p)
    elif scale is None:
        scale = q.shape[-1] ** -0.5

    shift = _causal_shift(causal, causal_alignment, q.shape[1], k.shape[1], key_lengths)
    use_multi = manager.enable_multi_gpu if enable_multi_gpu is None else (
        bool(enable_multi_gpu) and torch.cuda.is_available())
    profile = manager.enable_profiling or enable_profiling
    if profile:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(torch.cuda.current_stream(q.device))

    if use_multi and len(manager.devices) > 1:
        result = _execute_multi_gpu(q, k, v, scale, causal, dropout_p, bias, block_size_m, block_size_n,
                                    enable_autotuning, return_softmax_lse, manager, key_lengths, shift,
                                    dropout_origin, dropout_stream)
    else:
        result = FlashAttentionV100Function.apply(q, k, v, scale, causal, dropout_p, bias, block_size_m,
                                                  block_size_n, enable_autotuning, return_softmax_lse,
                                                  False, True, None, True, optimization_strategy, False, 1, 0,
                                                  key_lengths, shift, dropout_origin, dropout_stream)
    if profile:
        end.record(torch.cuda.current_stream(q.device))
        end.synchronize()
        _record_performance(manager, start.elapsed_time(end), q.shape, k.shape[1], causal)
    return result


def _causal_shift(causal, alignment: str, seq_q: int, seq_k: int, key_lengths) -> int:
    """Offset of the causal mask's diagonal: key j is visible to query i iff j <= i + shift.
    "top_left" (the reference: kernels/forward_kernel.py:179-182 masks row >= col) is 0;
    "bottom_right" lets the last query see every key, shift = Nk - Nq (decoding and chunked prefill
    against a longer key/value cache)."""
    if alignment not in ("top_left", "bottom_right"):
        raise ValueError('causal_alignment must be "top_left" or "bottom_right"')
    if not causal or alignment == "top_left":
        return 0
    if seq_k < seq_q:
        raise ValueError(f"bottom-right causal alignment needs Nk >= Nq (got Nq={seq_q}, Nk={seq_k}): "
                         "the first queries would see no key")
    if key_lengths is not None:
        raise ValueError("bottom-right causal alignment is defined by the tensors' lengths: it cannot be "
                         "combined with key_lengths")
    return seq_k - seq_q


def _execute_multi_gpu(q, k, v, scale, causal, dropout_p, bias, block_size_m, block_size_n,
                       enable_autotuning, return_softmax_lse, manager, key_lengths=None, causal_shift=0,
                       dropout_origin=None, dropout_stream=None):
    """Single-process sharding over manager.devices (reference interface.py:351-434).

    Shards are planned over heads or batch; each device gets its slice by an
    asynchronous peer copy on its own stream, runs the same op independently,
    and the pieces are gathered on the input's device.  All steps are
    differentiable torch ops around the autograd Function, so backward runs the
    same way in reverse.  Unlike the reference there is no global
    torch.cuda.synchronize(): ordering is by stream events.

    Dropout: one (seed, offset) is drawn for the whole call and every shard indexes the stream by its
    columns' place in the whole problem, so the mask does not depend on how the call was split.
    """
    from .ops.attention import next_dropout_stream
    if dropout_p > 0.0 and dropout_stream is None:
        dropout_stream = next_dropout_stream()
    b_base, h_base, h_total = dropout_origin if dropout_origin is not None else (0, 0, q.shape[2])
    devices = manager.devices
    group = q.shape[2] // k.shape[2]
    _, shards = manager.plan_shards(q.shape[0], q.shape[2], k.shape[2], len(devices))
    home = q.device
    home_stream = torch.cuda.current_stream(home)
    ready = torch.cuda.Event()
    ready.record(home_stream)
    outs, lses, done = [], [], []
    for dev, shard in zip(devices, shards):
        if shard[0] == shard[1] or shard[2] == shard[3]:
            continue
        kv_shard = _kv_shard(shard, group)
        st = manager.stream(dev) if dev != home else home_stream
        with torch.cuda.device(dev), torch.cuda.stream(st):
            st.wait_event(ready)
            ql = _slice(q, shard).to(dev, non_blocking=True)
            kl = _slice(k, kv_shard).to(dev, non_blocking=True)
            vl = _slice(v, kv_shard).to(dev, non_blocking=True)
            bl = None
            if bias is not None:
                # the shard's part of the bias (broadcast dimensions stay whole)
                bl = bias
                if bl.shape[0] > 1:
                    bl = bl[shard[0]:shard[1]]
                if bl.shape[1] > 1:
                    bl = bl[:, shard[2]:shard[3]]
                bl = bl.to(dev, non_blocking=True)
            ll = key_lengths[shard[0]:shard[1]].to(dev, non_blocking=True) if key_lengths is not None else None
            res = FlashAttentionV100Function.apply(ql, kl, vl, scale, causal, dropout_p, bl, block_size_m,
                                                   block_size_n, enable_autotuning, return_softmax_lse,
                                                   False, True, None, True, manager.optimization_strategy, False, 1, 0, ll, causal_shift,
                                                   (b_base + shard[0], h_base + shard[2], h_total), dropout_stream)
            o_l, lse_l = res if return_softmax_lse else (res, None)
            outs.append((shard, o_l.to(home, non_blocking=True)))
            if lse_l is not None:
                lses.append((shard, lse_l.to(home, non_blocking=True)))
            ev = torch.cuda.Event()
            ev.record(st)
            done.append(ev)
    for ev in done:
        home_stream.wait_event(ev)
    head_split = len({(s[0], s[1]) for s, _ in outs}) == 1
    out = torch.cat([t for _, t in outs], dim=2 if head_split else 0)
    if return_softmax_lse:
        lse = torch.cat([t for _, t in lses], dim=1 if head_split else 0)
        return out, lse
    return out


def _record_performance(manager, elapsed_ms, q_shape, seq_len_k, causal):
    """Reference interface.py:576-608, with device-timed milliseconds and the
    attention FLOP count 4*B*H*Nq*Nk*D (halved when causal)."""
    b, nq, h, d = q_shape
    flops = 4.0 * b * h * nq * seq_len_k * d * (0.5 if causal else 1.0)
    manager.performance_history.append({
        "input_shape": tuple(q_shape), "execution_time_ms": elapsed_ms,
        "throughput_tflops": flops / (elapsed_ms * 1e-3) / 1e12 if elapsed_ms > 0 else 0.0,
        "peak_memory_mb": torch.cuda.max_memory_allocated() / 1024 ** 2,
        "success": True, "optimization_strategy": manager.optimization_strategy,
        "num_devices": len(manager.devices),
    })
    if len(manager.performance_history) > 100:
        manager.performance_history = manager.performance_history[-50:]


def flash_attention_v100_causal(q, k, v, **kwargs):
    """Reference interface.py:612-619."""
    return flash_attention_v100(q, k, v, causal=True, **kwargs)


def flash_attention_v100_with_dropout(q, k, v, dropout_p: float, **kwargs):
    """Reference interface.py:622-630."""
    return flash_attention_v100(q, k, v, dropout_p=dropout_p, **kwargs)


def flash_attention_v100_multi_gpu(q, k, v, **kwargs):
    """Reference interface.py:633-640."""
    return flash_attention_v100(q, k, v, enable_multi_gpu=True, **kwargs)


@contextlib.contextmanager
def flash_attention_performance_mode(strategy: str = "speed"):
    """Reference interface.py:644-654: swap in a manager with another strategy."""
    global _global_manager
    old = _global_manager
    try:
        _global_manager = FlashAttentionV100Manager(optimization_strategy=strategy)
        yield
    finally:
        _global_manager = old


@contextlib.contextmanager
def flash_attention_memory_mode():
    """Reference interface.py:657-661."""
    with flash_attention_performance_mode("memory"):
        yield


__all__ = [
    "flash_attention_v100", "flash_attention_v100_causal", "flash_attention_v100_with_dropout",
    "flash_attention_v100_multi_gpu", "FlashAttentionV100Manager", "get_flash_attention_manager",
    "flash_attention_performance_mode", "flash_attention_memory_mode", "plan_shards",
]
