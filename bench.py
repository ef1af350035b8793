"""Benchmark of the attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3]

N > 1 is launched with torch.distributed.run (one rank per GPU).  The workload
is then split over the ranks the way the package's shard planner splits it
(heads when they divide, else batch): the ONE problem, e.g. cfg3's 128
(batch, head) columns as 16 / 8 / 4 heads per GPU at 2 / 4 / 8 GPUs, with every
rank's shard resident on its GPU (strong scaling).  The (batch x heads) grid has
no exchange step, so NCCL is used only for the barrier and the max-over-ranks
reduction of the timings.  Rank 0 prints ONE JSON line.  `--replicas` instead
gives every rank the whole workload (weak scaling).

A step is one forward + backward pass of the workload (default: B4 N4096 H32
D128 bf16 causal, the Llama-7B-like layer) through the public API; the timed
steps replay a CUDA graph of one such step (`--no-graph`: eager).  `value` is
device-resident throughput in TFLOP/s (4*B*H*N^2*D forward, 2.5x that backward,
halved when causal); `e2e` repeats the measurement with the step's inputs
copied from pinned host memory and its results copied back inside the timed
region.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "flash-attn-v100_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "attention_fwd_bwd_tflops"
UNIT = "TFLOP/s"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0


# ----------------------------------------------------------------------------- helpers
class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.12)
            self.proc.terminate()          # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clock, top = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            try:
                watts = float(parts[2])
            except ValueError:
                watts = float("nan")
            if watts < 300.0:        # not under load yet (or no longer); unknown power counts as load
                continue
            sm.append(clock)
            mx.append(top)
            power.append(watts)
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w": statistics.median(power)}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), "measured (cuBLAS bf16 burst, MEASURED_PEAKS.json)", d
    except (OSError, KeyError, ValueError):
        return FALLBACK_BF16_TFLOPS, "fallback (earlier measurement on this pool)", {}


# dram__bytes_read.sum + dram__bytes_write.sum per launch, from an ncu capture of these kernels at batch 1
# of the default workload (32 (batch, head) columns of N4096 D128 bf16 causal), scaled by the number of
# columns: traffic is proportional to it, every column being independent.
NCU_DRAM_BYTES_PER_BATCH = {"fwd": 127.6e6, "bwd_preprocess": 214.8e6, "bwd_dkdv": 202.2e6, "bwd_dq": 157.9e6}


def ncu_traffic(kernel: str, w):
    """DRAM bytes per launch for the default workload's shape family, else None."""
    if (w.N, w.D, w.causal) != (4096, 128, True) or kernel not in NCU_DRAM_BYTES_PER_BATCH:
        return None
    return NCU_DRAM_BYTES_PER_BATCH[kernel] * w.B * w.H / 32.0


def time_steps(fn, steps: int, device, world: int):
    """ms per step of `fn`, CUDA events on the current stream, max over ranks."""
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


# ----------------------------------------------------------------------------- CPU side
def cpu_reference_throughput(w, budget_s: float = 12.0, max_heads: int = 64):
    """The reference's PyTorch math attention path (restated in oracle/) timed on
    this box's host cores, forward + backward through autograd, on a bounded
    sample of (batch, head) columns of the workload.  Returns (TFLOP/s, cores, sample)."""
    from flash_attention_v100.testing import make_inputs
    from oracle import attention_oracle as ao
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    one = w.shrink(B=1, H=1)
    t = make_inputs(one)
    args = [t[n].float() for n in ("q", "k", "v", "d_o")]
    ao.attention_forward_backward(*args, causal=w.causal, scale=w.scale)       # warm-up
    done, t0 = 0, time.perf_counter()
    while done < max_heads and (time.perf_counter() - t0 < budget_s or done == 0):
        ao.attention_forward_backward(*args, causal=w.causal, scale=w.scale)
        done += 1
    elapsed = time.perf_counter() - t0
    flops = (one.fwd_flops() + one.bwd_flops()) * done
    sample = (f"{done} of {w.B * w.H} (batch, head) columns of {w.name}, fp32 math path "
              f"(dense N x N scores), {elapsed:.1f} s")
    return flops / elapsed / 1e12, cores, sample, elapsed / done


def run_reference(args, w):
    """--impl reference: the reference's own CPU implementation of the path.  The
    reference is pure Python (nothing to compile into oracle/_ref) and its tree is
    not present on the GPU box, so the oracle port stands in (kind "port")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ms = []
    value = cores = sample = None
    for _ in range(max(1, min(args.steps, 3))):
        value, cores, sample, per_col = cpu_reference_throughput(w, budget_s=8.0, max_heads=48)
        ms.append(per_col * 1e3 * w.B * w.H)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.median(ms),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": w.name, "parallelism": "host cores only",
                   "note": "ms_per_step extrapolated from the sampled columns to the whole workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------- GPU side
def shard_of(w, world: int, rank: int, replicas: bool):
    """This rank's part of the workload: (local workload, dropout origin, description).  With more
    than one rank the problem is split by the package's planner, heads first, then batch."""
    if world == 1 or replicas:
        return w, None, ("the whole workload" if world == 1 else "replicas: every rank runs the whole workload")
    from flash_attention_v100.interface import plan_shards
    kind, shards = plan_shards(w.B, w.H, world)
    b0, b1, h0, h1 = shards[rank]
    sizes = sorted({(s[1] - s[0], s[3] - s[2]) for s in shards})
    what = "%s: %s (batch, heads) per rank" % (kind, ", ".join("%dx%d" % x for x in sizes))
    local = w.shrink(B=b1 - b0, H=h1 - h0)
    return local, (b0, h0, w.H), what


def bind_to_gpu_numa_node(index: int):
    """Pin this process to the CPUs of the NUMA node its GPU hangs off, before any pinned host
    memory is allocated (first touch then places the buffers on that node).  Returns a description
    of what was done; does nothing when the topology cannot be read."""
    try:
        props = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0:
            return {"numa_node": None, "bound": False}
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "bound": True, "cpus": len(cpus)}
    except (OSError, ValueError, AttributeError):
        return {"numa_node": None, "bound": False}


def run_ours(args, whole):
    import flash_attention_v100 as fa
    from flash_attention_v100.kernels import _cabi
    from flash_attention_v100.ops import attention as ops
    from flash_attention_v100.testing import make_inputs, DROPOUT_SEED, DROPOUT_OFFSET

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    numa = bind_to_gpu_numa_node(local) if world > 1 else {"numa_node": None, "bound": False}
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _cabi.load()

    w, origin, split = shard_of(whole, world, rank, args.replicas)
    host = make_inputs(w, seed=w.seed + rank, pin=True)              # pinned host copies of this rank's shard
    dev = {n: t.to(device, non_blocking=True) for n, t in host.items()}
    torch.cuda.synchronize(device)
    stream = (DROPOUT_SEED, DROPOUT_OFFSET)

    q, k, v = (dev[n].requires_grad_(True) for n in ("q", "k", "v"))

    def step():
        if w.dropout_p > 0:
            fa.set_dropout_seed(*stream)
        o = fa.flash_attention_v100(q, k, v, causal=w.causal, scale=w.scale, dropout_p=w.dropout_p,
                                    enable_multi_gpu=False, dropout_origin=origin, optimization_strategy=args.strategy,
                                    dropout_stream=stream if origin is not None else None)
        o.backward(dev["d_o"])
        q.grad = k.grad = v.grad = None
        return o

    # e2e: the step's inputs start in pinned host memory and its results end there.  The
    # package's host-operand entry point cuts the batch into chunks and overlaps the copies
    # of one chunk with the kernels of another (three streams), as a user with host-resident
    # operands would call it.
    back = {n: torch.empty(host["q"].shape, dtype=w.dtype).pin_memory() for n in ("o", "dq", "dk", "dv")}
    host_step = fa.HostAttentionStep(host["q"].shape, host["k"].shape, w.dtype, device, causal=w.causal,
                                     scale=w.scale, dropout_p=w.dropout_p)

    def step_e2e():
        host_step(host, back, *stream)

    # the same traffic on one stream (copy in, autograd op, copy out), to show what the overlap buys
    stage = {n: torch.empty_like(dev[n]) for n in ("q", "k", "v", "d_o")}

    def step_e2e_serial():
        for n in ("q", "k", "v", "d_o"):
            stage[n].copy_(host[n], non_blocking=True)
        qq, kk, vv = (stage[n].detach().requires_grad_(True) for n in ("q", "k", "v"))
        if w.dropout_p > 0:
            fa.set_dropout_seed(*stream)
        o = fa.flash_attention_v100(qq, kk, vv, causal=w.causal, scale=w.scale, dropout_p=w.dropout_p,
                                    enable_multi_gpu=False)
        o.backward(stage["d_o"])
        for n, t in (("o", o.detach()), ("dq", qq.grad), ("dk", kk.grad), ("dv", vv.grad)):
            back[n].copy_(t, non_blocking=True)

    # The device-resident step is replayed from a CUDA graph of one public-API step (forward + backward
    # through autograd): at 8 GPUs a rank's step is 0.33 ms of kernels, and eight Python processes on one
    # host's cores cannot issue the launches and allocations of an eager step that fast (0.386 ms eager).
    eager_step, launch = step, "eager"
    for _ in range(max(3, args.warmup)):
        step()
    if not args.no_graph:
        try:
            torch.cuda.synchronize(device)
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                eager_step()
            torch.cuda.current_stream(device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            # thread_local: a CUDA call by another thread of the process (NCCL's watchdog polls events)
            # must not invalidate the capture; the step's own launches, the autograd thread's
            # included, go to the capturing stream either way
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                eager_step()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(device)
            step, launch = graph.replay, "CUDA graph of one step through the public API, replayed"
        except Exception as exc:                      # time eager steps and say so in the line
            print(f"bench: graph capture failed ({exc!r}); timing eager steps", file=sys.stderr)
            launch = f"eager (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize(device)
    with ClockSampler(local) as clocks:
        ms_step = time_steps(step, args.steps, device, world)
        # nvidia-smi takes ~100 ms to start and then samples every 50 ms: keep the same load on the GPU
        # (untimed) until the sampler has seen about half a second of it
        for _ in range(int(500.0 / max(ms_step, 0.05)) + 1):
            step()
        torch.cuda.synchronize(device)
    clock_info = clocks.summary()
    for _ in range(2):
        step_e2e()
    ms_e2e = time_steps(step_e2e, max(3, args.steps // 2), device, world)
    step_e2e_serial()
    ms_e2e_serial = time_steps(step_e2e_serial, 3, device, world)

    # per-kernel timing, each launch alone (live CUDA events), for the roofline
    with torch.no_grad():
        o, lse = ops.launch_forward(dev["q"], dev["k"], dev["v"], w.scale, w.causal, w.dropout_p, *stream)
    p = ops._base_params(dev["q"].detach(), dev["k"].detach(), dev["v"].detach(), o, lse, w.scale, w.causal,
                         w.dropout_p, *stream)
    grads = [torch.empty_like(dev[n]) for n in ("q", "k", "v")]
    p.d_o = ops._tensor4(dev["d_o"])
    p.dq, p.dk, p.dv = (ops._tensor4(g) for g in grads)
    lib = _cabi.load()
    if args.strategy == "speed":
        p.variant = _cabi.VARIANT_TCGEN05
    nbytes = int(lib.fa_b200_bwd_workspace_bytes(ctypes.byref(p)))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), nbytes
    # dropout: the keep bits are written once (by the forward) and read by all three kernels
    nbits = int(lib.fa_b200_dropout_bits_bytes(ctypes.byref(p)))
    bits = torch.empty(max(nbits, 16), dtype=torch.uint8, device=device)
    if nbits:
        p.dropout_bits, p.dropout_bits_bytes = bits.data_ptr(), nbits

    def call(fn, phases):
        def run():
            p.bwd_phases = phases
            rc = fn(ctypes.byref(p))
            if rc != 0:
                _cabi.raise_for_status(rc, "bench")
        return run

    call(lib.fa_b200_fwd, 0)()         # fills the keep bits (dropout_bits_ready = 0)
    call(lib.fa_b200_bwd, 0)()
    ksteps = max(5, args.steps)
    fwd_and_bits_ms = time_steps(call(lib.fa_b200_fwd, 0), ksteps, device, world) if nbits else None
    p.dropout_bits_ready = 1
    # --strategy speed at D = 64 in fp16/bf16 takes the one-kernel backward: phase 2 is the kernel that
    # produces dK, dV and the fp32 dQ sums (5 GEMMs), phase 4 the conversion of the sums to dQ; the
    # default is the deterministic two-pass form at every size
    one_kernel = (args.strategy == "speed" and w.D == 64 and w.dtype in (torch.float16, torch.bfloat16))
    k2, k4 = ("bwd_dkdvdq", "bwd_dq_convert") if one_kernel else ("bwd_dkdv", "bwd_dq")
    kern_ms = {
        "fwd": time_steps(call(lib.fa_b200_fwd, 0), ksteps, device, world),
        "bwd_preprocess": time_steps(call(lib.fa_b200_bwd, 1), ksteps, device, world),
        k2: time_steps(call(lib.fa_b200_bwd, 2), ksteps, device, world),
        k4: time_steps(call(lib.fa_b200_bwd, 4), ksteps, device, world),
    }
    if nbits:
        kern_ms["dropout_bits"] = max(0.0, fwd_and_bits_ms - kern_ms["fwd"])     # its own launch before the forward
    p.bwd_phases = 0
    status = ops._status_word(device)

    unit_gemm = w.fwd_flops() / 2.0            # one N x N x D GEMM over the workload (causal-halved)
    kernels = {
        # name: (ms, GEMMs counted by the metric's FLOP formula, GEMMs the kernel executes)
        "fwd": (kern_ms["fwd"], 2, 2),
    }
    if one_kernel:
        kernels[k2] = (kern_ms[k2], 5, 5)
    else:
        kernels[k2] = (kern_ms[k2], 4, 4)
        kernels[k4] = (kern_ms[k4], 1, 3)       # S and dP are recomputed here: executed, not counted
    peak, peak_kind, peaks_file = measured_peak()
    dom = max(kernels, key=lambda n: kernels[n][0])
    dom_ms, dom_alg, dom_exec = kernels[dom]
    achieved = dom_alg * unit_gemm / (dom_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "peak_kind": peak_kind, "frac_of_nominal_2250": achieved / NOMINAL_BF16_TFLOPS,
        "executed_tflops": dom_exec * unit_gemm / (dom_ms * 1e-3) / 1e12,
        "traffic": ncu_traffic(dom, w),
        "per_kernel_ms": kern_ms,
        "per_kernel_tflops_counted": {n: a * unit_gemm / (ms * 1e-3) / 1e12 for n, (ms, a, _) in kernels.items()},
    }

    # strong scaling: the ranks together ran the one workload; replicas: each ran all of it
    total_flops = (whole.fwd_flops() + whole.bwd_flops()) * (world if args.replicas else 1)
    value = total_flops / (ms_step * 1e-3) / 1e12
    host_gbs_rank = (host_step.h2d_bytes + host_step.d2h_bytes) / (ms_e2e * 1e-3) / 1e9   # both directions
    host_gbs = torch.tensor([host_gbs_rank], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(host_gbs, op=dist.ReduceOp.SUM)
    bound = torch.tensor([1.0 if numa.get("bound") else 0.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(bound, op=dist.ReduceOp.SUM)
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e12
    tb = w.tensor_bytes()
    fwd_tf = w.fwd_flops() / (kern_ms["fwd"] * 1e-3) / 1e12
    bwd_ms = kern_ms["bwd_preprocess"] + kern_ms[k2] + kern_ms[k4]
    bwd_tf = w.bwd_flops() / (bwd_ms * 1e-3) / 1e12

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v_cpu, cores, sample, _ = cpu_reference_throughput(w)
        cpu = {"value": v_cpu, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak" if (args.replicas and world > 1) else "strong", "vs_baseline": None,
            "dtype": {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[w.dtype],
            "data": "synthetic",
            "config": {
                "workload": whole.name, "B": whole.B, "N": whole.N, "H": whole.H, "D": whole.D,
                "causal": whole.causal, "dropout_p": whole.dropout_p, "optimization_strategy": args.strategy,
                "launch": launch, "split": split, "per_gpu": "B%d H%d of the workload, resident on the GPU" % (w.B, w.H),
                "parallelism": f"(batch x heads) shards, {world} rank(s), no data-path collective",
                "l2": ("not flushed: q, k, v, o, dO, dQ, dK, dV are %.0f MB each (working set %.0f MB), %s the 126 MB L2"
                       % (tb / 1e6, 8 * tb / 1e6, "larger than" if tb > 126 * 2 ** 20 else
                          ("working set larger than" if 8 * tb > 126 * 2 ** 20 else "SMALLER than: L2-resident run,"))),
            },
            "per_gpu_tflops": value / world,
            "frac_of_nominal_bf16_peak": value / world / NOMINAL_BF16_TFLOPS,
            "frac_of_measured_bf16_peak": value / world / peak,
            "fwd_tflops": fwd_tf, "bwd_tflops": bwd_tf,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": host_step.h2d_bytes, "d2h_bytes_per_step": host_step.d2h_bytes,
                    "api": "HostAttentionStep: %d (batch, head-group) chunks, copies and kernels on three streams"
                           % len(host_step.chunks),
                    "single_stream_ms_per_step": ms_e2e_serial,
                    "host_gbs_per_rank": host_gbs_rank, "host_gbs_all_ranks": float(host_gbs.item()),
                    "ranks_bound_to_gpu_numa_node": int(bound.item())},
            # per step: 1 forward + 3 backward kernels of this library (+ 1 that writes the dropout bits)
            "gpu_launches": (5 if nbits else 4) * args.steps,
            "clocks": clock_info,
            "status_word": int(status[0]),
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--strategy", choices=("balanced", "speed"), default="balanced",
                    help="optimization_strategy of the public entry: 'speed' allows the backward whose dQ is not bit-reproducible")
    ap.add_argument("--replicas", action="store_true",
                    help="N > 1: every rank runs the whole workload (weak scaling) instead of its shard of it")
    ap.add_argument("--batch", type=int, default=None, help="override the workload's batch (small profiling cases)")
    ap.add_argument("--heads", type=int, default=None, help="override the workload's head count")
    ap.add_argument("--dtype", choices=("fp16", "bf16"), default=None, help="override the workload's dtype (A/B runs)")
    ap.add_argument("--no-graph", action="store_true", help="time eager steps instead of replaying a CUDA graph of one")
    ap.add_argument("--dropout-p", type=float, default=None, help="override the workload's dropout rate (A/B runs)")
    args = ap.parse_args()
    from flash_attention_v100.testing import WORKLOADS
    w = WORKLOADS[args.workload]
    if args.batch is not None or args.heads is not None:
        b, h = args.batch or w.B, args.heads or w.H
        w = w.shrink(B=b, H=h, name=f"{w.name} [reduced to B{b} H{h}: not the benchmark size]")
    if args.dtype is not None:
        dt = {"fp16": torch.float16, "bf16": torch.bfloat16}[args.dtype]
        if dt != w.dtype:
            w = w.shrink(dtype=dt, name=f"{w.name} [dtype overridden to {args.dtype}: not the benchmark dtype]")
    if args.dropout_p is not None and args.dropout_p != w.dropout_p:
        w = w.shrink(dropout_p=args.dropout_p,
                     name=f"{w.name} [dropout overridden to {args.dropout_p}: not the benchmark's rate]")
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
