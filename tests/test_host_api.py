"""C-ABI surface and host logic that need no GPU."""
import ctypes
import inspect
import os
import re

import pytest
import torch

import flash_attention_v100 as fa
from flash_attention_v100.kernels import _cabi, tile_table
from flash_attention_v100.ops import memory

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    names = _declared_symbols()
    assert "fa_b200_fwd" in names and "fa_b200_bwd" in names
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_cabi.EXPORTS)


def test_params_struct_size_is_accepted():
    lib = _cabi.load()
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = 2, 128, 128, 4, 4, 64
    p.dtype = _cabi.FA_B200_BF16
    assert lib.fa_b200_bwd_workspace_bytes(ctypes.byref(p)) >= 2 * 4 * 128 * 4
    p.struct_bytes = 8
    assert lib.fa_b200_bwd_workspace_bytes(ctypes.byref(p)) == 0
    assert lib.fa_b200_fwd(ctypes.byref(p)) == _cabi.FA_EINVAL
    assert b"struct_bytes" in lib.fa_b200_last_error()


@pytest.mark.parametrize("field,value,code", [
    ("H", 0, _cabi.FA_EINVAL), ("Hkv", 3, _cabi.FA_EINVAL), ("dtype", 7, _cabi.FA_EINVAL),
    ("dropout_p", 1.0, _cabi.FA_EINVAL), ("dropout_p", -0.1, _cabi.FA_EINVAL),
    ("variant", 9, _cabi.FA_EINVAL), ("scale", float("nan"), _cabi.FA_EINVAL),
])
def test_bad_arguments_are_refused_before_any_cuda_call(field, value, code):
    lib = _cabi.load()
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = 1, 16, 16, 4, 4, 64
    p.scale = 0.125
    setattr(p, field, value)
    assert lib.fa_b200_fwd(ctypes.byref(p)) == code
    assert lib.fa_b200_bwd(ctypes.byref(p)) == code


def test_null_pointers_are_refused():
    lib = _cabi.load()
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = 1, 16, 16, 4, 4, 64
    p.scale = 0.125
    assert lib.fa_b200_fwd(ctypes.byref(p)) == _cabi.FA_EINVAL
    assert b"null" in lib.fa_b200_last_error()
    with pytest.raises(ValueError):
        _cabi.raise_for_status(_cabi.FA_EINVAL, "x")
    with pytest.raises(RuntimeError):
        _cabi.raise_for_status(_cabi.FA_ECUDA, "x")


def test_empty_problem_is_ok_without_pointers():
    lib = _cabi.load()
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = 0, 16, 16, 4, 4, 64
    assert lib.fa_b200_fwd(ctypes.byref(p)) == _cabi.FA_OK


def test_strerror_covers_all_codes():
    lib = _cabi.load()
    seen = {lib.fa_b200_strerror(c) for c in range(0, -7, -1)}
    assert len(seen) == 7 and b"unknown status" not in seen


def test_tile_table_keys_and_families():
    cfg = fa.get_enhanced_config(4096, 128, dtype=torch.bfloat16, causal=True)
    for key in ("BLOCK_M", "BLOCK_N", "BLOCK_K", "NUM_STAGES", "NUM_WARPS"):   # reference config.py:288-348
        assert key in cfg
    assert cfg["BLOCK_K"] == 128 and cfg["VARIANT"] == "tcgen05_2pass"     # what AUTO runs: the deterministic form
    assert tile_table.lookup(64, torch.float32)["VARIANT"] == "simt"
    assert tile_table.lookup(96, torch.float16)["VARIANT"] == "simt"
    with pytest.raises(ValueError):
        tile_table.lookup(256, torch.float16)
    cfg8 = fa.get_enhanced_config(4096, 128, 8)
    assert cfg8["ENABLE_MULTI_GPU"] and cfg8["PARALLELIZATION_STRATEGY"] == "head_parallel"


def test_workspace_estimates():
    n = memory.backward_workspace_bytes(4, 4096, 4096, 32, 128, torch.bfloat16)
    assert n >= 4 * 32 * 4096 * 4
    est = memory.estimate_peak_memory_usage(4, 4096, 4096, 32, 128, torch.bfloat16)
    assert est["total_memory_mb"] > 8 * 128          # eight 134 MB tensors at least
    assert est["total_memory_mb"] < 4 * 32 * 4096 * 4096 * 2 / 2 ** 20   # far below the N^2 scores
    # dropout on the tensor-core kernels: the call's keep bits, two bits of storage per score
    bits = memory.dropout_bits_bytes(32, 2048, 2048, 16, 64, torch.bfloat16, 0.1)
    assert bits == 32 * 16 * 2048 * 2048 // 4
    assert memory.dropout_bits_bytes(32, 2048, 2048, 16, 64, torch.bfloat16, 0.0) == 0
    assert memory.dropout_bits_bytes(2, 200, 333, 4, 64, torch.float16, 0.5, num_heads_kv=2) == 2 * 4 * 256 * 384 // 4
    assert memory.dropout_bits_bytes(2, 256, 256, 4, 64, torch.float32, 0.5) == 0      # CUDA-core kernels
    with_p = memory.estimate_peak_memory_usage(32, 2048, 2048, 16, 64, torch.bfloat16, dropout_p=0.1)
    assert abs(with_p["dropout_bits_memory_mb"] - bits / 2 ** 20) < 1e-6


def test_tile_table_reports_the_constants_the_kernels_are_compiled_from():
    """The lookup and the kernels read one header (csrc/tile_config.cuh).  The header's numbers are
    parsed here as text and compared with what the library reports; the kernel sources are checked to
    take their stage counts, register split and warp counts from the header and not from literals."""
    import re
    csrc = os.path.join(ROOT, "flash-attn-v100_b200", "csrc")
    hdr = open(os.path.join(csrc, "tile_config.cuh")).read()

    def const(name):
        return int(re.search(r"constexpr \w+ %s = ([0-9]+)" % name, hdr).group(1))

    def fn(name):      # constexpr int f(...) { return <expr>; } evaluated with Python's ternary
        body = re.search(r"constexpr int %s\(([^)]*)\) \{ return (.*?); \}" % name, hdr)
        args = [a.split()[-1] for a in body.group(1).split(",")]
        expr = re.sub(r"(\S+) == (\d+) \? (\d+) : ", r"\3 if \1 == \2 else ", body.group(2))
        expr = re.sub(r"\((\w+) \? (\d+) : (\d+)\)", r"(\2 if \1 else \3)", expr)
        return lambda *v: eval(expr, dict(zip(args, v)))

    fwd_stages, u_stages, w_stages = fn("fwd_kv_stages"), fn("bwd_u_stages"), fn("bwd_w_stages")
    for D in (64, 128):
        for dt in (torch.float16, torch.bfloat16):
            for causal in (False, True):
                f = tile_table.lookup(D, dt, causal, False)
                b = tile_table.lookup(D, dt, causal, True)
                assert (f["BLOCK_M"], f["BLOCK_N"]) == (const("kBlockM"), const("kBlockN"))
                assert f["NUM_STAGES"] == fwd_stages(D) and f["NUM_WARPS"] == const("kFwdWarps")
                assert f["Q_TILES_PER_CTA"] == const("kFwdQTilesPerCta")
                assert (f["REGS_SOFTMAX"], f["REGS_OTHER"]) == (const("kFwdRegsSoftmax"), const("kFwdRegsOther"))
                assert b["NUM_STAGES"] == u_stages(D, False) and b["W_STAGES"] == w_stages(D)
                assert b["NUM_WARPS"] == 4 * const("kBwdWarpgroups") + 4
                assert b["ONE_KERNEL_BACKWARD"] == (D == 64)
    assert fwd_stages(128) == 2 and fwd_stages(64) == 4 and u_stages(128, False) == 3 and u_stages(128, True) == 2
    fwd = open(os.path.join(csrc, "fwd_sm100.cu")).read()
    bwd = open(os.path.join(csrc, "bwd_sm100.cu")).read()
    for needle in ("tile::fwd_kv_stages(D)", "tile::kFwdRegsSoftmax", "tile::kFwdWarps", "tile::kFwdHalfSignalAt"):
        assert needle in fwd, needle
    for needle in ("tile::bwd_u_stages(D, kMasks)", "tile::bwd_w_stages(D)", "tile::kBwdWarpgroups",
                   "tile::kBwdOverlapMaxKvBytes", "tile::kBwdGroupBytes"):
        assert needle in bwd, needle


def test_workspace_size_follows_the_backward_variant():
    """Regions (each starts on a 256-byte boundary): the two per-row vectors and the per-column ranges
    (max |dO|, max |V|) for every tensor-core call; for bf16 the row exponents and the fp16 copies of Q,
    dO and K the kernels stream; for the one-kernel backward (D = 64) the fp32 dQ sums instead of the
    copy of K.  fp32 (CUDA-core tiles) needs one vector."""
    lib = _cabi.load()
    B, N, H = 2, 300, 4

    def size(D, dtype, variant):
        p = _cabi.Params()
        p.struct_bytes = ctypes.sizeof(_cabi.Params)
        p.B, p.Nq, p.Nk, p.H, p.Hkv, p.D = B, N, N, H, H, D
        p.dtype, p.scale, p.variant = dtype, 0.125, variant
        return int(lib.fa_b200_bwd_workspace_bytes(ctypes.byref(p)))

    up = lambda n: -(-n // 256) * 256
    rows = B * H * 384 * 4                                # B * H * ceil128(Nq) floats
    ranges = up(B * H * 2 * 4)
    vectors = 2 * rows + ranges

    def tensor(D):
        return up(B * N * H * D * 2)

    bf16, fp16 = tile_table.dtype_enum(torch.bfloat16), tile_table.dtype_enum(torch.float16)
    assert rows % 256 == 0
    assert size(128, fp16, _cabi.VARIANT_AUTO) == vectors
    assert size(64, fp16, _cabi.VARIANT_TCGEN05_2PASS) == vectors
    assert size(64, fp16, _cabi.VARIANT_AUTO) == vectors                  # AUTO is the two-pass form
    assert size(64, fp16, _cabi.VARIANT_TCGEN05) == vectors + rows * 64
    assert size(128, bf16, _cabi.VARIANT_AUTO) == vectors + rows + 3 * tensor(128)
    assert size(64, bf16, _cabi.VARIANT_TCGEN05_2PASS) == vectors + rows + 3 * tensor(64)
    assert size(64, bf16, _cabi.VARIANT_TCGEN05) == vectors + rows + 2 * tensor(64) + rows * 64
    assert size(64, tile_table.dtype_enum(torch.float32), _cabi.VARIANT_AUTO) <= vectors
    assert _cabi.VARIANT_NAMES[_cabi.VARIANT_TCGEN05_2PASS] == "tcgen05_2pass"


def test_dq_reproducibility_table():
    from flash_attention_v100.testing import dq_is_bit_reproducible
    assert dq_is_bit_reproducible("tcgen05_2pass", torch.bfloat16, 64)
    assert dq_is_bit_reproducible("simt", torch.float16, 64)
    assert dq_is_bit_reproducible("auto", torch.bfloat16, 128)
    assert dq_is_bit_reproducible("auto", torch.float32, 64)
    assert dq_is_bit_reproducible("auto", torch.float16, 64)          # the default is deterministic
    assert not dq_is_bit_reproducible("tcgen05", torch.float16, 64)   # the opt-in fast variant is not, at D = 64
    assert not dq_is_bit_reproducible("tcgen05", torch.bfloat16, 64, 0.1)
    assert dq_is_bit_reproducible("tcgen05", torch.bfloat16, 128)


def test_public_signatures_match_the_reference():
    sig = inspect.signature(fa.flash_attention_v100)
    assert list(sig.parameters) == [
        "q", "k", "v", "causal", "scale", "dropout_p", "bias", "block_size_m", "block_size_n",
        "enable_autotuning", "return_softmax_lse", "optimization_strategy", "enable_multi_gpu",
        "enable_profiling", "fallback_on_error", "validate_inputs",     # reference interface.py:199-217
        "key_lengths", "causal_alignment", "dropout_origin", "dropout_stream"]   # this build's additions, last and optional
    assert sig.parameters["causal"].default is False and sig.parameters["dropout_p"].default == 0.0
    fwd = inspect.signature(fa.FlashAttentionV100Function.forward)
    assert list(fwd.parameters)[1:] == [
        "q", "k", "v", "scale", "causal", "dropout_p", "bias", "block_size_m", "block_size_n",
        "enable_autotuning", "return_softmax_lse", "enable_gradient_checkpointing",
        "enable_mixed_precision", "num_checkpoints", "memory_efficient", "performance_mode",
        "enable_multi_gpu", "world_size", "rank",                          # reference ops/attention.py:50-72
        "key_lengths", "causal_shift", "dropout_origin", "dropout_stream"]   # additions, after the reference's 19
    mgr = inspect.signature(fa.FlashAttentionV100Manager.__init__)
    assert list(mgr.parameters)[1:] == ["enable_multi_gpu", "optimization_strategy", "enable_profiling"]
    assert fa.SUPPORTED_DTYPES == {torch.float16, torch.bfloat16, torch.float32}


def test_validation_errors_match_the_reference():
    q = torch.zeros(2, 8, 4, 16)
    with pytest.raises(ValueError, match="4-dimensional"):
        fa.flash_attention_v100(q[0], q, q)
    with pytest.raises(ValueError, match="Batch sizes must match"):
        fa.flash_attention_v100(q, q[:1], q)
    with pytest.raises(ValueError, match="Head dimensions must match"):
        fa.flash_attention_v100(q, q[..., :8], q)
    with pytest.raises(ValueError, match="same dtype"):
        fa.flash_attention_v100(q, q.half(), q)
    with pytest.raises(ValueError, match="Unsupported dtype"):
        fa.flash_attention_v100(q.double(), q.double(), q.double())
    with pytest.raises(ValueError, match="divisible"):
        fa.flash_attention_v100(q, q[:, :, :3], q[:, :, :3])
    with pytest.raises(ValueError, match="dropout_p must be in"):
        fa.utils.validate_inputs(q, q, q, None, None, 1.5, require_cuda=False)
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        fa.flash_attention_v100(q, q, q)      # no CPU path: CPU tensors are refused, not computed
    with pytest.raises(TypeError):
        fa.flash_attention_v100(1, q, q)


def test_manager_is_a_context_manager_and_caches_configs():
    m = fa.FlashAttentionV100Manager(enable_multi_gpu=False)
    with m as mm:
        assert fa.get_flash_attention_manager() is mm
    c1 = m.get_optimal_config(1024, 1024, 8, 64)
    assert m.get_optimal_config(1024, 1024, 8, 64) is c1
    assert m.get_optimal_config(1024, 1024, 8, 64, force_recompute=True) is not c1


def test_causal_shift_of_the_alignments():
    from flash_attention_v100.interface import _causal_shift
    assert _causal_shift(True, "top_left", 10, 50, None) == 0
    assert _causal_shift(True, "bottom_right", 10, 50, None) == 40
    assert _causal_shift(True, "bottom_right", 50, 50, None) == 0
    assert _causal_shift(False, "bottom_right", 50, 10, None) == 0      # no mask: nothing to align
    with pytest.raises(ValueError):
        _causal_shift(True, "bottom_right", 50, 10, None)
    with pytest.raises(ValueError):
        _causal_shift(True, "bottom_right", 10, 50, object())
    with pytest.raises(ValueError):
        _causal_shift(True, "center", 10, 10, None)


def test_combine_operand_checks_need_no_device():
    """launch_combine refuses malformed operands before it touches the library."""
    from flash_attention_v100.ops.attention import launch_combine
    acc = torch.zeros(1, 8, 2, 64)
    part = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="partial, an output"):
        launch_combine(acc)
    with pytest.raises(ValueError, match="fp32"):
        launch_combine(acc.half(), part)
    with pytest.raises(ValueError, match="dense within a batch entry"):
        launch_combine(torch.zeros(1, 8, 2, 128)[..., :64], part)
    with pytest.raises(ValueError, match="same dtype"):
        launch_combine(acc, part, out=torch.zeros(1, 8, 2, 64, dtype=torch.float16))
    with pytest.raises(ValueError, match="lse_acc"):
        launch_combine(acc, part, lse_acc=torch.zeros(1, 8, 2), lse_part=torch.zeros(1, 2, 8))
    with pytest.raises(ValueError, match="lse_part"):
        launch_combine(acc, part, lse_acc=torch.zeros(1, 2, 8), lse_part=torch.zeros(1, 2, 8, dtype=torch.float64))


def test_combine_params_struct_matches_the_header():
    """Field order and size of fa_b200_combine_params as the header declares them (LP64)."""
    header = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "fa_b200.h")).read()
    body = header[header.index("typedef struct fa_b200_combine_params {"):header.index("} fa_b200_combine_params;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = re.findall(r"\b(\w+)(?:, (\w+))?(?:, (\w+))?(?:, (\w+))?;", body)
    declared = [n for group in names for n in group if n]
    assert declared == [f[0] for f in _cabi.CombineParams._fields_]
    assert ctypes.sizeof(_cabi.CombineParams) == 8 + 8 + 8 + 32 + 8 + 32 + 4 * 8 + 8 + 3 * 8
