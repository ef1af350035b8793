"""ctypes binding of libfa_b200.so (the C ABI declared in include/fa_b200.h).

The reference launches Triton kernels from Python
(kernels/forward_kernel.py:349-385, kernels/backward_kernel.py:279-316); this
module is the equivalent launch layer for the hand-written sm_100a kernels.
There is no fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_DIR, "lib", "libfa_b200.so")

ABI_VERSION = 3
FA_B200_F16, FA_B200_BF16, FA_B200_F32 = 0, 1, 2
VARIANT_AUTO, VARIANT_SIMT, VARIANT_TCGEN05, VARIANT_TCGEN05_2PASS = 0, 1, 2, 3
VARIANT_NAMES = {VARIANT_AUTO: "auto", VARIANT_SIMT: "simt", VARIANT_TCGEN05: "tcgen05",
                 VARIANT_TCGEN05_2PASS: "tcgen05_2pass"}

FA_OK, FA_EINVAL, FA_EUNSUPPORTED, FA_EALIGN, FA_EWORKSPACE, FA_ECUDA, FA_ETIMEOUT = 0, -1, -2, -3, -4, -5, -6

EXPORTS = (
    "fa_b200_fwd", "fa_b200_bwd", "fa_b200_bwd_static", "fa_b200_bwd_workspace_bytes", "fa_b200_tile_config",
    "fa_b200_dropout_mask_host", "fa_b200_dropout_mask_device", "fa_b200_dropout_effective_p",
    "fa_b200_philox4x32_10", "fa_b200_strerror", "fa_b200_last_error", "fa_b200_version", "fa_b200_combine",
    "fa_b200_copy_rows", "fa_b200_selftest_wait_timeout", "fa_b200_dropout_bits_bytes",
)


class Tensor4(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64),
                ("stride_n", ctypes.c_int64), ("stride_h", ctypes.c_int64)]


class Params(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", ctypes.c_size_t),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
        ("d_o", Tensor4), ("dq", Tensor4), ("dk", Tensor4), ("dv", Tensor4),
        ("lse", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("status_word", ctypes.c_void_p),
        ("stream", ctypes.c_void_p),
        ("seed", ctypes.c_uint64), ("offset", ctypes.c_uint64),
        ("B", ctypes.c_int32), ("Nq", ctypes.c_int32), ("Nk", ctypes.c_int32),
        ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("causal", ctypes.c_int32),
        ("variant", ctypes.c_int32), ("device", ctypes.c_int32),
        ("scale", ctypes.c_float), ("dropout_p", ctypes.c_float),
        ("bwd_phases", ctypes.c_int32), ("causal_shift", ctypes.c_int32),
        ("bias", Tensor4), ("d_scores", ctypes.c_void_p), ("kv_lengths", ctypes.c_void_p),
        ("rng_batch_offset", ctypes.c_int32), ("rng_head_offset", ctypes.c_int32), ("rng_heads", ctypes.c_int32),
        ("wait_limit_ms", ctypes.c_int32),
        ("o_lo", Tensor4),
        ("dropout_bits", ctypes.c_void_p), ("dropout_bits_bytes", ctypes.c_size_t),
        ("dropout_bits_ready", ctypes.c_int32),
    ]


class CombineParams(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", ctypes.c_size_t),
        ("acc", ctypes.c_void_p), ("lse_acc", ctypes.c_void_p),
        ("part", Tensor4), ("lse_part", ctypes.c_void_p), ("out", Tensor4),
        ("B", ctypes.c_int32), ("N", ctypes.c_int32), ("H", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("first", ctypes.c_int32), ("device", ctypes.c_int32),
        ("reserved", ctypes.c_int32), ("stream", ctypes.c_void_p),
        ("acc_stride_b", ctypes.c_int64), ("lse_stride_b", ctypes.c_int64), ("lse_stride_h", ctypes.c_int64),
    ]


class Tile(ctypes.Structure):
    _fields_ = [("variant", ctypes.c_int32), ("block_m", ctypes.c_int32), ("block_n", ctypes.c_int32),
                ("q_tiles_per_cta", ctypes.c_int32), ("kv_stages", ctypes.c_int32),
                ("num_warps", ctypes.c_int32), ("w_stages", ctypes.c_int32), ("regs_softmax", ctypes.c_int32),
                ("regs_other", ctypes.c_int32), ("one_kernel_backward", ctypes.c_int32)]


_lib = None
_lock = threading.Lock()


class FlashAttentionLibraryError(RuntimeError):
    """libfa_b200.so is missing or refuses to load."""


def load():
    """Load the shared library once; raise loudly if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise FlashAttentionLibraryError(
                f"{LIB_PATH} not found: build it with "
                f"`python {os.path.join(os.path.dirname(_PKG_DIR), 'csrc', 'build.py')}` "
                "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name in EXPORTS:
            if not hasattr(lib, name):
                raise FlashAttentionLibraryError(f"{LIB_PATH} does not export {name}")
        pp = ctypes.POINTER(Params)
        lib.fa_b200_fwd.argtypes = [pp]
        lib.fa_b200_fwd.restype = ctypes.c_int
        lib.fa_b200_bwd.argtypes = [pp]
        lib.fa_b200_bwd.restype = ctypes.c_int
        lib.fa_b200_bwd_static.argtypes = [pp]
        lib.fa_b200_bwd_static.restype = ctypes.c_int
        lib.fa_b200_bwd_workspace_bytes.argtypes = [pp]
        lib.fa_b200_bwd_workspace_bytes.restype = ctypes.c_size_t
        lib.fa_b200_dropout_bits_bytes.argtypes = [pp]
        lib.fa_b200_dropout_bits_bytes.restype = ctypes.c_size_t
        lib.fa_b200_combine.argtypes = [ctypes.POINTER(CombineParams)]
        lib.fa_b200_combine.restype = ctypes.c_int
        lib.fa_b200_copy_rows.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t,
                                          ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        lib.fa_b200_copy_rows.restype = ctypes.c_int
        lib.fa_b200_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.fa_b200_selftest_wait_timeout.restype = ctypes.c_int
        lib.fa_b200_tile_config.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(Tile)]
        lib.fa_b200_tile_config.restype = ctypes.c_int
        lib.fa_b200_dropout_mask_host.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float] + \
            [ctypes.c_int] * 4 + [ctypes.c_void_p]
        lib.fa_b200_dropout_mask_host.restype = ctypes.c_int
        lib.fa_b200_dropout_mask_device.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float] + \
            [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.fa_b200_dropout_mask_device.restype = ctypes.c_int
        lib.fa_b200_dropout_effective_p.argtypes = [ctypes.c_float]
        lib.fa_b200_dropout_effective_p.restype = ctypes.c_float
        lib.fa_b200_philox4x32_10.argtypes = [ctypes.POINTER(ctypes.c_uint32)] * 3
        lib.fa_b200_philox4x32_10.restype = None
        lib.fa_b200_strerror.argtypes = [ctypes.c_int]
        lib.fa_b200_strerror.restype = ctypes.c_char_p
        lib.fa_b200_last_error.argtypes = []
        lib.fa_b200_last_error.restype = ctypes.c_char_p
        lib.fa_b200_version.argtypes = []
        lib.fa_b200_version.restype = ctypes.c_int
        if lib.fa_b200_version() != ABI_VERSION:
            raise FlashAttentionLibraryError("ABI version mismatch")
        _lib = lib
    return _lib


def raise_for_status(rc: int, what: str) -> None:
    """Map a fa_b200_status to the exception types the reference API raises."""
    if rc == FA_OK:
        return
    lib = load()
    msg = f"{what}: {lib.fa_b200_strerror(rc).decode()}: {lib.fa_b200_last_error().decode()}"
    if rc in (FA_EINVAL, FA_EUNSUPPORTED, FA_EALIGN):
        raise ValueError(msg)
    raise RuntimeError(msg)


def philox4x32_10(counter, key):
    c = (ctypes.c_uint32 * 4)(*counter)
    k = (ctypes.c_uint32 * 2)(*key)
    out = (ctypes.c_uint32 * 4)()
    load().fa_b200_philox4x32_10(c, k, out)
    return tuple(out)
