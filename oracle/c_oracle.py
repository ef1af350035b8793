"""ctypes binding of oracle/cpu_ref.c (double-precision C restatement).

TEST INFRASTRUCTURE: imported only by tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline leg.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libfa_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "cpu_ref.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.fa_oracle_philox4x32_10.restype = None
        _lib.fa_oracle_dropout_mask.restype = None
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t=ctypes.c_float):
    return a.ctypes.data_as(ctypes.POINTER(t))


def forward(q, k, v, causal=False, scale=None, keep=None, dropout_p=0.0, causal_shift=0):
    """q (B,Nq,H,D), k/v (B,Nk,Hkv,D) numpy -> (o, lse) float32."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Nq, H, D = q.shape
    Nk, Hkv = k.shape[1], k.shape[2]
    if scale is None:
        scale = D ** -0.5
    o = np.empty_like(q)
    lse = np.empty((B, H, Nq), np.float32)
    kp = None
    if keep is not None:
        keep = np.ascontiguousarray(keep, dtype=np.uint8)
        kp = _p(keep, ctypes.c_uint8)
    rc = lib().fa_oracle_forward(_p(q), _p(k), _p(v), B, Nq, Nk, H, Hkv, D, (1 + int(causal_shift)) if causal else 0,
                                 ctypes.c_double(scale), kp, ctypes.c_double(dropout_p), _p(o), _p(lse))
    assert rc == 0
    return o, lse


def backward(q, k, v, o, lse, d_o, causal=False, scale=None, keep=None, dropout_p=0.0, causal_shift=0):
    q, k, v, o, lse, d_o = (_f32(t) for t in (q, k, v, o, lse, d_o))
    B, Nq, H, D = q.shape
    Nk, Hkv = k.shape[1], k.shape[2]
    if scale is None:
        scale = D ** -0.5
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    kp = None
    if keep is not None:
        keep = np.ascontiguousarray(keep, dtype=np.uint8)
        kp = _p(keep, ctypes.c_uint8)
    rc = lib().fa_oracle_backward(_p(q), _p(k), _p(v), _p(o), _p(lse), _p(d_o), B, Nq, Nk, H, Hkv, D,
                                  (1 + int(causal_shift)) if causal else 0, ctypes.c_double(scale), kp, ctypes.c_double(dropout_p),
                                  _p(dq), _p(dk), _p(dv))
    assert rc == 0
    return dq, dk, dv


def philox4x32_10(ctr, key):
    c = (ctypes.c_uint32 * 4)(*ctr)
    k = (ctypes.c_uint32 * 2)(*key)
    out = (ctypes.c_uint32 * 4)()
    lib().fa_oracle_philox4x32_10(c, k, out)
    return tuple(out)


def dropout_mask(seed, offset, p, B, H, Nq, Nk):
    out = np.empty((B, H, Nq, Nk), np.uint8)
    lib().fa_oracle_dropout_mask(ctypes.c_uint64(seed), ctypes.c_uint64(offset), ctypes.c_double(p),
                                 B, H, Nq, Nk, _p(out, ctypes.c_uint8))
    return out
