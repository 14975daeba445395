"""ctypes front-end of the CPU oracle ``librosa_oracle.so``.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  Nothing under ``rosa_soft_b200/`` imports it.

All array arguments are numpy arrays; floating inputs are float32 views of the
operator's input dtype (bf16/fp16 values are exactly representable), outputs of
the VJP are float64.  Shapes use the packed layout ``[N, H, D]`` with
``cu_seqlens``; a dense ``[B, T, H, D]`` call is ``N = B*T`` with uniform offsets
(the reference's varlen oracle is defined as exactly that loop,
rosa_soft/soft_reference.py:682-701).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "librosa_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "rosa_oracle.c")
    stale = (
        force
        or not os.path.exists(_LIB_PATH)
        or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    )
    if stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "librosa_oracle.so"])
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_hash_counter.restype = ctypes.c_uint32
        _lib.oracle_hash_counter.argtypes = [ctypes.c_uint32]
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct)) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _offsets(cu_seqlens, n_tokens, batch=None):
    if cu_seqlens is None:
        seq = n_tokens // batch
        cu_seqlens = np.arange(batch + 1, dtype=np.int64) * seq
    cu = np.ascontiguousarray(cu_seqlens, dtype=np.int64)
    assert cu[0] == 0 and cu[-1] == n_tokens and np.all(np.diff(cu) >= 0)
    return cu


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following oracle calls (launchers may have exported OMP_NUM_THREADS=1)."""
    _load().oracle_set_num_threads(ctypes.c_int(int(n)))


def hash_counter(x: int) -> int:
    return int(_load().oracle_hash_counter(ctypes.c_uint32(x & 0xFFFFFFFF)))


def pack_symbols(x: np.ndarray) -> np.ndarray:
    """[..., D] logits -> [...] uint32 symbols (bit d set iff x[..., d] > 0)."""
    x = _f32(x)
    rows = int(np.prod(x.shape[:-1]))
    out = np.empty(x.shape[:-1], dtype=np.uint32)
    _load().oracle_pack_symbols(
        _p(x, ctypes.c_float), ctypes.c_int64(rows), ctypes.c_int(x.shape[-1]), _p(out, ctypes.c_uint32)
    )
    return out


def dropout_keep_mask(batch, batch_offset, heads, queries, routes, seed, p) -> np.ndarray:
    keep = np.empty((batch, heads, queries, routes), dtype=np.uint8)
    _load().oracle_dropout_keep_mask(
        ctypes.c_int(batch), ctypes.c_int(batch_offset), ctypes.c_int(heads), ctypes.c_int(queries),
        ctypes.c_int(routes), ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), ctypes.c_float(p),
        _p(keep, ctypes.c_uint8),
    )
    return keep.astype(bool)


def hard_routes(qsym, ksym, cu_seqlens, max_suffix_length):
    """Packed symbols [N, H] -> (route [N, H] int32 local index, 0 = null; match length)."""
    qsym = np.ascontiguousarray(qsym, dtype=np.uint32)
    ksym = np.ascontiguousarray(ksym, dtype=np.uint32)
    n, h = qsym.shape
    cu = _offsets(cu_seqlens, n)
    route = np.zeros((n, h), dtype=np.int32)
    mlen = np.zeros((n, h), dtype=np.int32)
    _load().oracle_hard_routes(
        _p(qsym, ctypes.c_uint32), _p(ksym, ctypes.c_uint32), _p(cu, ctypes.c_int64),
        ctypes.c_int64(len(cu) - 1), ctypes.c_int(h), ctypes.c_int64(max_suffix_length),
        _p(route, ctypes.c_int32), _p(mlen, ctypes.c_int32),
    )
    return route, mlen


def hard_forward(q, k, v, cu_seqlens, max_suffix_length):
    """q,k [N,H,D], v [N,Hv,Dv] -> (out [N,H,Dv] float32 in {-1,0,1}, route [N,H])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    n, h, d = q.shape
    hv, dv = v.shape[1:]
    cu = _offsets(cu_seqlens, n)
    out = np.empty((n, h, dv), dtype=np.float32)
    route = np.empty((n, h), dtype=np.int32)
    _load().oracle_hard_forward(
        _p(q, ctypes.c_float), _p(k, ctypes.c_float), _p(v, ctypes.c_float), _p(cu, ctypes.c_int64),
        ctypes.c_int64(len(cu) - 1), ctypes.c_int64(n), ctypes.c_int(h), ctypes.c_int(d),
        ctypes.c_int(hv), ctypes.c_int(dv), ctypes.c_int64(max_suffix_length),
        _p(out, ctypes.c_float), _p(route, ctypes.c_int32),
    )
    return out, route


def hard_inference(qsym, ksym, payload, cu_seqlens, max_suffix_length):
    """Packed symbols [N,H] uint32, payload [N,Hp,Dp] -> (out [N,H,Dp], matched_end [N,H] int64)."""
    qsym = np.ascontiguousarray(qsym, dtype=np.uint32)
    ksym = np.ascontiguousarray(ksym, dtype=np.uint32)
    payload = _f32(payload)
    n, h = qsym.shape
    hp, dp = payload.shape[1:]
    cu = _offsets(cu_seqlens, n)
    out = np.empty((n, h, dp), dtype=np.float32)
    end = np.empty((n, h), dtype=np.int64)
    _load().oracle_hard_inference(
        _p(qsym, ctypes.c_uint32), _p(ksym, ctypes.c_uint32), _p(payload, ctypes.c_float),
        _p(cu, ctypes.c_int64), ctypes.c_int64(len(cu) - 1), ctypes.c_int64(n), ctypes.c_int(h),
        ctypes.c_int(hp), ctypes.c_int(dp), ctypes.c_int64(max_suffix_length),
        _p(out, ctypes.c_float), _p(end, ctypes.c_int64),
    )
    return out, end


def surrogate_vjp(q, k, v, grad_out, cu_seqlens, max_suffix_length, scale=1.0, dropout_p=0.0,
                  mismatch_scale=3.0, seed=0, batch_offset=0, mask=7, head_offset=0):
    """Float64 gradients (dq, dk, dv) of the reference's dense surrogate; None where masked off."""
    q, k, v, go = _f32(q), _f32(k), _f32(v), _f32(grad_out)
    n, h, d = q.shape
    hv, dv = v.shape[1:]
    cu = _offsets(cu_seqlens, n)
    dq = np.empty((n, h, d), dtype=np.float64) if mask & 1 else None
    dk = np.empty((n, h, d), dtype=np.float64) if mask & 2 else None
    dvv = np.empty((n, hv, dv), dtype=np.float64) if mask & 4 else None
    _load().oracle_surrogate_vjp(
        _p(q, ctypes.c_float), _p(k, ctypes.c_float), _p(v, ctypes.c_float), _p(go, ctypes.c_float),
        _p(cu, ctypes.c_int64), ctypes.c_int64(len(cu) - 1), ctypes.c_int64(n), ctypes.c_int(h),
        ctypes.c_int(d), ctypes.c_int(hv), ctypes.c_int(dv), ctypes.c_int64(max_suffix_length),
        ctypes.c_double(scale), ctypes.c_double(dropout_p), ctypes.c_double(mismatch_scale),
        ctypes.c_int64(seed), ctypes.c_int64(batch_offset), ctypes.c_int64(head_offset),
        _p(dq, ctypes.c_double), _p(dk, ctypes.c_double), _p(dvv, ctypes.c_double),
    )
    return dq, dk, dvv
