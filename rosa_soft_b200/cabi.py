"""ctypes front-end of ``librosa_soft_b200.so`` (the C ABI of include/rosa_soft_b200.h).

This is the binding a non-torch host would write; the test-suite and the benchmark use it to
drive the library with raw device pointers (taken from torch tensors, which only serve as
device memory here).  Loading fails loudly when the shared object is absent.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librosa_soft_b200.so")

F32, F16, BF16 = 0, 1, 2

EXPORTED_SYMBOLS = (
    "rosa_b200_abi_version",
    "rosa_b200_last_error",
    "rosa_b200_hard_forward_workspace_bytes",
    "rosa_b200_hard_forward",
    "rosa_b200_hard_forward_static",
    "rosa_b200_pack_symbols",
    "rosa_b200_hard_forward_packed",
    "rosa_b200_hard_forward_routes",
    "rosa_b200_surrogate_vjp_workspace_bytes",
    "rosa_b200_surrogate_vjp",
    "rosa_b200_hard_inference_workspace_bytes",
    "rosa_b200_hard_inference",
    "rosa_b200_stream_workspace_bytes",
    "rosa_b200_stream_update",
    "rosa_b200_read_status",
    "rosa_b200_decode_status",
    "rosa_b200_profile_enable",
    "rosa_b200_profile_collect",
)

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise OSError(f"{LIB_PATH} not found: run `python rosa_soft_b200/build.py`")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32, f32, sz = (ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                             ctypes.c_size_t)
    lib.rosa_b200_abi_version.restype = i32
    lib.rosa_b200_last_error.restype = ctypes.c_char_p
    lib.rosa_b200_hard_forward_workspace_bytes.restype = sz
    lib.rosa_b200_hard_forward_workspace_bytes.argtypes = [i64, i32, i64]
    lib.rosa_b200_hard_forward.restype = i32
    lib.rosa_b200_hard_forward.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, i32, vp, i64, i64,
                                           i64, vp, vp, vp, vp, vp, sz, vp]
    lib.rosa_b200_hard_forward_static.restype = i32
    lib.rosa_b200_hard_forward_static.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, i32, vp, i64,
                                                  i64, i64, vp, vp, vp, vp, vp]
    lib.rosa_b200_pack_symbols.restype = i32
    lib.rosa_b200_pack_symbols.argtypes = [vp, i32, i64, i32, i32, i64, i64, vp, vp]
    lib.rosa_b200_hard_forward_packed.restype = i32
    lib.rosa_b200_hard_forward_packed.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, i32, vp, i64,
                                                  i64, i64, vp, vp, vp, sz, vp]
    lib.rosa_b200_hard_forward_routes.restype = i32
    lib.rosa_b200_hard_forward_routes.argtypes = [vp, sz, i64, i32, i64, vp, vp, vp]
    lib.rosa_b200_surrogate_vjp_workspace_bytes.restype = sz
    lib.rosa_b200_surrogate_vjp_workspace_bytes.argtypes = [i64, i32, i32, i32, i32, i64, i64, i64,
                                                            i32]
    lib.rosa_b200_surrogate_vjp.restype = i32
    lib.rosa_b200_surrogate_vjp.argtypes = [vp, vp, vp, vp, i32, i64, i32, i32, i32, i32, vp, i64,
                                            i64, i64, vp, vp, vp, f32, f32, f32, i32, i64, i64, vp,
                                            vp, vp, vp, sz, vp]
    lib.rosa_b200_hard_inference_workspace_bytes.restype = sz
    lib.rosa_b200_hard_inference_workspace_bytes.argtypes = [i64, i32, i64]
    lib.rosa_b200_hard_inference.restype = i32
    lib.rosa_b200_hard_inference.argtypes = [vp, vp, vp, i64, i32, i32, i32, vp, i64, i64, i64, vp,
                                             vp, vp, sz, vp]
    lib.rosa_b200_stream_workspace_bytes.restype = sz
    lib.rosa_b200_stream_workspace_bytes.argtypes = [i64, i32]
    lib.rosa_b200_stream_update.restype = i32
    lib.rosa_b200_stream_update.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i64, vp,
                                            vp, vp, vp, i64, i64, vp, vp, vp, sz, vp]
    lib.rosa_b200_read_status.restype = i32
    lib.rosa_b200_read_status.argtypes = [vp, vp, ctypes.POINTER(i32)]
    lib.rosa_b200_decode_status.restype = i32
    lib.rosa_b200_decode_status.argtypes = [i32, i32]
    lib.rosa_b200_profile_enable.restype = None
    lib.rosa_b200_profile_enable.argtypes = [i32]
    lib.rosa_b200_profile_collect.restype = i32
    lib.rosa_b200_profile_collect.argtypes = [ctypes.POINTER(ctypes.c_char_p),
                                              ctypes.POINTER(f32), ctypes.POINTER(i32), i32]
    _lib = lib
    return lib


def profile_enable(on: bool) -> None:
    load().rosa_b200_profile_enable(1 if on else 0)


def profile_collect() -> dict:
    """{kernel name: (total milliseconds, launches)} of the launches recorded since the last call."""
    cap = 64
    names = (ctypes.c_char_p * cap)()
    ms = (ctypes.c_float * cap)()
    launches = (ctypes.c_int * cap)()
    n = load().rosa_b200_profile_collect(names, ms, launches, cap)
    return {names[i].decode(): (float(ms[i]), int(launches[i])) for i in range(n)}


def last_error() -> str:
    return load().rosa_b200_last_error().decode()


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"rosa_soft_b200 C ABI error {rc}: {last_error()}")


def dtype_code(torch_dtype) -> int:
    import torch

    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[torch_dtype]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def hard_forward(q, k, v, cu_seqlens, max_suffix_length, want_routes=True, stream=None):
    """Device tensors in the packed view: q,k [N,H,D], v [N,Hv,Dv]; dense batches pass
    ``cu_seqlens=(B, T)``.  Returns (out, packed_q, packed_k, route_token)."""
    import torch

    lib = load()
    N, H, D = q.shape
    Hv, Dv = v.shape[1:]
    if isinstance(cu_seqlens, tuple):
        S, T = cu_seqlens
        cu, sym_shape = None, (S, H, T)
    else:
        S, T = cu_seqlens.numel() - 1, 0
        cu, sym_shape = cu_seqlens, (H, N)
    out = torch.empty((N, H, Dv), dtype=q.dtype, device=q.device)
    pq = torch.empty(sym_shape, dtype=torch.int32, device=q.device)
    pk = torch.empty_like(pq)
    routes = torch.empty((N, H), dtype=torch.int32, device=q.device) if want_routes else None
    nbytes = lib.rosa_b200_hard_forward_workspace_bytes(N, H, S)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    st = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    check(lib.rosa_b200_hard_forward(_ptr(q), _ptr(k), _ptr(v), dtype_code(q.dtype), N, H, D, Hv,
                                     Dv, _ptr(cu), S, T, int(max_suffix_length), _ptr(out),
                                     _ptr(pq), _ptr(pk), _ptr(routes), _ptr(ws), nbytes,
                                     ctypes.c_void_p(st)))
    return out, pq, pk, routes, ws


def pack_symbols(x, cu_seqlens, stream=None):
    """Sign bits of logits x [N, H, D] as int32 words in the operator's symbol layout: [S, H, T]
    for a dense batch (``cu_seqlens=(S, T)``), [H, N] otherwise."""
    import torch

    N, H, D = x.shape
    if isinstance(cu_seqlens, tuple):
        S, T = cu_seqlens
        out = torch.empty((S, H, T), dtype=torch.int32, device=x.device)
    else:
        S, T = cu_seqlens.numel() - 1, 0
        out = torch.empty((H, N), dtype=torch.int32, device=x.device)
    st = stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream
    check(load().rosa_b200_pack_symbols(_ptr(x), dtype_code(x.dtype), N, H, D, S, T, _ptr(out),
                                        ctypes.c_void_p(st)))
    return out


def hard_forward_packed(packed_q, packed_k, v, bits, cu_seqlens, max_suffix_length, stream=None):
    """Forward on symbols the caller already holds; returns (int8 output [N, H, Dv], route_token,
    workspace)."""
    import torch

    lib = load()
    N, Hv, Dv = v.shape
    if isinstance(cu_seqlens, tuple):
        S, T = cu_seqlens
        H, cu = packed_q.shape[1], None
    else:
        S, T = cu_seqlens.numel() - 1, 0
        H, cu = packed_q.shape[0], cu_seqlens
    out = torch.empty((N, H, Dv), dtype=torch.int8, device=v.device)
    routes = torch.empty((N, H), dtype=torch.int32, device=v.device)
    nbytes = lib.rosa_b200_hard_forward_workspace_bytes(N, H, S)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=v.device)
    st = stream if stream is not None else torch.cuda.current_stream(v.device).cuda_stream
    check(lib.rosa_b200_hard_forward_packed(_ptr(packed_q), _ptr(packed_k), _ptr(v),
                                            dtype_code(v.dtype), N, H, int(bits), Hv, Dv, _ptr(cu),
                                            S, T, int(max_suffix_length), _ptr(out), _ptr(routes),
                                            _ptr(ws), nbytes, ctypes.c_void_p(st)))
    return out, routes, ws


def hard_forward_routes(ws, N, H, num_seq, stream=None):
    """Selected route (local position, 0 = null) and winning match length, int32 [N, H], of the
    :func:`hard_forward` call that filled the workspace ``ws``."""
    import torch

    route = torch.empty((N, H), dtype=torch.int32, device=ws.device)
    length = torch.empty((N, H), dtype=torch.int32, device=ws.device)
    st = stream if stream is not None else torch.cuda.current_stream(ws.device).cuda_stream
    check(load().rosa_b200_hard_forward_routes(_ptr(ws), ws.numel(), N, H, num_seq, _ptr(route),
                                               _ptr(length), ctypes.c_void_p(st)))
    return route, length


def hard_forward_static(q, k, v, cu_seqlens, max_suffix_length, stream=None):
    """Same as :func:`hard_forward` through the entry point that takes no workspace: the only
    device memory touched besides the arguments is the fixed scratch array inside the library.
    The output tensors below are the caller's buffers; the library allocates nothing."""
    import torch

    lib = load()
    N, H, D = q.shape
    Hv, Dv = v.shape[1:]
    if isinstance(cu_seqlens, tuple):
        S, T = cu_seqlens
        cu, sym_shape = None, (S, H, T)
    else:
        S, T = cu_seqlens.numel() - 1, 0
        cu, sym_shape = cu_seqlens, (H, N)
    out = torch.empty((N, H, Dv), dtype=q.dtype, device=q.device)
    pq = torch.empty(sym_shape, dtype=torch.int32, device=q.device)
    pk = torch.empty_like(pq)
    routes = torch.empty((N, H), dtype=torch.int32, device=q.device)
    st = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    check(lib.rosa_b200_hard_forward_static(_ptr(q), _ptr(k), _ptr(v), dtype_code(q.dtype), N, H,
                                            D, Hv, Dv, _ptr(cu), S, T, int(max_suffix_length),
                                            _ptr(out), _ptr(pq), _ptr(pk), _ptr(routes),
                                            ctypes.c_void_p(st)))
    return out, pq, pk, routes


def surrogate_vjp(q, k, v, go, cu_seqlens, packed_q, packed_k, max_suffix_length, scale=1.0,
                  dropout_p=0.0, mismatch_scale=3.0, seed=None, mask=7, batch_offset=0,
                  head_offset=0, stream=None):
    """Returns float32 (dq, dk, dv); entries masked off are ``None``."""
    import torch

    lib = load()
    N, H, D = q.shape
    Hv, Dv = v.shape[1:]
    if isinstance(cu_seqlens, tuple):
        S, T = cu_seqlens
        cu = None
    else:
        S, T = cu_seqlens.numel() - 1, 0
        cu = cu_seqlens
    f32 = dict(dtype=torch.float32, device=q.device)
    dq = torch.empty((N, H, D), **f32) if mask & 1 else None  # (mask bit 0x100: testing aid)
    dk = torch.empty((N, H, D), **f32) if mask & 2 else None
    dv = torch.empty((N, Hv, Dv), **f32) if mask & 4 else None
    nbytes = lib.rosa_b200_surrogate_vjp_workspace_bytes(N, H, D, Hv, Dv, S, T,
                                                         int(max_suffix_length), mask)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    st = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    check(lib.rosa_b200_surrogate_vjp(_ptr(q), _ptr(k), _ptr(v), _ptr(go), dtype_code(q.dtype), N,
                                      H, D, Hv, Dv, _ptr(cu), S, T, int(max_suffix_length),
                                      _ptr(packed_q), _ptr(packed_k), _ptr(seed), float(scale),
                                      float(dropout_p), float(mismatch_scale), mask,
                                      int(batch_offset), int(head_offset), _ptr(dq), _ptr(dk),
                                      _ptr(dv), _ptr(ws), nbytes, ctypes.c_void_p(st)))
    return dq, dk, dv, ws


def hard_inference(qsym, ksym, payload, cu_seqlens, max_suffix_length, stream=None):
    """qsym, ksym int32 [N,H]; payload float32 [N,Hp,Dp]. Returns (out, matched_end)."""
    import torch

    lib = load()
    N, H = qsym.shape
    Hp, Dp = payload.shape[1:]
    if isinstance(cu_seqlens, tuple):
        S, T = cu_seqlens
        cu = None
    else:
        S, T = cu_seqlens.numel() - 1, 0
        cu = cu_seqlens
    out = torch.empty((N, H, Dp), dtype=torch.float32, device=qsym.device)
    end = torch.empty((N, H), dtype=torch.int64, device=qsym.device)
    nbytes = lib.rosa_b200_hard_inference_workspace_bytes(N, H, S)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=qsym.device)
    st = stream if stream is not None else torch.cuda.current_stream(qsym.device).cuda_stream
    check(lib.rosa_b200_hard_inference(_ptr(qsym), _ptr(ksym), _ptr(payload), N, H, Hp, Dp,
                                       _ptr(cu), S, T, int(max_suffix_length), _ptr(out), _ptr(end),
                                       _ptr(ws), nbytes, ctypes.c_void_p(st)))
    return out, end, ws


def stream_update(query, key, payload, chunk_offsets, qk_bits, payload_bits, max_suffix_length,
                  key_masks, query_history, payload_history, lengths, max_length_after, stream=None):
    """One chunked update of the GPU streaming runtime.

    query/key uint8 [n, H], payload uint8 [n, Hp], chunk_offsets int32 [slots + 1] (device);
    state tensors as described in include/rosa_soft_b200.h.  Returns (output uint8 [n, H],
    matched_key_end int64 [n, H], workspace)."""
    import torch

    lib = load()
    n, H = query.shape
    Hp = payload.shape[1]
    slots = chunk_offsets.numel() - 1
    capacity = query_history.shape[-1]
    out = torch.empty((n, H), dtype=torch.uint8, device=query.device)
    end = torch.empty((n, H), dtype=torch.int64, device=query.device)
    nbytes = lib.rosa_b200_stream_workspace_bytes(n, H)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=query.device)
    st = stream if stream is not None else torch.cuda.current_stream(query.device).cuda_stream
    check(lib.rosa_b200_stream_update(_ptr(query), _ptr(key), _ptr(payload), _ptr(chunk_offsets), n,
                                      slots, H, Hp, int(qk_bits), int(payload_bits),
                                      int(max_suffix_length), _ptr(key_masks), _ptr(query_history),
                                      _ptr(payload_history), _ptr(lengths), capacity,
                                      int(max_length_after), _ptr(out), _ptr(end), _ptr(ws), nbytes,
                                      ctypes.c_void_p(st)))
    return out, end, ws


def read_status(ws, stream=None) -> int:
    """Status of the last call that used the workspace tensor ``ws``; ``ws=None`` asks for the last
    workspace-free forward on the current device.  Synchronises the stream."""
    import torch

    device = ws.device if ws is not None else None
    st = stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
    status = ctypes.c_int(0)
    check(load().rosa_b200_read_status(_ptr(ws), ctypes.c_void_p(st), ctypes.byref(status)))
    return status.value
