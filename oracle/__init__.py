"""ctypes front of the CPU oracle (``bivmoe_oracle.c``).

Test infrastructure only: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py`` for its CPU-baseline / reference arm.  The shipped package
never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libbivmoe_oracle.so")

LEVEL_NAMES = {0: "scalar", 1: "avx2", 2: "avxvnni"}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "bivmoe_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


class _Experts(C.Structure):
    _fields_ = [("ty", C.c_int32), ("_pad", C.c_int32), ("cols", C.c_int64), ("rows", C.c_int64),
                ("n", C.c_int64), ("data", C.c_void_p), ("stride", C.c_int64),
                ("offset", C.c_int64)]


class _Moe(C.Structure):
    _fields_ = [("n_embd", C.c_int32), ("n_expert", C.c_int32), ("n_expert_used", C.c_int32),
                ("n_ff_exp", C.c_int32), ("n_ff_shexp", C.c_int32), ("has_shared", C.c_int32),
                ("router", C.c_void_p),
                ("gate", _Experts), ("up", _Experts), ("down", _Experts),
                ("sh_gate", _Experts), ("sh_up", _Experts), ("sh_down", _Experts),
                ("sh_gate_inp", C.c_void_p)]


_TAP_FIELDS = ["logits", "ids", "weights", "counts", "order", "pair_out", "shared_out",
               "shared_gate", "act_q", "act_d", "act_s", "mid_q", "mid_d", "mid"]


class _Taps(C.Structure):
    _fields_ = [(f, C.c_void_p) for f in _TAP_FIELDS]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_row_size.restype = C.c_long
        L.orc_row_size.argtypes = [C.c_int, C.c_long]
        L.orc_dot.restype = C.c_float
        L.orc_dot.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 5 + [C.c_long]
        L.orc_dot_f32.restype = C.c_float
        L.orc_dot_f32.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_long]
        L.orc_axpy.restype = None
        L.orc_axpy.argtypes = [C.c_int, C.c_void_p, C.c_float, C.c_void_p, C.c_long]
        L.orc_sigmoid.restype = C.c_float
        L.orc_sigmoid.argtypes = [C.c_float]
        L.orc_silu.restype = C.c_float
        L.orc_silu.argtypes = [C.c_float]
        L.orc_q8_quantize.restype = None
        L.orc_q8_quantize.argtypes = [C.c_void_p, C.c_long, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_dequantize_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_long]
        L.orc_block_dots.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_long, C.c_void_p]
        L.orc_matmul.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_long, C.c_long, C.c_void_p,
                                 C.c_long, C.c_void_p, C.c_int]
        L.orc_rms_norm.restype = None
        L.orc_rms_norm.argtypes = [C.c_int, C.c_void_p, C.c_long, C.c_void_p, C.c_long, C.c_float]
        L.orc_softmax.restype = None
        L.orc_softmax.argtypes = [C.c_void_p, C.c_long]
        L.orc_route.restype = None
        L.orc_route.argtypes = [C.c_void_p, C.c_long, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_moe_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_void_p, C.c_int,
                                      C.c_int, C.c_void_p]
        L.orc_moe_stack.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_void_p,
                                    C.c_long, C.c_int, C.c_int]
        _lib = L
    return _lib


def host_level() -> int:
    """The kernel level the reference would run on this host (0 scalar, 1 avx2, 2 avxvnni)."""
    return lib().orc_host_level()


def max_threads() -> int:
    return lib().orc_max_threads()


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def f16_to_f32(h: int) -> float:
    return lib().orc_f16_to_f32(h)


def bf16_to_f32(h: int) -> float:
    return lib().orc_bf16_to_f32(h)


def q8_quantize(x):
    x = _f32(x)
    qs = np.empty(x.shape, np.int8)
    d = np.empty(x.shape[:-1] + (x.shape[-1] // 32,), np.float32)
    s = np.empty_like(d)
    lib().orc_q8_quantize(_p(x), x.size, _p(qs), _p(d), _p(s))
    return qs, d, s


def dequantize_row(ty, row_bytes, n):
    row_bytes = np.ascontiguousarray(row_bytes, dtype=np.uint8)
    out = np.empty(n, np.float32)
    assert lib().orc_dequantize_row(ty, _p(row_bytes), _p(out), n) == 0
    return out


def dot(level, ty, w, x):
    """One weight row (bytes) against one f32 activation row, as the reference's
    ``dot`` after ``Input::q8``."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = _f32(x)
    qs, d, s = q8_quantize(x)
    return lib().orc_dot(level, ty, _p(w), _p(x), _p(qs), _p(d), _p(s), x.size)


def dot_f32(level, a, b):
    a, b = _f32(a), _f32(b)
    return lib().orc_dot_f32(level, _p(a), _p(b), a.size)


def axpy(level, y, a, x):
    y = _f32(y).copy()
    x = _f32(x)
    lib().orc_axpy(level, _p(y), a, _p(x), x.size)
    return y


def block_dots(ty, w, xq):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    xq = np.ascontiguousarray(xq, dtype=np.int8)
    out = np.empty(xq.size // 32, np.int32)
    assert lib().orc_block_dots(ty, _p(w), _p(xq), xq.size, _p(out)) == 0
    return out


def matmul(level, ty, w, rows, cols, x, threads=1):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = _f32(x).reshape(-1, cols)
    out = np.empty((x.shape[0], rows), np.float32)
    assert lib().orc_matmul(level, ty, _p(w), rows, cols, _p(x), x.shape[0], _p(out), threads) == 0
    return out


def rms_norm(level, x, w, eps):
    x = _f32(x).copy()
    w = _f32(w)
    lib().orc_rms_norm(level, _p(x), x.size // w.size, _p(w), w.size, eps)
    return x


def route(logits, k):
    logits = _f32(logits)
    ids = np.empty(k, np.int32)
    w = np.empty(k, np.float32)
    scratch = np.empty(logits.size, np.float32)
    lib().orc_route(_p(logits), logits.size, k, _p(ids), _p(w), _p(scratch))
    return ids, w


def _experts(st) -> _Experts:
    e = _Experts()
    if st is None:
        return e
    e.ty, e.cols, e.rows, e.n = st.ty, st.cols, st.rows, st.n
    e.data, e.stride, e.offset = st.data.ctypes.data, st.stride, st.offset
    return e


def _moe_struct(layer) -> _Moe:
    m = _Moe()
    m.n_embd, m.n_expert, m.n_expert_used = layer.n_embd, layer.n_expert, layer.n_expert_used
    m.n_ff_exp, m.n_ff_shexp, m.has_shared = layer.n_ff_exp, layer.n_ff_shexp, int(layer.has_shared)
    m.router = layer.router.ctypes.data
    m.gate, m.up, m.down = _experts(layer.gate), _experts(layer.up), _experts(layer.down)
    m.sh_gate, m.sh_up, m.sh_down = (_experts(layer.sh_gate), _experts(layer.sh_up),
                                     _experts(layer.sh_down))
    m.sh_gate_inp = layer.sh_gate_inp.ctypes.data if layer.has_shared else None
    return m


def moe_forward(layer, h, level=None, threads=1, taps=False):
    """The reference's ``Model::moe`` on f32 rows ``h`` [n, n_embd].  Returns the
    delta [n, n_embd]; with ``taps`` also a dict of intermediates."""
    level = host_level() if level is None else level
    h = _f32(h)
    n, e, k, ne, ff = h.shape[0], layer.n_embd, layer.n_expert_used, layer.n_expert, layer.n_ff_exp
    out = np.empty((n, e), np.float32)
    m = _moe_struct(layer)
    t = None
    tap = {}
    if taps:
        quant_down = layer.down.ty not in (0, 1, 30)
        tap = dict(
            logits=np.empty((n, ne), np.float32), ids=np.empty((n, k), np.int32),
            weights=np.empty((n, k), np.float32), counts=np.empty(ne, np.int32),
            order=np.empty(n * k, np.int32), pair_out=np.empty((n * k, e), np.float32),
            shared_out=np.empty((n, e), np.float32) if layer.has_shared else None,
            shared_gate=np.empty(n, np.float32) if layer.has_shared else None,
            act_q=np.empty((n, e), np.int8), act_d=np.empty((n, e // 32), np.float32),
            act_s=np.empty((n, e // 32), np.float32),
            mid_q=np.empty((n * k, ff), np.int8) if quant_down else None,
            mid_d=np.empty((n * k, ff // 32), np.float32) if quant_down else None,
            mid=np.empty((n * k, ff), np.float32))
        t = _Taps()
        for f in _TAP_FIELDS:
            setattr(t, f, tap[f].ctypes.data if tap[f] is not None else None)
    rc = lib().orc_moe_forward(C.byref(m), _p(h), n, _p(out), level, threads,
                               C.byref(t) if t is not None else None)
    if rc:
        raise RuntimeError(f"oracle moe_forward failed: {rc}")
    return (out, tap) if taps else out


def moe_stack(layers, norm_w, eps, x0, level=None, threads=1):
    """``x += moe_l(rms_norm(x, norm_w[l]))`` over the layers; returns the final x."""
    level = host_level() if level is None else level
    x = _f32(x0).copy()
    arr = (_Moe * len(layers))(*[_moe_struct(l) for l in layers])
    nw = [_f32(w) for w in norm_w]
    ptrs = (C.c_void_p * len(layers))(*[w.ctypes.data for w in nw])
    rc = lib().orc_moe_stack(arr, len(layers), ptrs, eps, _p(x), x.shape[0], level, threads)
    if rc:
        raise RuntimeError(f"oracle moe_stack failed: {rc}")
    return x
