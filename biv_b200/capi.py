"""ctypes binding of ``libbivmoe.so`` (the C ABI declared in ``include/bivmoe.h``).

There is no CPU fallback: importing this module without the built library
raises, and so does every call that returns a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# BIVMOE_LIB names another build of the library (a development aid for comparing builds)
LIB_PATH = os.environ.get("BIVMOE_LIB") or os.path.join(_HERE, "libbivmoe.so")

OK, ERR_ARGUMENT, ERR_UNSUPPORTED, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = range(7)
STATUS_NAMES = {1: "argument", 2: "unsupported (NoKernel)", 3: "out of memory", 4: "cuda",
                5: "nccl", 6: "timeout"}

(TAP_LOGITS, TAP_IDS, TAP_WEIGHTS, TAP_COUNTS, TAP_ORDER, TAP_ACT_Q, TAP_ACT_D, TAP_ACT_S,
 TAP_MID, TAP_PAIR_OUT, TAP_SHARED_OUT, TAP_SHARED_GATE) = range(12)

ROUTE_NOALLOC_MAX_LOGITS = 512 * 257

# every symbol include/bivmoe.h declares
SYMBOLS = ["bivmoe_create", "bivmoe_destroy", "bivmoe_forward", "bivmoe_forward_host", "bivmoe_forward_profile",
           "bivmoe_set_post_norm", "bivmoe_forward_stack", "bivmoe_tap", "bivmoe_tap_block_dots",
           "bivmoe_route_noalloc", "bivmoe_numerics", "bivmoe_memory", "bivmoe_launch_count", "bivmoe_last_error",
           "bivmoe_global_error", "bivmoe_ep_create", "bivmoe_ep_route", "bivmoe_ep_shared",
           "bivmoe_ep_experts", "bivmoe_ep_combine", "bivmoe_ep_status", "bivmoe_forward_host_async",
           "bivmoe_host_wait", "bivmoe_int8_peak", "bivmoe_dense_create", "bivmoe_ep_peer_info",
           "bivmoe_ep_peer_attach", "bivmoe_ep_peer_dispatch", "bivmoe_ep_peer_experts",
           "bivmoe_ep_peer_combine", "bivmoe_status", "bivmoe_last_oom_bytes", "bivmoe_ep_peer_signal",
           "bivmoe_ep_peer_wait", "bivmoe_ep_peer_barrier", "bivmoe_ep_peer_wait_limit"]


class BivMoeError(RuntimeError):
    """A non-zero status from the library; ``code`` is the BIVMOE_ERR_* value.
    Maps to the reference's ``Error::Backend`` / ``NoKernel`` / ``OutOfMemory``
    (engine/src/error.rs:36-68)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"bivmoe status {code} ({STATUS_NAMES.get(code, '?')}): {message}")
        self.code = code


class Experts(C.Structure):
    _fields_ = [("ggml_type", C.c_int32), ("reserved", C.c_int32), ("cols", C.c_int64),
                ("rows", C.c_int64), ("n", C.c_int64), ("data", C.c_void_p),
                ("stride_bytes", C.c_int64), ("offset_bytes", C.c_int64)]


class Desc(C.Structure):
    _fields_ = [("n_embd", C.c_int32), ("n_expert", C.c_int32), ("n_expert_used", C.c_int32),
                ("n_ff_exp", C.c_int32), ("n_ff_shexp", C.c_int32), ("max_tokens", C.c_int32),
                ("device", C.c_int32), ("reserved", C.c_int32), ("router", C.c_void_p),
                ("gate", Experts), ("up", Experts), ("down", Experts),
                ("sh_gate", Experts), ("sh_up", Experts), ("sh_down", Experts),
                ("sh_gate_inp", C.c_void_p)]


_lib = None


class PeerInfo(C.Structure):
    """``bivmoe_peer_info``: how another rank reaches this rank's exchange block."""
    _fields_ = [("ipc_handle", C.c_uint8 * 64), ("base", C.c_void_p), ("pid", C.c_int64),
                ("bytes", C.c_int64), ("device", C.c_int32), ("reserved", C.c_int32)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; "
                "g.build()'` (or `make -C biv_b200/csrc`); there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        vp, i32 = C.c_void_p, C.c_int32
        L.bivmoe_create.argtypes = [C.POINTER(Desc), C.POINTER(vp)]
        L.bivmoe_dense_create.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(Experts),
                                          C.POINTER(Experts), C.POINTER(Experts), C.POINTER(vp)]
        L.bivmoe_destroy.argtypes = [vp]
        L.bivmoe_destroy.restype = None
        L.bivmoe_forward.argtypes = [vp, vp, vp, i32, i32, vp]
        L.bivmoe_forward_host.argtypes = [vp, vp, vp, i32]
        L.bivmoe_forward_host_async.argtypes = [vp, vp, vp, i32]
        L.bivmoe_host_wait.argtypes = [vp]
        L.bivmoe_int8_peak.argtypes = [vp, C.POINTER(C.c_double)]
        L.bivmoe_forward_profile.argtypes = [vp, vp, vp, i32, vp, C.POINTER(C.c_float)]
        L.bivmoe_set_post_norm.argtypes = [vp, vp, C.c_float]
        L.bivmoe_forward_stack.argtypes = [C.POINTER(vp), i32, vp, i32, vp]
        L.bivmoe_tap.argtypes = [vp, i32, vp, C.c_size_t]
        L.bivmoe_tap_block_dots.argtypes = [vp, i32, i32, i32, i32, vp]
        L.bivmoe_route_noalloc.argtypes = [vp, vp, i32, vp, vp, vp]
        L.bivmoe_ep_create.argtypes = [C.POINTER(Desc), i32, i32, i32, C.POINTER(vp)]
        L.bivmoe_ep_route.argtypes = [vp, vp, i32, vp, vp, vp, vp]
        L.bivmoe_ep_shared.argtypes = [vp, vp, vp]
        L.bivmoe_ep_experts.argtypes = [vp, vp, vp, i32, vp, vp]
        L.bivmoe_ep_combine.argtypes = [vp, vp, vp, i32, i32, vp]
        L.bivmoe_ep_status.argtypes = [vp, vp]
        L.bivmoe_ep_peer_info.argtypes = [vp, C.POINTER(PeerInfo)]
        L.bivmoe_ep_peer_attach.argtypes = [vp, C.POINTER(PeerInfo)]
        L.bivmoe_ep_peer_dispatch.argtypes = [vp, vp, i32, vp]
        L.bivmoe_ep_peer_experts.argtypes = [vp, vp]
        L.bivmoe_ep_peer_combine.argtypes = [vp, vp, i32, i32, vp]
        L.bivmoe_status.argtypes = [vp, vp]
        L.bivmoe_last_oom_bytes.restype = C.c_uint64
        L.bivmoe_ep_peer_signal.argtypes = [vp, vp]
        L.bivmoe_ep_peer_wait.argtypes = [vp, vp]
        L.bivmoe_ep_peer_barrier.argtypes = [vp, vp]
        L.bivmoe_ep_peer_wait_limit.argtypes = [vp, C.c_uint64]
        L.bivmoe_numerics.argtypes = [vp, C.c_char_p, C.c_size_t]
        L.bivmoe_memory.argtypes = [vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.bivmoe_launch_count.restype = C.c_uint64
        L.bivmoe_last_error.argtypes = [vp]
        L.bivmoe_last_error.restype = C.c_char_p
        L.bivmoe_global_error.restype = C.c_char_p
        _lib = L
    return _lib


def check(code: int, handle=None):
    if code:
        L = lib()
        msg = (L.bivmoe_last_error(handle) if handle else L.bivmoe_global_error()) or b""
        raise BivMoeError(code, msg.decode(errors="replace"))
