"""Host-side mirror of the reference's MoE feed-forward interface, over the C ABI.

The reference's CPU backend exposes this path as ``Model::moe(&self, m: &Moe,
h: &[f32], n) -> Vec<f32>`` (engine/src/model.rs:861) on tensors gathered by
``Loader::ffn`` (model.rs:377-421); its Metal backend as ``encode_moe``
(engine/src/metal/mod.rs:2140-2266), which adds into the residual.  ``Moe``
below is that object for a B200: construction uploads the GGUF-layout tensors,
``moe`` / ``moe_`` run the layer on device rows, ``moe_host`` is the CPU
backend's calling convention (host rows in, host delta out).

torch is used for device memory and streams only; all arithmetic is in
``libbivmoe.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import capi
from .workloads import ExpertStack, MoeLayer


def _experts(st: Optional[ExpertStack]) -> capi.Experts:
    e = capi.Experts()
    if st is not None:
        e.ggml_type, e.cols, e.rows, e.n = st.ty, st.cols, st.rows, st.n
        e.data, e.stride_bytes, e.offset_bytes = st.data.ctypes.data, st.stride, st.offset
    return e


def fill_desc(layer: MoeLayer, max_tokens: int, device: int):
    """The ``bivmoe_desc`` of a layer, and the host arrays it points into (keep them
    alive until the create call returns)."""
    d = capi.Desc()
    d.n_embd, d.n_expert, d.n_expert_used = layer.n_embd, layer.n_expert, layer.n_expert_used
    d.n_ff_exp, d.n_ff_shexp = layer.n_ff_exp, layer.n_ff_shexp if layer.has_shared else 0
    d.max_tokens, d.device = max_tokens, device
    keep = [np.ascontiguousarray(layer.router, dtype=np.float32)]
    d.router = keep[0].ctypes.data
    d.gate, d.up, d.down = _experts(layer.gate), _experts(layer.up), _experts(layer.down)
    if layer.has_shared:
        d.sh_gate, d.sh_up, d.sh_down = (_experts(layer.sh_gate), _experts(layer.sh_up),
                                         _experts(layer.sh_down))
        keep.append(np.ascontiguousarray(layer.sh_gate_inp, dtype=np.float32))
        d.sh_gate_inp = keep[1].ctypes.data
    return d, keep


class Moe:
    """One MoE feed-forward layer resident on a B200."""

    def __init__(self, layer: MoeLayer, max_tokens: int, device: int = 0):
        self._h = None
        L = capi.lib()
        d, self._keep = fill_desc(layer, max_tokens, device)
        h = C.c_void_p()
        capi.check(L.bivmoe_create(C.byref(d), C.byref(h)))
        self._adopt(h, layer, max_tokens, device)

    @classmethod
    def dense(cls, gate: ExpertStack, up: ExpertStack, down: ExpertStack, max_tokens: int,
              device: int = 0) -> "Moe":
        """``Ffn::Dense`` (engine/src/model.rs:853-858): ``down(silu(gate h) * up h)`` with
        single matrices; ``moe`` / ``moe_`` / ``moe_host`` then compute the dense block."""
        self = cls.__new__(cls)
        self._h = None
        g, u, dn = _experts(gate), _experts(up), _experts(down)
        h = C.c_void_p()
        capi.check(capi.lib().bivmoe_dense_create(device, gate.cols, gate.rows, max_tokens,
                                                  C.byref(g), C.byref(u), C.byref(dn), C.byref(h)))
        layer = MoeLayer(gate.cols, 1, 1, gate.rows, 0, np.zeros((1, gate.cols), np.float32),
                         gate=gate, up=up, down=down)
        self._adopt(h, layer, max_tokens, device)
        return self

    def _adopt(self, h, layer, max_tokens, device):
        self._h = h
        self.n_embd, self.n_expert, self.k = layer.n_embd, layer.n_expert, layer.n_expert_used
        self.n_ff_exp, self.has_shared = layer.n_ff_exp, layer.has_shared
        self.max_tokens, self.device = max_tokens, device
        self.quantised_down = layer.down.ty not in (0, 1, 30)
        self.last_n = 0

    def close(self):
        if self._h is not None:
            capi.lib().bivmoe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- forward ---------------------------------------------------------
    def _stream(self):
        import torch
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def moe(self, h):
        """``Model::moe``: the delta for device rows ``h`` [n, n_embd] (torch, f32, cuda)."""
        import torch
        out = torch.empty_like(h)
        self.moe_(h, out, accumulate=False)
        return out

    def moe_(self, h, out, accumulate: bool = True):
        """Metal's convention: ``out (+)= moe(h)`` in place, asynchronous on the
        current torch stream."""
        import torch
        assert h.is_cuda and h.dtype == torch.float32 and h.is_contiguous()
        assert out.is_cuda and out.dtype == torch.float32 and out.is_contiguous()
        assert h.shape == out.shape and h.shape[-1] == self.n_embd
        n = h.numel() // self.n_embd
        capi.check(capi.lib().bivmoe_forward(self._h, C.c_void_p(h.data_ptr()),
                                             C.c_void_p(out.data_ptr()), n, int(accumulate),
                                             self._stream()), self._h)
        self.last_n = n
        return out

    def moe_host(self, h_host, out_host=None):
        """The CPU backend's convention: host rows in, host delta out (numpy f32 or
        pinned torch CPU tensors); copies and a stream sync are inside the call."""
        hp, n = _host_ptr(h_host, self.n_embd)
        if out_host is None:
            out_host = np.empty((n, self.n_embd), np.float32)
        op, n2 = _host_ptr(out_host, self.n_embd)
        assert n == n2
        capi.check(capi.lib().bivmoe_forward_host(self._h, hp, op, n), self._h)
        self.last_n = n
        return out_host

    def moe_host_async(self, h_host, out_host):
        """The first half of ``moe_host``: enqueue and return.  ``out_host`` is valid
        after ``wait()``; one pass per layer object may be outstanding."""
        hp, n = _host_ptr(h_host, self.n_embd)
        op, n2 = _host_ptr(out_host, self.n_embd)
        assert n == n2
        capi.check(capi.lib().bivmoe_forward_host_async(self._h, hp, op, n), self._h)
        self.last_n = n

    def wait(self):
        capi.check(capi.lib().bivmoe_host_wait(self._h), self._h)

    def status(self):
        """Waits for the current stream and raises if a kernel of this layer recorded a
        failure on the device (a bounded wait that gave up) since the last report."""
        capi.check(capi.lib().bivmoe_status(self._h, self._stream()), self._h)

    STAGES = ("router", "topk", "sort", "quantize", "gateup", "down", "combine")

    def profile(self, h, out) -> dict:
        """One pass with CUDA events between the stages; device milliseconds per stage."""
        ms = (C.c_float * 7)()
        n = h.numel() // self.n_embd
        capi.check(capi.lib().bivmoe_forward_profile(self._h, C.c_void_p(h.data_ptr()),
                                                     C.c_void_p(out.data_ptr()), n,
                                                     self._stream(), ms), self._h)
        self.last_n = n
        return dict(zip(self.STAGES, [float(v) for v in ms]))

    def route_noalloc(self, h, ids_out, weights_out):
        """The routing step alone, through the entry point that allocates nothing:
        fills the caller's ``ids_out`` [n, k] int32 and ``weights_out`` [n, k] f32
        (device tensors) for device rows ``h``.  Limited to
        ``n * (n_expert + 1) <= capi.ROUTE_NOALLOC_MAX_LOGITS``."""
        import torch
        n = h.numel() // self.n_embd
        assert h.is_cuda and h.dtype == torch.float32 and h.is_contiguous()
        assert ids_out.is_cuda and ids_out.dtype == torch.int32 and ids_out.is_contiguous()
        assert weights_out.is_cuda and weights_out.dtype == torch.float32 and weights_out.is_contiguous()
        assert ids_out.numel() == n * self.k and weights_out.numel() == n * self.k
        capi.check(capi.lib().bivmoe_route_noalloc(self._h, C.c_void_p(h.data_ptr()), n,
                                                   C.c_void_p(ids_out.data_ptr()),
                                                   C.c_void_p(weights_out.data_ptr()),
                                                   self._stream()), self._h)

    def set_post_norm(self, w, eps: float):
        w = np.ascontiguousarray(w, dtype=np.float32)
        assert w.size == self.n_embd
        capi.check(capi.lib().bivmoe_set_post_norm(self._h, w.ctypes.data, eps), self._h)

    # ---- observability ---------------------------------------------------
    def int8_peak(self) -> float:
        """Measured int8 tensor-pipe peak of this GPU, tera-operations per second."""
        v = C.c_double()
        capi.check(capi.lib().bivmoe_int8_peak(self._h, C.byref(v)), self._h)
        return v.value

    def numerics(self) -> str:
        buf = C.create_string_buffer(512)
        capi.check(capi.lib().bivmoe_numerics(self._h, buf, 512), self._h)
        return buf.value.decode()

    def memory(self):
        w, s = C.c_uint64(), C.c_uint64()
        capi.check(capi.lib().bivmoe_memory(self._h, C.byref(w), C.byref(s)), self._h)
        return w.value, s.value

    # ---- parity taps (test only) ------------------------------------------
    def tap(self, which: int) -> np.ndarray:
        n, k, e, ne, ff = self.last_n, self.k, self.n_embd, self.n_expert, self.n_ff_exp
        shape, dt = {
            capi.TAP_LOGITS: ((n, ne), np.float32), capi.TAP_IDS: ((n, k), np.int32),
            capi.TAP_WEIGHTS: ((n, k), np.float32), capi.TAP_COUNTS: ((ne,), np.int32),
            capi.TAP_ORDER: ((n * k,), np.int32), capi.TAP_ACT_Q: ((n, e), np.int8),
            capi.TAP_ACT_D: ((n, e // 32), np.float32), capi.TAP_ACT_S: ((n, e // 32), np.float32),
            capi.TAP_MID: ((n * k, ff), np.float32), capi.TAP_PAIR_OUT: ((n * k, e), np.float32),
            capi.TAP_SHARED_OUT: ((n, e), np.float32), capi.TAP_SHARED_GATE: ((n,), np.float32),
        }[which]
        out = np.empty(shape, dt)
        capi.check(capi.lib().bivmoe_tap(self._h, which, out.ctypes.data, out.nbytes), self._h)
        return out

    def tap_block_dots(self, matrix: int, expert: int, row: int, act_row: int) -> np.ndarray:
        cols = self.n_embd if matrix % 3 != 2 else self.n_ff_exp
        out = np.empty(cols // 32, np.int32)
        capi.check(capi.lib().bivmoe_tap_block_dots(self._h, matrix, expert, row, act_row,
                                                    out.ctypes.data), self._h)
        return out


def _host_ptr(a, e):
    if isinstance(a, np.ndarray):
        assert a.dtype == np.float32 and a.flags.c_contiguous
        return C.c_void_p(a.ctypes.data), a.size // e
    import torch
    assert isinstance(a, torch.Tensor) and not a.is_cuda and a.dtype == torch.float32
    assert a.is_contiguous()
    return C.c_void_p(a.data_ptr()), a.numel() // e


class MoeStack:
    """A run of MoE layers with the residual carried on the device: the FFN half
    of ``Model::layer`` (engine/src/model.rs:788-790) for each layer."""

    def __init__(self, layers: Sequence[Moe]):
        self.layers = list(layers)
        self._arr = (C.c_void_p * len(layers))(*[l._h for l in layers])

    def forward_(self, x):
        import torch
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        l0 = self.layers[0]
        n = x.numel() // l0.n_embd
        capi.check(capi.lib().bivmoe_forward_stack(self._arr, len(self.layers),
                                                   C.c_void_p(x.data_ptr()), n, l0._stream()),
                   l0._h)
        for l in self.layers:
            l.last_n = n
        return x


def launch_count() -> int:
    return int(capi.lib().bivmoe_launch_count())
