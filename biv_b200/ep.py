"""Expert parallelism: one process per GPU, experts sharded ``n_expert / W`` per
rank.  A token's row travels once to every rank that owns one of its experts and
one partial sum per row comes back.  The rows move either through
``torch.distributed`` all-to-alls (NCCL over NVLink between GPUs; gloo between CPU
processes in the tests) or, between the GPUs of one node, as stores of the library's
own kernels into the other ranks' memory (``EpMoe(exchange="peer")``,
``ep_pass_peer``): no packing, no counts on the host, no host wait.

The reference has no multi-device path (one ``MTLDevice``,
engine/src/metal/mod.rs:450-462; the CPU backend loops over the experts in one
process, engine/src/model.rs:875), so this module mirrors nothing there: it
runs ``Model::moe`` (model.rs:861-898) split at its two natural seams - after
routing (rows leave for the ranks that own their experts) and after the expert
products (outputs return to the rows' home rank for the weighted sum).

``ep_plan`` and ``ep_pass`` are the host logic, independent of where the rows
live; the arithmetic is behind a ``steps`` object - ``DeviceSteps`` below calls
the ``bivmoe_ep_*`` entry points of ``libbivmoe.so`` and is the only
implementation this package ships.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, replace
from typing import List, Optional

import numpy as np

from . import capi
from .workloads import ExpertStack, MoeLayer


@dataclass
class EpPlan:
    """What one rank sends and receives, from everyone's per-destination row counts."""
    send_splits: List[int]      # rows this rank sends to each rank (grouped by destination)
    recv_splits: List[int]      # rows it receives from each rank
    m: int                      # rows received in all


def ep_plan(counts_all: np.ndarray, rank: int) -> EpPlan:
    """``counts_all`` [W][W]: entry [s][d] = rows rank s has for rank d (a token's row
    goes once to every rank that owns at least one of its experts)."""
    W = counts_all.shape[0]
    assert counts_all.shape == (W, W) and 0 <= rank < W
    recv = [int(v) for v in counts_all[:, rank]]
    return EpPlan([int(v) for v in counts_all[rank]], recv, sum(recv))


def local_experts(layer: MoeLayer, rank: int, world: int) -> MoeLayer:
    """The layer as rank ``rank`` holds it: its slice of every ``*_exps`` stack (a
    byte range of the same tensor - experts are outermost, model.rs:353), the
    router and the shared expert whole."""
    assert layer.n_expert % world == 0
    nl = layer.n_expert // world

    def cut(st: ExpertStack) -> ExpertStack:
        return ExpertStack(st.ty, st.cols, st.rows, nl, st.data, st.stride,
                           st.offset + rank * nl * st.stride)
    return replace(layer, gate=cut(layer.gate), up=cut(layer.up), down=cut(layer.down))


class TorchComm:
    """The two collectives of a pass over a ``torch.distributed`` process group
    (NCCL between GPUs, gloo between CPU processes)."""

    def __init__(self, group=None):
        self.group = group

    def all_gather(self, out_flat, piece):
        import torch.distributed as dist
        dist.all_gather_into_tensor(out_flat, piece, group=self.group)

    def all_to_all(self, recv, send, recv_splits, send_splits):
        import torch.distributed as dist
        dist.all_to_all_single(recv, send, recv_splits, send_splits, group=self.group)

    def barrier(self, device):
        """Stream-ordered on the current stream: a one-element all-reduce."""
        import torch
        import torch.distributed as dist
        if getattr(self, "_one", None) is None or self._one.device != device:
            self._one = torch.zeros(1, dtype=torch.int32, device=device)
        dist.all_reduce(self._one, group=self.group)

    def all_gather_bytes(self, blob: bytes, device):
        """Every rank's ``blob`` (same length everywhere), in rank order."""
        import torch
        import torch.distributed as dist
        W = dist.get_world_size(self.group)
        mine = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(device)
        out = torch.empty(W * len(blob), dtype=torch.uint8, device=device)
        dist.all_gather_into_tensor(out, mine, group=self.group)
        raw = out.cpu().numpy().tobytes()
        return [raw[r * len(blob):(r + 1) * len(blob)] for r in range(W)]


def ep_pass(steps, h, out, accumulate: bool, comm=None):
    """One pass of the layer over this rank's rows ``h`` [n, n_embd] into ``out``.

    ``steps`` supplies ``rank``, ``world``, ``k`` and
    ``route(h) -> (send_rows, send_tags, send_counts)``, ``shared(h)``,
    ``rows(count)`` / ``tags(count)`` (scratch tensors [count, n_embd] f32 and
    [count, 2k] i32; ``rows`` hands out two distinct buffers in turn),
    ``experts(recv_rows, recv_tags, m) -> out_rows`` and
    ``combine(returned_rows, out, accumulate)``; ``comm`` the two collectives
    (``TorchComm`` over the default process group when None)."""
    comm = comm or TorchComm()
    return ep_pass_finish(steps, h, out, accumulate, comm, ep_pass_begin(steps, h, comm))


def ep_pass_begin(steps, h, comm):
    """The part of a pass before its host synchronisation: routing and the exchange of
    the row counts, enqueued and not waited for.  A host that keeps two passes in flight
    (two micro-batches, each with its own ``steps`` and stream) begins both before it
    finishes either, so that one pass's exchanges overlap the other's kernels."""
    import torch
    W = steps.world
    send_rows, send_tags, send_counts = steps.route(h)
    flat = torch.empty((W * W,), dtype=torch.int32, device=send_counts.device)
    comm.all_gather(flat, send_counts)
    return send_rows, send_tags, flat


def ep_pass_finish(steps, h, out, accumulate: bool, comm, begun):
    W, rank = steps.world, steps.rank
    send_rows, send_tags, flat = begun
    counts_host = flat.view(W, W).cpu().numpy()     # the one host synchronisation of the pass
    plan = ep_plan(counts_host, rank)
    steps.shared(h)                                  # overlaps the exchange where it can
    n_send = sum(plan.send_splits)
    recv_rows, recv_tags = steps.rows(plan.m), steps.tags(plan.m)
    comm.all_to_all(recv_rows, send_rows[:n_send], plan.recv_splits, plan.send_splits)
    comm.all_to_all(recv_tags, send_tags[:n_send], plan.recv_splits, plan.send_splits)
    out_rows = steps.experts(recv_rows, recv_tags, plan.m)
    returned = steps.rows(n_send)
    comm.all_to_all(returned, out_rows, plan.send_splits, plan.recv_splits)
    steps.combine(returned, out, accumulate)
    return plan


def ep_pass_peer(steps, h, out, accumulate: bool, comm, lib_barrier: bool = False):
    """The pass with the library's own exchange kernels (stores into the peers' memory over
    NVLink, ``bivmoe_ep_peer_*``): no packing by destination, no counts on the host, no
    host wait.  The two stream-ordered barriers are ``comm``'s, or with ``lib_barrier`` the
    library's own (``bivmoe_ep_peer_barrier``: flag words in the ranks' blocks, bounded
    waits), which makes the pass five library calls and nothing else - no communicator."""
    barrier = steps.peer_barrier if lib_barrier else (lambda: comm.barrier(h.device))
    steps.peer_dispatch(h)
    steps.shared(h)                 # on the side stream: needs only h, so it also runs while
                                    # this rank waits for the slowest rank's rows
    barrier()                       # every rank's rows are where their owners read them
    steps.peer_experts()
    barrier()                       # the partial sums are back; the receive buffers are free
    steps.peer_combine(out, accumulate)


class DeviceSteps:
    """The ``bivmoe_ep_*`` entry points on one B200 (torch for memory and streams)."""

    def __init__(self, layer: MoeLayer, max_tokens: int, rank: int, world: int, device: int = 0,
                 max_recv_rows: Optional[int] = None):
        import torch
        from .moe import fill_desc
        self._h = None
        self.rank, self.world, self.device = rank, world, device
        self.n_embd, self.n_expert, self.k = layer.n_embd, layer.n_expert, layer.n_expert_used
        self.max_tokens = max_tokens
        nl = layer.n_expert // world
        self.max_recv = max_recv_rows or world * max_tokens
        local = local_experts(layer, rank, world)
        d, self._keep = fill_desc(local, max_tokens, device)
        d.n_expert = layer.n_expert
        h = C.c_void_p()
        capi.check(capi.lib().bivmoe_ep_create(C.byref(d), rank, world, self.max_recv, C.byref(h)))
        self._h = h
        dev = torch.device("cuda", device)
        max_send = max_tokens * min(world, self.k)
        self._send = torch.empty((max_send, self.n_embd), dtype=torch.float32, device=dev)
        self._send_tags = torch.empty((max_send, 2 * self.k), dtype=torch.int32, device=dev)
        self._counts = torch.empty((world,), dtype=torch.int32, device=dev)
        self._bufs = [torch.empty((max(self.max_recv, max_send), self.n_embd),
                                  dtype=torch.float32, device=dev) for _ in range(2)]
        self._recv_tags = torch.empty((self.max_recv, 2 * self.k), dtype=torch.int32, device=dev)
        self._out_rows = torch.empty((self.max_recv, self.n_embd), dtype=torch.float32, device=dev)
        self._turn = 0
        self._side = torch.cuda.Stream(device=dev)
        self._n = 0

    def close(self):
        if self._h is not None:
            capi.lib().bivmoe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self, s=None):
        import torch
        s = s or torch.cuda.current_stream(self.device)
        return C.c_void_p(s.cuda_stream)

    def route(self, h):
        import torch
        assert h.is_cuda and h.dtype == torch.float32 and h.is_contiguous()
        n = h.numel() // self.n_embd
        self._n = n
        capi.check(capi.lib().bivmoe_ep_route(self._h, C.c_void_p(h.data_ptr()), n,
                                              C.c_void_p(self._send.data_ptr()),
                                              C.c_void_p(self._send_tags.data_ptr()),
                                              C.c_void_p(self._counts.data_ptr()), self._stream()),
                   self._h)
        return self._send, self._send_tags, self._counts

    def shared(self, h):
        import torch
        cur = torch.cuda.current_stream(self.device)
        self._side.wait_stream(cur)
        capi.check(capi.lib().bivmoe_ep_shared(self._h, C.c_void_p(h.data_ptr()),
                                               self._stream(self._side)), self._h)

    def rows(self, count: int):
        self._turn ^= 1
        return self._bufs[self._turn][:count]

    def tags(self, count: int):
        return self._recv_tags[:count]

    def experts(self, recv_rows, recv_tags, m: int):
        capi.check(capi.lib().bivmoe_ep_experts(self._h, C.c_void_p(recv_rows.data_ptr()),
                                                C.c_void_p(recv_tags.data_ptr()), m,
                                                C.c_void_p(self._out_rows.data_ptr()),
                                                self._stream()), self._h)
        return self._out_rows[:m]

    def combine(self, returned, out, accumulate: bool):
        import torch
        torch.cuda.current_stream(self.device).wait_stream(self._side)   # the shared expert is done
        capi.check(capi.lib().bivmoe_ep_combine(self._h, C.c_void_p(returned.data_ptr()),
                                                C.c_void_p(out.data_ptr()), self._n,
                                                int(accumulate), self._stream()), self._h)

    def status(self):
        capi.check(capi.lib().bivmoe_ep_status(self._h, self._stream()), self._h)

    # ---- the peer-store exchange --------------------------------------------
    def peer_info(self) -> bytes:
        info = capi.PeerInfo()
        capi.check(capi.lib().bivmoe_ep_peer_info(self._h, C.byref(info)), self._h)
        return bytes(info)

    def peer_attach(self, infos):
        arr = (capi.PeerInfo * self.world)(*[capi.PeerInfo.from_buffer_copy(b) for b in infos])
        capi.check(capi.lib().bivmoe_ep_peer_attach(self._h, arr), self._h)

    def peer_dispatch(self, h):
        import torch
        assert h.is_cuda and h.dtype == torch.float32 and h.is_contiguous()
        n = h.numel() // self.n_embd
        self._n = n
        capi.check(capi.lib().bivmoe_ep_peer_dispatch(self._h, C.c_void_p(h.data_ptr()), n,
                                                      self._stream()), self._h)

    def peer_experts(self):
        capi.check(capi.lib().bivmoe_ep_peer_experts(self._h, self._stream()), self._h)

    def peer_signal(self):
        capi.check(capi.lib().bivmoe_ep_peer_signal(self._h, self._stream()), self._h)

    def peer_wait(self):
        capi.check(capi.lib().bivmoe_ep_peer_wait(self._h, self._stream()), self._h)

    def peer_barrier(self):
        capi.check(capi.lib().bivmoe_ep_peer_barrier(self._h, self._stream()), self._h)

    def peer_wait_limit(self, microseconds: int):
        capi.check(capi.lib().bivmoe_ep_peer_wait_limit(self._h, microseconds), self._h)

    def peer_combine(self, out, accumulate: bool):
        import torch
        torch.cuda.current_stream(self.device).wait_stream(self._side)   # the shared expert is done
        capi.check(capi.lib().bivmoe_ep_peer_combine(self._h, C.c_void_p(out.data_ptr()), self._n,
                                                     int(accumulate), self._stream()), self._h)


class EpMoe:
    """``Moe`` (moe.py) for a layer whose experts are spread over the ranks of a
    process group; every rank passes its own rows."""

    def __init__(self, layer: MoeLayer, max_tokens: int, rank: int, world: int, device: int = 0,
                 comm=None, max_recv_rows: Optional[int] = None, exchange: str = "all_to_all",
                 barrier: str = "comm"):
        """``exchange``: "all_to_all" (the communicator's collectives move the rows) or
        "peer" (the library's kernels store them into the peers' memory; the ranks are on
        the GPUs of one node; all ranks construct the object together).  ``barrier`` (peer
        form): "comm" - the communicator's stream-ordered barrier - or "lib" - the
        library's own, for ranks on different GPUs; the communicator is then used at
        construction only."""
        import torch
        assert exchange in ("all_to_all", "peer") and barrier in ("comm", "lib")
        self.lib_barrier = barrier == "lib"
        self.steps = DeviceSteps(layer, max_tokens, rank, world, device, max_recv_rows)
        self.comm = comm or TorchComm()
        self.n_embd = layer.n_embd
        self.last_plan: Optional[EpPlan] = None
        self.exchange = exchange
        if exchange == "peer" and world > 1:
            infos = self.comm.all_gather_bytes(self.steps.peer_info(), torch.device("cuda", device))
            self.steps.peer_attach(infos)

    def moe_(self, h, out, accumulate: bool = True):
        if self.exchange == "peer" and self.steps.world > 1:
            ep_pass_peer(self.steps, h, out, accumulate, self.comm, self.lib_barrier)
        else:
            self.last_plan = ep_pass(self.steps, h, out, accumulate, self.comm)
        return out

    def capture(self, h, out, accumulate: bool = False):
        """One pass over fixed tensors as a CUDA graph (``.replay()`` runs it): the peer
        exchange has no host step, so the whole pass - this rank's kernels, its stores into
        the peers and the two barrier all-reduces - is one graph launch.  Run the pass
        eagerly a few times first, then bring all ranks to the same point (a process-group
        barrier and a device synchronize) before any of them captures; all ranks capture
        and replay together."""
        import torch
        assert self.exchange == "peer", "the all-to-all form reads the row counts on the host"
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.moe_(h, out, accumulate)
        return g

    def begin(self, h):
        """``moe_`` in two halves (see ``ep_pass_begin``): enqueue the routing."""
        self._begun = (h, ep_pass_begin(self.steps, h, self.comm))

    def finish(self, out, accumulate: bool = True):
        h, begun = self._begun
        self.last_plan = ep_pass_finish(self.steps, h, out, accumulate, self.comm, begun)
        return out

    def moe(self, h):
        import torch
        out = torch.empty_like(h)
        return self.moe_(h, out, accumulate=False)

    def status(self):
        self.steps.status()

    def close(self):
        self.steps.close()
