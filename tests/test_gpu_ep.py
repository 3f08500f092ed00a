"""Expert parallelism on the GPU, through the bivmoe_ep_* entry points.

One GPU: W ranks as threads of this process, each with its own layer object on
cuda:0, exchanging rows through ``ThreadComm`` (tensor copies between barriers).
This runs the device steps exactly as W processes would, without a second GPU.
Two or more GPUs: the same pass as real processes over NCCL.

Gates: every rank's output equals the single-GPU layer's output on the same rows
up to the association of the f32 sum over a token's experts (the ranks return
partial sums), and is within the layer tolerance of the CPU oracle.
"""
import os
import socket
import threading

import numpy as np
import pytest

import oracle
from biv_b200 import workloads as W
from helpers import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3


class ThreadComm:
    """The two collectives of ``ep_pass`` between threads of one process whose
    tensors live on one device and are produced on one stream."""

    class Shared:
        def __init__(self, world):
            self.world = world
            self.barrier = threading.Barrier(world)
            self.slots = [None] * world

    def __init__(self, shared, rank):
        self.sh, self.rank = shared, rank

    def _publish(self, value):
        self.sh.slots[self.rank] = value
        self.sh.barrier.wait()
        got = list(self.sh.slots)
        self.sh.barrier.wait()
        return got

    def all_gather(self, out_flat, piece):
        pieces = self._publish(piece)
        n = piece.numel()
        for r, p in enumerate(pieces):
            out_flat[r * n:(r + 1) * n].copy_(p)
        self.sh.barrier.wait()          # nobody's piece is overwritten before all have read it

    def all_to_all(self, recv, send, recv_splits, send_splits):
        sends = self._publish((send, send_splits))
        at = 0
        for r, (rows, splits) in enumerate(sends):
            lo = sum(splits[:self.rank])
            c = splits[self.rank]
            assert c == recv_splits[r]
            recv[at:at + c].copy_(rows[lo:lo + c])
            at += c
        self.sh.barrier.wait()

    def barrier(self, device):
        # the ranks launch on one stream: the order of the launches is the order of the work
        self.sh.barrier.wait()

    def all_gather_bytes(self, blob, device):
        return self._publish(blob)


def _run_threads(world, layer, h, max_tokens, exchange="all_to_all"):
    import torch
    from biv_b200.ep import EpMoe
    n_per = h.shape[0] // world
    shared = ThreadComm.Shared(world)
    outs, errs = [None] * world, [None] * world
    plans = [None] * world

    def rank_main(r):
        try:
            torch.cuda.set_device(0)
            m = EpMoe(layer, max_tokens, r, world, 0, comm=ThreadComm(shared, r), exchange=exchange)
            try:
                hr = torch.from_numpy(np.ascontiguousarray(h[r * n_per:(r + 1) * n_per])).cuda()
                for _ in range(2):       # twice: the scratch buffers are reused
                    out = m.moe(hr)
                m.status()
                outs[r] = out.cpu().numpy()
                plans[r] = m.last_plan
            finally:
                m.close()
        except BaseException as e:      # noqa: BLE001 - reported by the main thread
            errs[r] = e
            shared.barrier.abort()

    ts = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for e in errs:
        if e is not None and not isinstance(e, threading.BrokenBarrierError):
            raise e
    for e in errs:
        if e is not None:
            raise e
    return np.concatenate(outs), plans


def _small(cfg, n):
    if cfg == "mtp_stack":      # Q5_K gate/up, Q6_K down; one layer of the stack
        return W.mtp_stack(n_seq=n // 5, n_tok=5, n_layers=1, **W.SMALL)
    return getattr(W, cfg)(n=n, **W.SMALL)


def _single_gpu(layer, h):
    import torch
    from biv_b200.moe import Moe
    m = Moe(layer, h.shape[0])
    try:
        out = m.moe(torch.from_numpy(h).cuda())
        torch.cuda.synchronize()
        return out.cpu().numpy()
    finally:
        m.close()


@pytest.mark.parametrize("cfg,world,n", [("parity_q8_0", 2, 16), ("decode_q4k", 4, 24),
                                         ("mtp_stack", 2, 10), ("ep_bf16", 2, 32),
                                         ("ep_bf16", 4, 12)])
def test_ranks_as_threads_match_the_single_gpu_layer(cfg, world, n):
    wl = _small(cfg, n)
    layer, h = wl.layers[0], np.ascontiguousarray(wl.h)
    got, plans = _run_threads(world, layer, h, max_tokens=n // world)
    # a rank routes its rows alone, so the reference is the layer applied per rank
    n_per = n // world
    want = np.concatenate([_single_gpu(layer, np.ascontiguousarray(h[r * n_per:(r + 1) * n_per]))
                           for r in range(world)])
    # (BF16: an owner's groups gather the rows of every rank and can pass the 9 rows from
    # which the tensor-core kernel - f32 rows as two bf16 terms, 2^-17 of a value - takes
    # over from the float kernel that the rank alone would use)
    atol = (3e-5 if cfg == "ep_bf16" else 1e-6) * float(np.abs(want).max())
    np.testing.assert_allclose(got, want, rtol=0, atol=atol)
    ref = oracle.moe_forward(layer, h)
    assert rel_err(got, ref) < TOL
    # a token's row goes once to every rank that owns one of its experts
    k = layer.n_expert_used
    assert n <= sum(p.m for p in plans) <= n * min(world, k)


@pytest.mark.parametrize("cfg,world,n", [("parity_q8_0", 2, 16), ("decode_q4k", 4, 24),
                                         ("mtp_stack", 2, 10), ("ep_bf16", 4, 12)])
def test_peer_store_exchange_ranks_as_threads(cfg, world, n):
    """The exchange by the library's own kernels (stores into the ranks' blocks): the same
    result as the all-to-all form, bit for bit - the rows, their order per owner up to the
    regions' padding, and the order of every sum are the same."""
    wl = _small(cfg, n)
    layer, h = wl.layers[0], np.ascontiguousarray(wl.h)
    got, _ = _run_threads(world, layer, h, max_tokens=n // world, exchange="peer")
    want, _ = _run_threads(world, layer, h, max_tokens=n // world)
    assert np.array_equal(got, want)
    assert rel_err(got, oracle.moe_forward(layer, h)) < TOL


def test_peer_store_exchange_with_room_to_spare_and_ragged_ranks():
    """max_tokens above the rows in use (regions mostly padding), and a rank without rows."""
    import torch
    from biv_b200.ep import EpMoe
    wl = _small("decode_q4k", 12)
    layer, h = wl.layers[0], np.ascontiguousarray(wl.h)
    world, cap = 2, 16
    rows = [h[:12], h[:0]]
    shared = ThreadComm.Shared(world)
    outs, errs = [None] * world, [None] * world

    def rank_main(r):
        try:
            m = EpMoe(layer, cap, r, world, 0, comm=ThreadComm(shared, r), exchange="peer")
            try:
                hr = torch.from_numpy(np.ascontiguousarray(rows[r])).cuda()
                for _ in range(2):
                    out = m.moe(hr)
                m.status()
                outs[r] = out.cpu().numpy()
            finally:
                m.close()
        except BaseException as e:      # noqa: BLE001
            errs[r] = e
            shared.barrier.abort()

    ts = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for e in errs:
        if e is not None:
            raise e
    assert outs[1].shape == (0, layer.n_embd)
    assert rel_err(outs[0], oracle.moe_forward(layer, h)) < TOL


def test_full_size_layer_two_ranks_as_threads():
    """The BF16 configuration at its real shape, 512 rows: groups large and small."""
    wl = W.ep_bf16(n=512)
    layer, h = wl.layers[0], np.ascontiguousarray(wl.h)
    got, _ = _run_threads(2, layer, h, max_tokens=256)
    ref = oracle.moe_forward(layer, h, threads=oracle.max_threads())
    assert rel_err(got, ref) < TOL


def test_steps_reject_a_plain_layer_and_bad_sizes():
    import ctypes as C
    import torch
    from biv_b200 import capi
    from biv_b200.ep import DeviceSteps
    from biv_b200.moe import Moe
    wl = W.parity_q8_0(n=8, **W.SMALL)
    m = Moe(wl.layers[0], 8)
    try:
        with pytest.raises(capi.BivMoeError) as ei:
            capi.check(capi.lib().bivmoe_ep_status(m._h, None), m._h)
        assert ei.value.code == capi.ERR_ARGUMENT
    finally:
        m.close()
    st = DeviceSteps(wl.layers[0], 8, 0, 2, 0)
    try:
        h = torch.from_numpy(wl.h).cuda()
        with pytest.raises(capi.BivMoeError):       # more rows than max_tokens
            st.route(torch.cat([h, h]))
        with pytest.raises(capi.BivMoeError):       # a whole-layer call on a sharded layer
            capi.check(capi.lib().bivmoe_forward(st._h, C.c_void_p(h.data_ptr()),
                                                 C.c_void_p(h.data_ptr()), 8, 0, None), st._h)
        with pytest.raises(capi.BivMoeError):       # more received rows than max_recv_rows
            capi.check(capi.lib().bivmoe_ep_experts(st._h, C.c_void_p(h.data_ptr()),
                                                    C.c_void_p(h.data_ptr()), st.max_recv + 1,
                                                    C.c_void_p(h.data_ptr()), None), st._h)
        st.status()                                 # nothing failed on the device
    finally:
        st.close()


def test_a_whole_pass_through_the_c_abi_alone_with_the_library_barrier():
    """Two ranks as two layer objects on one GPU, driven from one host thread through
    ctypes only - no torch.distributed, no communicator: peer info gathered by hand, then
    per pass dispatch, barrier, shared, experts, barrier, combine.  The ranks share a GPU,
    so every rank's signal is enqueued before any rank's wait (a waiting kernel must never
    depend on a launch that may not be running beside it)."""
    import torch
    from biv_b200.ep import DeviceSteps
    wl = _small("decode_q4k", 24)
    layer, h = wl.layers[0], np.ascontiguousarray(wl.h)
    world, n_per = 2, 12
    ranks = [DeviceSteps(layer, n_per, r, world, 0) for r in range(world)]
    try:
        infos = [st.peer_info() for st in ranks]
        for st in ranks:
            st.peer_attach(infos)
            st.peer_wait_limit(200_000)     # 0.2 s: ample on one GPU, and it bounds the test
        hs = [torch.from_numpy(h[r * n_per:(r + 1) * n_per]).cuda() for r in range(world)]
        outs = [torch.empty_like(x) for x in hs]
        for _ in range(3):                  # thrice: the regions and the barrier numbers move on
            for st, x in zip(ranks, hs):
                st.peer_dispatch(x)
            for st in ranks:
                st.peer_signal()
            for st in ranks:
                st.peer_wait()
            for st, x in zip(ranks, hs):
                st.shared(x)
                st.peer_experts()
            for st in ranks:
                st.peer_signal()
            for st in ranks:
                st.peer_wait()
            for st, o in zip(ranks, outs):
                st.peer_combine(o, False)
        for st in ranks:
            st.status()                     # no wait gave up
        got = np.concatenate([o.cpu().numpy() for o in outs])
    finally:
        for st in ranks:
            st.close()
    want = np.concatenate([_single_gpu(layer, np.ascontiguousarray(h[r * n_per:(r + 1) * n_per]))
                           for r in range(world)])
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-6 * float(np.abs(want).max()))
    assert rel_err(got, oracle.moe_forward(layer, h)) < TOL


def test_a_rank_that_never_arrives_costs_its_peers_a_timeout_status_not_the_gpu():
    """The barrier's wait is bounded: when a rank never signals, the waiting kernel gives up
    after the limit (5 ms here), records BIVMOE_ERR_TIMEOUT, and the stream goes on;
    bivmoe_status reports it once and the layer stays usable.  No fault, no hang: the flag
    the kernel polls is simply never written."""
    import time
    import torch
    from biv_b200 import capi
    from biv_b200.ep import DeviceSteps
    wl = _small("parity_q8_0", 8)
    layer = wl.layers[0]
    ranks = [DeviceSteps(layer, 4, r, 2, 0) for r in range(2)]
    try:
        infos = [st.peer_info() for st in ranks]
        for st in ranks:
            st.peer_attach(infos)
            st.peer_wait_limit(5_000)
        ranks[0].peer_signal()              # rank 1 never does
        t0 = time.perf_counter()
        ranks[0].peer_wait()
        with pytest.raises(capi.BivMoeError) as ei:
            ranks[0].status()
        assert ei.value.code == capi.ERR_TIMEOUT
        assert time.perf_counter() - t0 < 2.0
        ranks[0].status()                   # reported once, then clear
        # the late rank arrives: both are in step again (each has one barrier behind it)
        ranks[1].peer_signal()
        ranks[1].peer_wait()
        ranks[1].status()
        for st in ranks:
            st.peer_signal()
        for st in ranks:
            st.peer_wait()
        for st in ranks:
            st.status()
        torch.cuda.synchronize()
    finally:
        for st in ranks:
            st.close()


def _nccl_worker(rank, world, port, cfg, n, tmp):
    import torch
    import torch.distributed as dist
    from biv_b200.ep import EpMoe
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        wl = getattr(W, cfg)(n=n, **W.SMALL)
        layer, n_per = wl.layers[0], n // world
        h = np.ascontiguousarray(wl.h[rank * n_per:(rank + 1) * n_per])
        m = EpMoe(layer, n_per, rank, world, rank)
        hd = torch.from_numpy(h).cuda(rank)
        out = m.moe(hd)
        m.status()
        # the exchange by peer stores (blocks opened through CUDA IPC handles): same bits
        mp_ = EpMoe(layer, n_per, rank, world, rank, exchange="peer")
        for _ in range(2):
            outp = mp_.moe(hd)
        mp_.status()
        assert torch.equal(outp, out)
        dist.barrier()      # nobody unmaps a block a peer may still write to
        mp_.close()
        # and with the library's own barrier in place of the communicator's: the pass is
        # five library calls per rank, the ranks meet through flag words in their blocks
        ml = EpMoe(layer, n_per, rank, world, rank, exchange="peer", barrier="lib")
        for _ in range(3):
            outl = ml.moe(hd)
        ml.status()
        assert torch.equal(outl, out)
        dist.barrier()
        ml.close()
        np.save(os.path.join(tmp, f"out{rank}.npy"), out.cpu().numpy())
        # the same rows as two micro-batches in flight, each with its own layer object and stream
        half = n_per // 2
        parts = [EpMoe(layer, half, rank, world, rank) for _ in range(2)]
        streams = [torch.cuda.Stream() for _ in range(2)]
        out2 = torch.empty_like(hd)
        torch.cuda.synchronize()
        for _ in range(2):
            for i in range(2):
                with torch.cuda.stream(streams[i]):
                    parts[i].begin(hd[i * half:(i + 1) * half])
            for i in range(2):
                with torch.cuda.stream(streams[i]):
                    parts[i].finish(out2[i * half:(i + 1) * half], accumulate=False)
        torch.cuda.synchronize()
        for p_ in parts:
            p_.status()
            p_.close()
        assert torch.equal(out2, out)
        m.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg", ["parity_q8_0", "ep_bf16"])
def test_two_processes_over_nccl(cfg, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    n, world = 32, 2
    mp.spawn(_nccl_worker, args=(world, port, cfg, n, str(tmp_path)), nprocs=world, join=True)
    wl = getattr(W, cfg)(n=n, **W.SMALL)
    layer = wl.layers[0]
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    ref = oracle.moe_forward(layer, wl.h)
    assert rel_err(got, ref) < TOL
