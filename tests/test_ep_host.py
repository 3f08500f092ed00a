"""Expert parallelism, host side: two gloo ranks on the CPU run ``ep_pass`` (the
count exchange, the split sizes, the two all-to-alls, the order in which rows
travel and return) with the oracle standing in for the device steps, and must
reproduce the single-process oracle on each rank's rows up to the association of
the f32 sum over a token's experts (by rank first)."""
import os
import socket

import numpy as np
import pytest

import oracle
from biv_b200 import workloads as wl
from biv_b200.ep import TorchComm, ep_pass, ep_pass_peer, ep_plan, local_experts

torch = pytest.importorskip("torch")


class OracleSteps:
    """The steps of ``ep_pass`` restated on numpy rows with the CPU oracle."""

    def __init__(self, layer, rank, world):
        self.layer, self.rank, self.world = layer, rank, world
        self.n_expert, self.k, self.n_embd = layer.n_expert, layer.n_expert_used, layer.n_embd
        self.local = local_experts(layer, rank, world)
        self.level = oracle.host_level()

    def route(self, h):
        hn = h.numpy()
        _, tap = oracle.moe_forward(self.layer, hn, taps=True)
        self.tap, self.n = tap, hn.shape[0]
        nl = self.n_expert // self.world
        dest = tap["ids"] // nl                                   # [n][k]
        rows, tags, counts, self.where = [], [], [], {}
        for d in range(self.world):                               # grouped by rank, token order inside
            toks = np.nonzero((dest == d).any(axis=1))[0]
            for t in toks:
                self.where[(int(t), d)] = len(rows)
                rows.append(hn[t])
                tags.append(np.concatenate([tap["ids"][t].astype(np.int32),
                                            tap["weights"][t].view(np.int32)]))
            counts.append(len(toks))
        rows = np.array(rows, np.float32).reshape(-1, self.n_embd)
        tags = np.array(tags, np.int32).reshape(-1, 2 * self.k)
        return torch.from_numpy(rows), torch.from_numpy(tags), torch.tensor(counts, dtype=torch.int32)

    def shared(self, h):
        pass   # the tap of route() already holds the shared expert's rows

    def rows(self, count):
        return torch.empty((count, self.n_embd), dtype=torch.float32)

    def tags(self, count):
        return torch.empty((count, 2 * self.k), dtype=torch.int32)

    def experts(self, recv_rows, recv_tags, m):
        rows, tags = recv_rows.numpy(), recv_tags.numpy()
        nl = self.n_expert // self.world
        out = np.zeros_like(rows)
        for i in range(m):
            ids, wts = tags[i, :self.k], tags[i, self.k:].view(np.float32)
            mine = [(int(e), float(w)) for e, w in zip(ids, wts) if e // nl == self.rank]
            assert mine, "a row arrived that has no expert here"
            for e, w in sorted(mine):                              # ascending expert id
                out[i] = oracle.axpy(self.level, out[i], w, self._ffn(e - self.rank * nl, rows[i:i + 1])[0])
        return torch.from_numpy(out)

    def _ffn(self, x, rows):
        """silu(gate x) * (up x) -> down of local expert x, through the oracle's layer
        with that one expert: its routing weight is exactly one."""
        L = self.local

        def one(st):
            return wl.ExpertStack(st.ty, st.cols, st.rows, 1, st.data, st.stride, st.offset + x * st.stride)
        sub = wl.MoeLayer(L.n_embd, 1, 1, L.n_ff_exp, 0, np.zeros((1, L.n_embd), np.float32),
                          one(L.gate), one(L.up), one(L.down))
        return oracle.moe_forward(sub, rows)

    @staticmethod
    def _sigmoid(g):
        """ops.rs:160-162, with the C library's expf as the oracle uses it."""
        import ctypes
        f = oracle.lib().orc_sigmoid
        f.restype, f.argtypes = ctypes.c_float, [ctypes.c_float]
        return f(float(g))

    def combine(self, returned, out, accumulate):
        ret, tap = returned.numpy(), self.tap
        res = np.zeros((self.n, self.n_embd), np.float32)
        for t in range(self.n):
            for d in range(self.world):                            # ascending rank
                if (t, d) in self.where:
                    res[t] = oracle.axpy(self.level, res[t], 1.0, ret[self.where[(t, d)]])
            if self.layer.has_shared:
                res[t] = oracle.axpy(self.level, res[t], float(self._sigmoid(tap["shared_gate"][t])),
                                     tap["shared_out"][t])
        o = out.numpy()
        o[...] = o + res if accumulate else res


class OraclePeerSteps(OracleSteps):
    """The steps of ``ep_pass_peer`` on the CPU: every rank's exchange block is a set of
    shared-memory tensors that the other rank's process writes into, split in regions of
    ``cap`` rows per source rank exactly as the library's device blocks are."""

    def __init__(self, layer, rank, world, blocks, cap):
        super().__init__(layer, rank, world)
        self.blocks, self.cap = blocks, cap

    def peer_dispatch(self, h):
        rows, tags, counts = self.route(h)              # grouped by rank, token order inside
        at = 0
        for d in range(self.world):
            c = int(counts[d])
            assert c <= self.cap
            blk = self.blocks[d]                        # stores into rank d's block, region [me]
            blk["rows"][self.rank, :c] = rows[at:at + c]
            blk["tags"][self.rank, :c] = tags[at:at + c]
            blk["counts"][self.rank] = c
            at += c
        self.base = np.concatenate([[0], np.cumsum(counts.numpy())])

    def peer_experts(self):
        mine = self.blocks[self.rank]
        for src in range(self.world):
            c = int(mine["counts"][src])                # rows past the count have no experts
            if c:
                out = self.experts(mine["rows"][src, :c], mine["tags"][src, :c], c)
                self.blocks[src]["returned"][self.rank, :c] = out   # region [me] of the home's block

    def peer_barrier(self, limit_s=20.0):
        """The library's barrier restated on the shared-memory blocks: barrier number e
        (every rank counts its own barriers, the numbers are never exchanged) is signalled
        by storing e into word [my rank] of every rank's flag array, and waited for by
        polling this rank's own array until every word has reached e - with a time limit."""
        import time
        self.epoch = getattr(self, "epoch", 0) + 1
        for d in range(self.world):
            self.blocks[d]["flags"][self.rank] = self.epoch
        t0 = time.monotonic()
        mine = self.blocks[self.rank]["flags"]
        while int(mine.min()) < self.epoch:
            assert time.monotonic() - t0 < limit_s, "a rank never reached the barrier"
            time.sleep(0.0005)

    def peer_combine(self, out, accumulate):
        ret = self.blocks[self.rank]["returned"]
        packed = torch.cat([ret[d, :int(self.base[d + 1] - self.base[d])] for d in range(self.world)])
        self.combine(packed, out, accumulate)


class GlooComm(TorchComm):
    def barrier(self, device):
        import torch.distributed as dist
        dist.barrier()


def _peer_worker(rank, world, port, cfg, rows_per_rank, cap, blocks, lib_barrier=False):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_all = sum(rows_per_rank)
        w = getattr(wl, cfg)(n=n_all, **wl.SMALL)
        layer = w.layers[0]
        lo = sum(rows_per_rank[:rank])
        h = np.ascontiguousarray(w.h[lo:lo + rows_per_rank[rank]])
        steps = OraclePeerSteps(layer, rank, world, blocks, cap)
        out = torch.zeros((h.shape[0], layer.n_embd), dtype=torch.float32)
        for _ in range(3):      # several times: the regions are reused, the second barrier frees them
            ep_pass_peer(steps, torch.from_numpy(h), out, False, GlooComm(), lib_barrier=lib_barrier)
        want = oracle.moe_forward(layer, h)
        np.testing.assert_allclose(out.numpy(), want, rtol=0, atol=4e-7 * float(np.abs(want).max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg,rows_per_rank,lib_barrier", [("parity_q8_0", (12, 12), False),
                                                          ("ep_bf16", (9, 3), False),
                                                          ("decode_q4k", (5, 11), True)])
def test_two_gloo_ranks_exchange_through_each_others_blocks(cfg, rows_per_rank, lib_barrier):
    import torch.multiprocessing as mp
    world, cap = 2, 16      # regions larger than any rank's rows: the rest is padding
    layer = getattr(wl, cfg)(n=4, **wl.SMALL).layers[0]
    e, k = layer.n_embd, layer.n_expert_used
    blocks = [{"rows": torch.zeros((world, cap, e)).share_memory_(),
               "returned": torch.zeros((world, cap, e)).share_memory_(),
               "tags": torch.zeros((world, cap, 2 * k), dtype=torch.int32).share_memory_(),
               "counts": torch.zeros((world,), dtype=torch.int32).share_memory_(),
               "flags": torch.zeros((world,), dtype=torch.int32).share_memory_()} for _ in range(world)]
    mp.spawn(_peer_worker, args=(world, _free_port(), cfg, rows_per_rank, cap, blocks, lib_barrier),
             nprocs=world, join=True)


def _worker(rank, world, port, cfg, n_per_rank):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = getattr(wl, cfg)(n=world * n_per_rank, **wl.SMALL)
        layer = w.layers[0]
        h = np.ascontiguousarray(w.h[rank * n_per_rank:(rank + 1) * n_per_rank])
        steps = OracleSteps(layer, rank, world)
        out = torch.zeros((n_per_rank, layer.n_embd), dtype=torch.float32)
        plan = ep_pass(steps, torch.from_numpy(h), out, False)
        want = oracle.moe_forward(layer, h)
        assert plan.m == sum(plan.recv_splits)
        assert n_per_rank <= sum(plan.send_splits) <= n_per_rank * min(world, layer.n_expert_used)
        # the sum over a token's experts is associated by rank first: f32 rounding apart
        np.testing.assert_allclose(out.numpy(), want, rtol=0, atol=4e-7 * float(np.abs(want).max()))
        # every row sent is a row received
        total = torch.tensor([plan.m - sum(plan.send_splits)])
        dist.all_reduce(total)
        assert int(total) == 0
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("cfg", ["parity_q8_0", "ep_bf16"])
def test_two_gloo_ranks_reproduce_the_single_process_oracle(cfg):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), cfg, 12), nprocs=2, join=True)


def test_plan_is_consistent_across_ranks():
    rng = np.random.default_rng(0)
    W = 4
    counts = rng.integers(0, 9, size=(W, W)).astype(np.int32)
    counts[1, 2] = 0                                         # rank 1 sends nothing to rank 2
    plans = [ep_plan(counts, r) for r in range(W)]
    for r in range(W):
        assert sum(plans[r].send_splits) == counts[r].sum()
        for d in range(W):
            assert plans[r].send_splits[d] == plans[d].recv_splits[r]
        assert plans[r].m == counts[:, r].sum()
    assert plans[2].recv_splits[1] == 0


def test_local_experts_are_a_byte_range_of_the_same_tensor():
    layer = wl.parity_q8_0(n=4, **wl.SMALL).layers[0]
    for r in range(4):
        loc = local_experts(layer, r, 4)
        assert loc.gate.data is layer.gate.data and loc.gate.n == layer.n_expert // 4
        for x in range(loc.gate.n):
            np.testing.assert_array_equal(loc.down.expert(x), layer.down.expert(r * loc.gate.n + x))
