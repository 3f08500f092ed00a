"""bivmoe_route_noalloc, the entry point for callers that cannot allocate device
memory (stream captures, foreign memory pools, latency-critical loops): its
scratch is an array built into the library instead of the layer's workspace.

Collected last on purpose: a run that stops at the first failure has then
already run every other test."""
import numpy as np
import pytest

from biv_b200 import capi, workloads as W

pytestmark = pytest.mark.gpu


def test_route_noalloc_matches_forward_twice_in_a_row():
    import torch
    from biv_b200.moe import Moe
    wl = W.decode_q4k(n=48, **W.SMALL)
    other = W.decode_q4k(n=48, seed=11, **W.SMALL)      # second call: different rows
    m = Moe(wl.layer, wl.n)
    try:
        k = wl.layer.n_expert_used
        ids = torch.empty(wl.n, k, dtype=torch.int32, device="cuda")
        wts = torch.empty(wl.n, k, dtype=torch.float32, device="cuda")
        for rows in (wl.h, other.h):
            h = torch.from_numpy(rows).cuda()
            m.moe(h)                                     # the existing entry point
            torch.cuda.synchronize()
            want_ids, want_w = m.tap(capi.TAP_IDS), m.tap(capi.TAP_WEIGHTS)
            ids.fill_(-1)
            wts.fill_(float("nan"))
            m.route_noalloc(h, ids, wts)                 # the one that allocates nothing
            torch.cuda.synchronize()
            # the same kernels on the same rows: integer ids exact, weights bit for bit
            assert np.array_equal(ids.cpu().numpy(), want_ids)
            assert np.array_equal(wts.cpu().numpy(), want_w)
    finally:
        m.close()


@pytest.mark.parametrize("n", [48, 300])
def test_route_noalloc_matches_the_oracle(n):
    """Against the CPU oracle's `route` on the oracle's own logits (not against the
    library): 48 rows take the router kernel that stages whole rows, 300 the one that
    moves K in chunks (from 256 rows on)."""
    import torch
    import oracle
    from biv_b200.moe import Moe
    from helpers import routing_mismatches
    wl = W.decode_q4k(n=n, **W.SMALL)
    _, tap = oracle.moe_forward(wl.layer, wl.h, level=oracle.host_level(), taps=True)
    m = Moe(wl.layer, wl.n)
    try:
        k = wl.layer.n_expert_used
        ids = torch.full((n, k), -1, dtype=torch.int32, device="cuda")
        wts = torch.full((n, k), float("nan"), dtype=torch.float32, device="cuda")
        m.route_noalloc(torch.from_numpy(wl.h).cuda(), ids, wts)
        torch.cuda.synchronize()
        got_ids, got_w = ids.cpu().numpy(), wts.cpu().numpy()
        assert not routing_mismatches(got_ids, tap["ids"], tap["logits"])
        same = (got_ids == tap["ids"]).all(axis=1)
        assert same.mean() > 0.99
        for t in np.nonzero(same)[0][:64]:      # and `route` itself, row by row
            want_ids, want_w = oracle.route(tap["logits"][t], k)
            assert np.array_equal(got_ids[t], want_ids)
            assert np.allclose(got_w[t], want_w, rtol=1e-5, atol=1e-7)
        assert np.allclose(got_w[same], tap["weights"][same], rtol=1e-5, atol=1e-7)
    finally:
        m.close()


def test_route_noalloc_without_rows_is_a_no_op_and_leaves_the_device_alone():
    import ctypes as C
    import torch
    from biv_b200.moe import Moe
    wl = W.decode_q4k(n=4, **W.SMALL)
    m = Moe(wl.layer, 4)
    try:
        # no rows: nothing to do, whatever the pointers (as the other entry points)
        capi.check(capi.lib().bivmoe_route_noalloc(m._h, None, 0, None, None, None), m._h)
        assert torch.cuda.current_device() == 0
    finally:
        m.close()


def test_route_noalloc_rejects_sizes_beyond_its_scratch():
    import torch
    from biv_b200.moe import Moe
    wl = W.decode_q4k(n=4, **W.SMALL)
    n_big = capi.ROUTE_NOALLOC_MAX_LOGITS // (wl.layer.n_expert + 1) + 1
    m = Moe(wl.layer, n_big)
    try:
        k = wl.layer.n_expert_used
        h = torch.zeros(n_big, wl.layer.n_embd, device="cuda")
        ids = torch.empty(n_big, k, dtype=torch.int32, device="cuda")
        wts = torch.empty(n_big, k, dtype=torch.float32, device="cuda")
        with pytest.raises(capi.BivMoeError) as ei:
            m.route_noalloc(h, ids, wts)
        assert ei.value.code == capi.ERR_ARGUMENT and "scratch" in str(ei.value)
        m.route_noalloc(h[: n_big - 1], ids[: n_big - 1], wts[: n_big - 1])   # the limit itself fits
        torch.cuda.synchronize()
    finally:
        m.close()
