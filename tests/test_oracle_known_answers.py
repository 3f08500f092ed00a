"""The reference's own known-answer tests for this path, restated against the
CPU oracle: this is what pins the oracle.

  engine/src/quant.rs:1652-1712  kernels_match_dequantized_dot
  engine/src/quant.rs:1566-1614  vnni_matches_avx2
  engine/src/quant.rs:1715-1738  bf16_and_f16
  engine/src/model.rs:1461-1474  route_picks_and_weighs
"""
import math

import numpy as np
import pytest

import oracle
from biv_b200 import workloads as W

MASK = (1 << 64) - 1


def rand_bytes(n, seed):
    """xorshift64 bytes, engine/src/quant.rs:1616-1625; returns (bytes, new seed)."""
    out = bytearray(n)
    for i in range(n):
        seed ^= (seed << 13) & MASK
        seed ^= seed >> 7
        seed ^= (seed << 17) & MASK
        out[i] = (seed >> 24) & 0xFF
    return np.frombuffer(bytes(out), dtype=np.uint8).copy(), seed


def rand_row(ty, n, seed):
    """engine/src/quant.rs:1628-1649: random blocks with f16 scales 0x2E66 (~0.1)."""
    be, bb = W._BLOCK[ty]
    b, seed = rand_bytes(W.row_size(ty, n), seed)
    blk = b.reshape(-1, bb)
    half = np.array([0x66, 0x2E], dtype=np.uint8)
    if ty in (W.Q8_0, W.Q4_0):
        blk[:, 0:2] = half
    elif ty == W.Q4_1:
        blk[:, 0:2] = half
        blk[:, 2:4] = np.array([0x66, 0xAE], dtype=np.uint8)   # ~-0.1
    elif ty in (W.Q4_K, W.Q5_K):
        blk[:, 0:2] = half
        blk[:, 2:4] = half
    elif ty == W.Q6_K:
        blk[:, 208:210] = half
    return blk.reshape(-1), seed


def probe_x(n=1024):
    i = np.arange(n, dtype=np.int64)
    return (((i * 7919) % 211).astype(np.float32) / np.float32(50.0) - np.float32(2.0))


LEVELS = [l for l in (0, 1, 2) if l <= oracle.host_level()]


def test_kernels_match_dequantized_dot():
    n = 1024
    x = probe_x(n)
    qs, d, s = oracle.q8_quantize(x)
    xd = (qs.astype(np.float32) * np.repeat(d, 32)).astype(np.float32)
    seed = 0x123456789ABCDEF1
    for ty in (W.Q4_0, W.Q4_1, W.Q8_0, W.Q4_K, W.Q5_K, W.Q6_K):
        w, seed = rand_row(ty, n, seed)
        wd = oracle.dequantize_row(ty, w, n)
        ref = np.float32(0)
        for a, b in zip(wd, xd):          # sequential f32 sum, as `.sum()` folds
            ref = np.float32(ref + np.float32(a * b))
        tol = 1e-3 * max(abs(float(ref)), 1.0)
        for level in LEVELS:
            got = oracle.dot(level, ty, w, x)
            assert abs(got - float(ref)) < tol, (W.TYPE_NAMES[ty], level, got, ref)
        # the reference's dot_x4 check: four scaled rows, same kernel per row
        for t in range(4):
            xt = (x * np.float32(t - 1.5)).astype(np.float32)
            one = oracle.dot(0, ty, w, xt)
            for level in LEVELS:
                assert abs(oracle.dot(level, ty, w, xt) - one) < tol


@pytest.mark.skipif(oracle.host_level() < 2, reason="host has no AVX-VNNI")
def test_vnni_matches_avx2():
    n = 1024
    x = probe_x(n)
    xs = []
    for t in range(4):
        v = x * np.float32(t - 1.5)
        idx = np.arange(n) % 5 == t
        v = np.where(idx, np.float32(1e3) * np.sign(x), v).astype(np.float32)
        xs.append(v)
    seed = 0x0BADCAFEDEADBEEF
    for ty in (W.Q4_0, W.Q4_1, W.Q8_0, W.Q4_K, W.Q5_K, W.Q6_K):
        w, seed = rand_row(ty, n, seed)
        if ty == W.Q8_0:
            w[2] = 0x80      # -128, the weight the sign trick cannot negate
        for xv in xs:
            a, b = oracle.dot(1, ty, w, xv), oracle.dot(2, ty, w, xv)
            assert np.float32(a).tobytes() == np.float32(b).tobytes(), (W.TYPE_NAMES[ty], a, b)


def test_bf16_and_f16():
    assert oracle.f16_to_f32(0x3C00) == 1.0
    assert oracle.f16_to_f32(0xC000) == -2.0
    assert oracle.f16_to_f32(0x0001) == 5.960464477539063e-8
    assert oracle.bf16_to_f32(0x3F80) == 1.0
    x = (np.arange(37, dtype=np.float32) * np.float32(0.25))
    want = float(np.sum(x.astype(np.float64) ** 2))
    w_bf16 = (x.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8)
    w_f32 = x.view(np.uint8)
    w_f16 = x.astype(np.float16).view(np.uint8)     # multiples of 1/4 below 512: exact in f16
    for level in LEVELS:
        lib = oracle.lib()
        got = lib.orc_dot(level, W.BF16, oracle._p(w_bf16), oracle._p(x), None, None, None, 37)
        assert abs(got - want) < 1e-3
        got = lib.orc_dot(level, W.F16, oracle._p(w_f16), oracle._p(x), None, None, None, 37)
        assert abs(got - want) < 1e-3
        got = lib.orc_dot(level, W.F32, oracle._p(w_f32), oracle._p(x), None, None, None, 37)
        assert abs(got - want) < 1e-3
        assert abs(oracle.dot_f32(level, x, x) - want) < 1e-3
        y = oracle.axpy(level, x, 2.0, x)
        assert np.array_equal(y, np.float32(3.0) * x)


def test_f16_conversion_matches_ieee_for_every_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    ok = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert ok.all()


def test_route_picks_and_weighs():
    l = np.array([math.log(2.0), 0.0, math.log(0.5), math.log(0.5)], dtype=np.float32)
    # the reference builds the logits as (ln p + 1) - 1 in f32
    l = ((np.array([np.log(np.float32(2.0)), 0, np.log(np.float32(0.5)), np.log(np.float32(0.5))],
                   dtype=np.float32) + np.float32(1.0)) - np.float32(1.0)).astype(np.float32)
    ids, w = oracle.route(l, 3)
    assert ids.tolist() == [0, 1, 2]        # the lower expert first among equals
    total = 0.5 + 0.25 + 0.125
    for wi, p in zip(w, (0.5, 0.25, 0.125)):
        assert abs(float(wi) - p / total) < 1e-6
    ids, w = oracle.route(l, 1)
    assert ids.tolist() == [0] and w.tolist() == [1.0]


def test_route_orders_non_finite_rows_like_total_cmp():
    """`route` sorts with f32::total_cmp (engine/src/model.rs:263), a total order: a row
    whose probabilities are all NaN (NaN or Inf activations) still yields k distinct, valid
    experts - the first k, the keys being equal - with NaN weights (`sum.max(2^-14)` passes
    a NaN sum over, and p / 2^-14 is NaN)."""
    for bad in (np.nan, np.inf, -np.inf):
        l = np.linspace(-1, 1, 16).astype(np.float32)
        l[5] = bad
        l[9] = -bad if np.isinf(bad) else bad     # +inf and -inf together: inf - inf is NaN
        ids, w = oracle.route(l, 4)
        if np.isnan(bad) or np.isinf(bad):
            assert ids.tolist() == [0, 1, 2, 3] and np.isnan(w).all(), (bad, ids, w)
    # one +inf alone is an ordinary maximum: p = 1 there (exp(inf - inf) is NaN, though:
    # the reference's softmax makes every p NaN as well)
    l = np.linspace(-1, 1, 16).astype(np.float32)
    l[7] = np.inf
    ids, w = oracle.route(l, 2)
    assert ids.tolist() == [0, 1] and np.isnan(w).all()
    # total_cmp ranks -0.0 below +0.0 and orders finite values as usual
    p = np.array([0.0, 3.0, -0.0, 3.0, 1.0], dtype=np.float32)
    ids, _ = oracle.route(p, 5)
    assert ids.tolist()[:2] == [1, 3]


def test_q4_generators_round_trip_through_the_reference_layouts():
    """The build's own Q4_0 / Q4_1 / F16 weight generators against the oracle's statement of
    the reference's dequantisation (engine/src/quant.rs:174-192): a value comes back within
    half a quantisation step of what went in."""
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((3, 256), dtype=np.float32) * np.float32(0.02))
    for ty, with_min in ((W.Q4_0, False), (W.Q4_1, True)):
        rows = W.quantize_q4(w, with_min)
        assert rows.shape == (3, W.row_size(ty, 256))
        for r in range(3):
            back = oracle.dequantize_row(ty, rows[r], 256)
            blk = w[r].reshape(-1, 32)
            step = ((blk.max(1) - blk.min(1)) / 15 if with_min else np.abs(blk).max(1) / 7)
            err = np.abs(back.reshape(-1, 32) - blk).max(1)
            # Q4_0 has no code for +8 steps: the block's positive extreme may clip by one step
            assert (err <= step * (0.51 if with_min else 1.01) + 1e-4 * step).all(), (ty, err / step)
    st = W.make_weights(rng, W.F16, 1, 2, 256)
    back = oracle.dequantize_row(W.F16, st.expert(0)[:512], 256)
    assert np.array_equal(back, st.expert(0)[:512].view(np.float16).astype(np.float32))
