"""Shared test helpers: the error metric of the parity gate, a routing
comparison that honours the stated tie exception, and an independent numpy
float64 statement of the layer used to cross-check the oracle's structure."""
import numpy as np

import oracle
from biv_b200 import workloads as W

FLOAT_TYPES = (W.F32, W.F16, W.BF16)


def rel_err(got, ref):
    """The parity gate's metric: max_i |got_i - ref_i| / max(|ref_i|, rms(ref)).
    The floor rms(ref) keeps outputs that cross zero from dominating."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    floor = max(float(np.sqrt(np.mean(ref ** 2))), 1e-30)
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), floor)))


def loose_err(got, ref):
    """The looser companion figure: ||got - ref||_inf / ||ref||_inf."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(got - ref)) / max(float(np.max(np.abs(ref))), 1e-30))


def routing_mismatches(ids_got, ids_ref, logits_ref, tie=1e-6):
    """Tokens whose expert lists differ for a reason other than a router-logit
    tie closer than `tie`: ids must be equal position by position, except that a
    differing position is excused when the two experts' reference logits are
    within `tie` of each other."""
    bad = []
    for t in range(ids_ref.shape[0]):
        if np.array_equal(ids_got[t], ids_ref[t]):
            continue
        for a, b in zip(ids_got[t], ids_ref[t]):
            if a != b and abs(float(logits_ref[t, a]) - float(logits_ref[t, b])) >= tie:
                bad.append(t)
                break
    return bad


def dequant_matrix(st, e):
    rb = W.row_size(st.ty, st.cols)
    m = st.expert(e).reshape(st.rows, rb)
    return np.stack([oracle.dequantize_row(st.ty, m[r], st.cols) for r in range(st.rows)]
                    ).astype(np.float64)


def _act(x, ty):
    """What the reference multiplies weights of type `ty` with: the f32 rows for
    float types, the dequantised Q8 rows otherwise."""
    if ty in FLOAT_TYPES:
        return x.astype(np.float64)
    qs, d, _ = oracle.q8_quantize(x.astype(np.float32))
    return qs.astype(np.float64) * np.repeat(d.astype(np.float64), 32, axis=-1)


def _ffn64(gate, up, down, e, x):
    g = _act(x, gate.ty) @ dequant_matrix(gate, e).T
    u = _act(x, up.ty) @ dequant_matrix(up, e).T
    g32, u32 = g.astype(np.float32), u.astype(np.float32)
    mid = (g32 / (1 + np.exp(-g32.astype(np.float64))) * u32).astype(np.float32)
    return _act(mid, down.ty) @ dequant_matrix(down, e).T


def layer_float64(layer, h, ids, weights):
    """The layer in float64 on dequantised operands, with the routing given."""
    n, k = ids.shape
    out = np.zeros((n, layer.n_embd))
    for e in range(layer.n_expert):
        toks, js = np.nonzero(ids == e)
        if toks.size == 0:
            continue
        y = _ffn64(layer.gate, layer.up, layer.down, e, h[toks])
        out[toks] += weights[toks, js][:, None].astype(np.float64) * y
    if layer.has_shared:
        y = _ffn64(layer.sh_gate, layer.sh_up, layer.sh_down, 0, h)
        g = h.astype(np.float64) @ layer.sh_gate_inp.astype(np.float64)
        out += (1 / (1 + np.exp(-g)))[:, None] * y
    return out
