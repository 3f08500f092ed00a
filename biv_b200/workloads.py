"""Seeded synthetic inputs for the qwen35moe MoE-FFN layer.

No GGUF model file is available where this library is built and measured, so
every weight tensor is generated: numpy ``default_rng(seed)`` (PCG64) streams
with the shapes, block formats and value distributions of the five benchmark
configurations.  The byte layouts are the GGUF ones the reference consumes
(engine/src/quant.rs:51-72 block sizes; 218-225 Q8_0; 286-346 Q4_K/Q5_K/Q6_K;
134-136 BF16), expert-major as ``Experts`` addresses them
(engine/src/model.rs:190-216: expert ``e`` starts at ``e*stride + offset``).

The reference has no weight quantiser (it only reads GGUF bytes), so the Q8_0
weight quantiser here is this library's own and is stated once:
``d32 = max|x|/127``, ``q = clamp(round_half_away(x/d32), -127, 127)``, stored
scale ``d = f16(d32)`` (round to nearest even).  Dots use the stored f16 ``d``.

The reference router has no bias term.  Where a configuration asks for biased
router logits, activation column 0 is the constant 1 and router column 0
carries the per-expert bias, so ``logit[e] = W[e,1:]·h[1:] + bias[e]`` exactly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

# ggml type ids (engine/src/quant.rs:30-48)
F32, F16, Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 3, 8, 12, 13, 14, 30
TYPE_NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q8_0: "Q8_0", Q4_K: "Q4_K",
              Q5_K: "Q5_K", Q6_K: "Q6_K", BF16: "BF16"}
_BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34),
          Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}


def row_size(ty: int, n: int) -> int:
    """Bytes of a row of ``n`` elements (engine/src/quant.rs:68-72)."""
    be, bb = _BLOCK[ty]
    if n % be:
        raise ValueError(f"{n} elements is not a whole number of {TYPE_NAMES[ty]} blocks")
    return n // be * bb


@dataclass
class ExpertStack:
    """A stack of same-shaped matrices, one per expert, in one byte tensor
    (mirrors ``Experts`` of engine/src/model.rs:190-204)."""
    ty: int
    cols: int
    rows: int
    n: int
    data: np.ndarray          # uint8, C-contiguous
    stride: int = 0           # bytes from one expert's matrix to the next
    offset: int = 0           # bytes from an expert's start to these rows

    def __post_init__(self):
        if not self.stride:
            self.stride = self.rows * row_size(self.ty, self.cols)
        assert self.data.dtype == np.uint8 and self.data.flags.c_contiguous
        assert self.data.size >= (self.n - 1) * self.stride + self.offset + self.matrix_bytes

    @property
    def matrix_bytes(self) -> int:
        return self.rows * row_size(self.ty, self.cols)

    def expert(self, e: int) -> np.ndarray:
        s = e * self.stride + self.offset
        return self.data[s:s + self.matrix_bytes]


@dataclass
class MoeLayer:
    """The tensors of one MoE feed-forward (mirrors ``Moe`` / ``SharedExpert`` /
    ``MoeConfig`` of engine/src/model.rs:57-66, 221-237)."""
    n_embd: int
    n_expert: int
    n_expert_used: int
    n_ff_exp: int
    n_ff_shexp: int
    router: np.ndarray                      # f32 [n_expert, n_embd]
    gate: ExpertStack
    up: ExpertStack
    down: ExpertStack
    sh_gate: Optional[ExpertStack] = None   # n = 1
    sh_up: Optional[ExpertStack] = None
    sh_down: Optional[ExpertStack] = None
    sh_gate_inp: Optional[np.ndarray] = None  # f32 [n_embd]

    @property
    def has_shared(self) -> bool:
        return self.sh_gate is not None

    def weight_bytes(self, experts_hit: Optional[int] = None) -> int:
        """Bytes of the weights one pass must read when ``experts_hit`` distinct
        experts are selected (all of them when None)."""
        hit = self.n_expert if experts_hit is None else experts_hit
        per = self.gate.matrix_bytes + self.up.matrix_bytes + self.down.matrix_bytes
        b = hit * per + self.router.nbytes
        if self.has_shared:
            b += (self.sh_gate.matrix_bytes + self.sh_up.matrix_bytes
                  + self.sh_down.matrix_bytes + self.sh_gate_inp.nbytes)
        return b


@dataclass
class Workload:
    name: str
    seed: int
    layers: list                # list[MoeLayer]; one entry except for the stack
    h: np.ndarray               # f32 [n, n_embd]: layer input (or residual x0 for a stack)
    norm_w: Optional[list] = None   # per-layer rms_norm weights for a stack
    eps: float = 1e-6
    notes: dict = field(default_factory=dict)

    @property
    def layer(self) -> MoeLayer:
        return self.layers[0]

    @property
    def n(self) -> int:
        return self.h.shape[0]


# --------------------------------------------------------------------------
# element codecs

def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, as a model converter would."""
    b = np.asarray(x, dtype=np.float32).view(np.uint32)
    r = ((b >> 16) & 1) + 0x7FFF
    return ((b + r) >> 16).astype(np.uint16)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32 [..., cols] -> Q8_0 bytes [..., cols/32*34] with this library's stated
    convention (module docstring)."""
    x = np.asarray(x, dtype=np.float32)
    lead, cols = x.shape[:-1], x.shape[-1]
    xb = x.reshape(-1, cols // 32, 32)
    amax = np.abs(xb).max(axis=-1, keepdims=True)
    d32 = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = np.where(d32 != 0, xb / d32, np.float32(0)).astype(np.float32)
    q = np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))
    q = np.clip(q, -127, 127).astype(np.int8)
    out = np.empty(xb.shape[:2] + (34,), dtype=np.uint8)
    out[..., 0:2] = f32_to_f16_bits(d32[..., 0])[..., None].view(np.uint8).reshape(
        xb.shape[0], xb.shape[1], 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(lead + (cols // 32 * 34,))


def quantize_q4(w: np.ndarray, with_min: bool) -> np.ndarray:
    """Rows of f32 as Q4_0 (``with_min`` false: ``d = amax/7``, nibble = ``round(x/d) + 8``)
    or Q4_1 (``d = (max - min)/15``, ``m = min``, nibble = ``round((x - m)/d)``) blocks; byte
    j of a block holds element j in its low half and element j + 16 in its high half
    (engine/src/quant.rs:174-192).  The reference only reads these formats: the
    quantiser is this module's own."""
    w = np.asarray(w, dtype=np.float32)
    lead, cols = w.shape[:-1], w.shape[-1]
    xb = w.reshape(-1, cols // 32, 32)
    if with_min:
        lo, hi = xb.min(axis=-1, keepdims=True), xb.max(axis=-1, keepdims=True)
        d32 = (hi - lo) / np.float32(15.0)
        off = lo
    else:
        d32 = np.abs(xb).max(axis=-1, keepdims=True) / np.float32(7.0)
        off = np.float32(-8.0) * d32
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d32 > 0, np.rint((xb - off) / d32), 0.0)
    q = np.clip(q, 0, 15).astype(np.uint8)
    head = 4 if with_min else 2
    out = np.empty(xb.shape[:2] + (head + 16,), dtype=np.uint8)
    out[..., 0:2] = f32_to_f16_bits(d32[..., 0])[..., None].view(np.uint8).reshape(
        xb.shape[0], xb.shape[1], 2)
    if with_min:
        out[..., 2:4] = f32_to_f16_bits(off[..., 0])[..., None].view(np.uint8).reshape(
            xb.shape[0], xb.shape[1], 2)
    out[..., head:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(lead + (cols // 32 * (head + 16),))


def _random_bytes(rng: np.random.Generator, n: int) -> np.ndarray:
    return np.frombuffer(rng.bytes(n), dtype=np.uint8).copy()


def random_kquant(rng: np.random.Generator, ty: int, n_rows: int, cols: int,
                  d_lo: float = 1e-3, d_hi: float = 5e-3, fast: bool = False) -> np.ndarray:
    """Random k-quant rows: uniform quant bits and packed 6-bit (or int8) sub-block
    scales, f16 ``d`` (and ``dmin``) drawn from U(d_lo, d_hi).  ``fast`` draws the bytes
    with ``rng.integers`` (an order of magnitude quicker than ``rng.bytes``, a different
    stream of the same distribution)."""
    be, bb = _BLOCK[ty]
    nblk = n_rows * (cols // be)
    if fast:
        raw = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)
    else:
        raw = _random_bytes(rng, nblk * bb).reshape(nblk, bb)
    d = f32_to_f16_bits(rng.uniform(d_lo, d_hi, nblk).astype(np.float32))
    if ty in (Q4_K, Q5_K):
        dmin = f32_to_f16_bits(rng.uniform(d_lo, d_hi, nblk).astype(np.float32))
        raw[:, 0:2] = d[:, None].view(np.uint8)
        raw[:, 2:4] = dmin[:, None].view(np.uint8)
    elif ty == Q6_K:
        raw[:, 208:210] = d[:, None].view(np.uint8)
    else:
        raise ValueError("not a k-quant on this path")
    return raw.reshape(n_rows, cols // be * bb)


def _stack(ty, cols, rows, n, data) -> ExpertStack:
    return ExpertStack(ty, cols, rows, n, np.ascontiguousarray(data.reshape(-1)))


def make_weights(rng, ty: int, n: int, rows: int, cols: int, sigma: float = 0.02,
                 fast: bool = False) -> ExpertStack:
    """``n`` matrices [rows, cols] of type ``ty``: N(0, sigma) values for Q8_0, Q4_0,
    Q4_1, BF16, F16 and F32; random blocks for the k-quants."""
    if ty in (Q4_K, Q5_K, Q6_K):
        return _stack(ty, cols, rows, n, random_kquant(rng, ty, n * rows, cols, fast=fast))
    rb = row_size(ty, cols)
    out = np.empty((n, rows * rb), dtype=np.uint8)
    for e in range(n):      # one expert at a time keeps the f32 temporary small
        w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(sigma)
        if ty == Q8_0:
            out[e] = quantize_q8_0(w).reshape(-1)
        elif ty in (Q4_0, Q4_1):
            out[e] = quantize_q4(w, ty == Q4_1).reshape(-1)
        elif ty == BF16:
            out[e] = f32_to_bf16_bits(w).view(np.uint8).reshape(-1)
        elif ty == F16:
            out[e] = w.astype(np.float16).view(np.uint8).reshape(-1)
        elif ty == F32:
            out[e] = w.view(np.uint8).reshape(-1)
        else:
            raise ValueError(f"no generator for type {ty}")
    return _stack(ty, cols, rows, n, out)


def make_layer(rng, *, n_embd=2048, n_expert=256, k=8, ff=512, ff_sh=512,
               gate_ty=Q8_0, up_ty=None, down_ty=None, router_bias=None,
               router_dist="normal", fast=False) -> MoeLayer:
    up_ty = gate_ty if up_ty is None else up_ty
    down_ty = gate_ty if down_ty is None else down_ty
    if router_dist == "uniform":   # same standard deviation as N(0, 0.02)
        a = 0.02 * np.sqrt(3.0)
        router = rng.uniform(-a, a, (n_expert, n_embd)).astype(np.float32)
    else:
        router = rng.standard_normal((n_expert, n_embd), dtype=np.float32) * np.float32(0.02)
    if router_bias is not None:
        router[:, 0] = np.asarray(router_bias, dtype=np.float32)
    layer = MoeLayer(
        n_embd, n_expert, k, ff, ff_sh, router,
        gate=make_weights(rng, gate_ty, n_expert, ff, n_embd, fast=fast),
        up=make_weights(rng, up_ty, n_expert, ff, n_embd, fast=fast),
        down=make_weights(rng, down_ty, n_expert, n_embd, ff, fast=fast))
    if ff_sh:
        layer.sh_gate = make_weights(rng, gate_ty, 1, ff_sh, n_embd, fast=fast)
        layer.sh_up = make_weights(rng, up_ty, 1, ff_sh, n_embd, fast=fast)
        layer.sh_down = make_weights(rng, down_ty, 1, n_embd, ff_sh, fast=fast)
        layer.sh_gate_inp = rng.standard_normal(n_embd, dtype=np.float32) * np.float32(0.02)
    return layer


def rms_normalise(x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    ss = (x.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    return (x / np.sqrt(ss + eps)).astype(np.float32)


# --------------------------------------------------------------------------
# the five benchmark configurations (shapes can be shrunk for CPU-sized tests)

ZIPF_ALPHA = 1.25   # scale of the Zipf(1.1) logit bias of the prefill configuration


def parity_q8_0(n=16, seed=0, **shape) -> Workload:
    """Configuration 1: 16 tokens, RMS-normalised N(0,1) rows, everything Q8_0."""
    rng = np.random.default_rng(seed)
    layer = make_layer(rng, gate_ty=Q8_0, **shape)
    h = rms_normalise(rng.standard_normal((n, layer.n_embd), dtype=np.float32))
    return Workload("parity_q8_0", seed, [layer], h)


def decode_q4k(n=64, seed=1, **shape) -> Workload:
    """Configuration 2: 64 single-token sequences, Q4_K experts, router logits
    skewed by a per-expert bias N(0,1)."""
    rng = np.random.default_rng(seed)
    n_expert = shape.get("n_expert", 256)
    bias = rng.standard_normal(n_expert).astype(np.float32)
    layer = make_layer(rng, gate_ty=Q4_K, router_bias=bias, **shape)
    h = rng.standard_normal((n, layer.n_embd), dtype=np.float32)
    h[:, 0] = 1.0
    return Workload("decode_q4k", seed, [layer], h, notes={"router_bias": "N(0,1)"})


def prefill_q8_0(n=4096, seed=2, alpha=ZIPF_ALPHA, **shape) -> Workload:
    """Configuration 3: 4096 tokens, Q8_0 experts, expert popularity Zipf(1.1):
    logit bias ``alpha * ln(rank^-1.1)`` over a seeded permutation of the experts."""
    rng = np.random.default_rng(seed)
    n_expert = shape.get("n_expert", 256)
    rank = rng.permutation(n_expert) + 1
    bias = (alpha * -1.1 * np.log(rank)).astype(np.float32)
    layer = make_layer(rng, gate_ty=Q8_0, router_bias=bias, **shape)
    h = rng.standard_normal((n, layer.n_embd), dtype=np.float32)
    h[:, 0] = 1.0
    return Workload("prefill_q8_0", seed, [layer], h,
                    notes={"router_bias": f"{alpha}*ln(rank^-1.1)"})


def mtp_stack(n_seq=32, n_tok=5, n_layers=40, seed=3, **shape) -> Workload:
    """Configuration 4: a stack of MoE FFN layers (gate/up Q5_K, down Q6_K) over
    32 sequences x 5 tokens, residual carried, rms_norm (weight 1) before each."""
    rng = np.random.default_rng(seed)
    layers = [make_layer(rng, gate_ty=Q5_K, down_ty=Q6_K, **shape) for _ in range(n_layers)]
    e = layers[0].n_embd
    x0 = rng.standard_normal((n_seq * n_tok, e), dtype=np.float32)
    return Workload("mtp_stack", seed, layers, x0,
                    norm_w=[np.ones(e, dtype=np.float32) for _ in range(n_layers)])


def mtp_stack_layer(l: int, seed=3, **shape):
    """Layer ``l`` of the streamed stack (``mtp_stack_streamed``): ``(MoeLayer, norm_w)``
    from the layer's own stream ``default_rng([seed, l])``."""
    rng = np.random.default_rng([seed, l])
    layer = make_layer(rng, gate_ty=Q5_K, down_ty=Q6_K, fast=True, **shape)
    return layer, np.ones(layer.n_embd, dtype=np.float32)


def mtp_stack_streamed(n_seq=32, n_tok=5, n_layers=40, seed=3, **shape):
    """Configuration 4 one layer at a time, for hosts that should not hold 40 layers of
    random weights (0.6 GB each) at once: returns ``(x0, eps, layers)`` where ``layers``
    yields ``(MoeLayer, norm_w)``.  Layer ``l`` comes from its own stream
    ``default_rng([seed, l])`` (``mtp_stack_layer``; layers can be built in any order, or
    on several host threads) and the rows from ``default_rng([seed, 1 << 20])``; the values
    differ from ``mtp_stack``'s, the distributions do not."""
    e = shape.get("n_embd", 2048)
    x0 = np.random.default_rng([seed, 1 << 20]).standard_normal((n_seq * n_tok, e), dtype=np.float32)
    return x0, 1e-6, (mtp_stack_layer(l, seed, **shape) for l in range(n_layers))


def ep_bf16(n=16384, seed=4, **shape) -> Workload:
    """Configuration 5: BF16 experts, uniform-random router so the load is
    balanced; the expert-parallel configuration."""
    rng = np.random.default_rng(seed)
    layer = make_layer(rng, gate_ty=BF16, router_dist="uniform", **shape)
    h = rng.standard_normal((n, layer.n_embd), dtype=np.float32)
    return Workload("ep_bf16", seed, [layer], h)


def typed_layer(gate_ty, down_ty=None, n=16, seed=5, **shape) -> Workload:
    """One layer of any weight types the reference has dot kernels for
    (engine/src/quant.rs:80-93), N(0, 1) rows normalised like configuration 1."""
    rng = np.random.default_rng(seed)
    layer = make_layer(rng, gate_ty=gate_ty, down_ty=down_ty, **shape)
    h = rms_normalise(rng.standard_normal((n, layer.n_embd), dtype=np.float32))
    name = f"typed_{TYPE_NAMES[gate_ty]}_{TYPE_NAMES[layer.down.ty]}"
    return Workload(name, seed, [layer], h)


CONFIGS = {"parity_q8_0": parity_q8_0, "decode_q4k": decode_q4k, "prefill_q8_0": prefill_q8_0,
           "mtp_stack": mtp_stack, "ep_bf16": ep_bf16}

# a shape every generator accepts, small enough for CPU-only tests
SMALL = dict(n_embd=256, n_expert=16, k=4, ff=256, ff_sh=256)
