"""Regenerates tests/golden/*.npz.

The reference is Rust and cannot be run where these fixtures were made, and
its own tests hold no vector for the whole layer, so the fixtures are outputs
of the CPU oracle at its scalar level (the restatement of the reference's
`scalar::*` kernels, engine/src/quant.rs:563-687) on seeded inputs that
`biv_b200.workloads` regenerates from the recorded arguments.  They pin the
oracle against drift and give the GPU tests a committed answer to meet.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from biv_b200 import workloads as W  # noqa: E402

CASES = {
    "parity_q8_0_small": ("parity_q8_0", dict(n=12)),
    "decode_q4k_small": ("decode_q4k", dict(n=24)),
    "prefill_q8_0_small": ("prefill_q8_0", dict(n=96)),
    "ep_bf16_small": ("ep_bf16", dict(n=20)),
    "kquant_mix_small": ("mtp_stack", dict(n_seq=5, n_tok=3, n_layers=1)),
}


def build(name):
    cfg, kw = CASES[name]
    return W.CONFIGS[cfg](**kw, **W.SMALL)


def main():
    for name in CASES:
        wl = build(name)
        out, tap = oracle.moe_forward(wl.layer, wl.h, level=0, taps=True)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), out=out, ids=tap["ids"], weights=tap["weights"],
            order=tap["order"], counts=tap["counts"], logits=tap["logits"], act_q=tap["act_q"],
            h_checksum=np.frombuffer(wl.h.tobytes(), np.uint32).sum(dtype=np.uint64),
            w_checksum=np.uint64(int(wl.layer.gate.data.astype(np.uint64).sum())
                                 + int(wl.layer.down.data.astype(np.uint64).sum())))
        print(name, out.shape, float(np.abs(out).max()))


if __name__ == "__main__":
    main()
