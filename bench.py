#!/usr/bin/env python
"""Benchmark of the qwen35moe MoE feed-forward layer on B200.

One "step" is one pass of the layer over one batch of synthetic rows (generated from
a seed; there is no dataset).  The headline workload at every N is the expert-parallel
configuration (BASELINE.json configs[4]): 16 384 tokens, BF16 experts, balanced
routing; at N = 1 the whole layer on one GPU, at N > 1 the experts sharded 256 / N per
GPU and the 16 384 rows split over the ranks (strong scaling), rows exchanged by the
library's own peer stores over NVLink (or NCCL all-to-alls, --ep-exchange).  `value`
is one pass at a time.  At N = 1 the line also carries the other configurations as
side objects - `decode` (configs[1]), `prefill` (configs[2]), `stack` (configs[3]) -
each with its roofline and its parity against the CPU oracle.  Prints ONE JSON line
(rank 0).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
  python bench.py --impl reference ...   # the CPU restatement of the reference's kernels
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from biv_b200 import workloads as W  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
MIN_TIMED_MS = 50.0     # the K-step loop is repeated until this much device time is covered
CPU_SAMPLE_TOKENS = 512  # rows of the headline workload the CPU arm times (scaled linearly)
GATE, FLIP_GATE = 1e-3, 1e-2

DTYPES = {
    "ep_bf16": "bf16 weights x f32 activations (two bf16 terms on the tensor core), f32 accumulation",
    "decode_q4k": "int8 x int8 -> int32 block dots, f32 scales",
    "prefill_q8_0": "int8 x int8 -> int32 block dots, f32 scales",
    "parity_q8_0": "int8 x int8 -> int32 block dots, f32 scales",
    "mtp_stack": "int8 x int8 -> int32 block dots, f32 scales",
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"], d.get("bf16_tflops"), "measured"
    return 6650.0, 1590.0, "fallback"


def make_workload(name, tokens=0):
    if name == "decode_q4k":
        return W.decode_q4k(n=tokens or 64)
    if name == "parity_q8_0":
        return W.parity_q8_0(n=tokens or 16)
    if name == "prefill_q8_0":
        return W.prefill_q8_0(n=tokens or 4096)
    if name == "ep_bf16":
        return W.ep_bf16(n=tokens or 16384)
    raise SystemExit(f"unknown workload {name}")


def describe(wl, world=1):
    l = wl.layer
    return (f"{wl.name}: {wl.n} tokens, hidden {l.n_embd}, {l.n_expert} experts top-{l.n_expert_used} + shared "
            f"expert, ff {l.n_ff_exp}, gate/up {W.TYPE_NAMES[l.gate.ty]} down {W.TYPE_NAMES[l.down.ty]}, "
            f"seed {wl.seed}")


def algorithmic_bytes(layer, n, experts_hit):
    """Bytes one pass must move at least: every selected expert's weights once,
    the shared expert, the router and gate vector, the rows in and out."""
    return layer.weight_bytes(experts_hit) + 2 * n * layer.n_embd * 4


def gateup_bytes(layer, n, experts_hit):
    """The dominant kernel of the decode shape (gate+up with SwiGLU): gate and up matrices
    of every selected expert and of the shared expert once, the Q8 rows of h once per
    (token, expert) pair, the f32 mid rows written."""
    k, e, ff = layer.n_expert_used, layer.n_embd, layer.n_ff_exp
    w = experts_hit * (layer.gate.matrix_bytes + layer.up.matrix_bytes)
    pairs = n * k
    if layer.has_shared:
        w += layer.sh_gate.matrix_bytes + layer.sh_up.matrix_bytes
        pairs += n
    quant = layer.gate.ty not in (W.F32, W.F16, W.BF16)
    act = n * (e + e // 32 * 8) if quant else n * e * 4
    return w + act + pairs * ff * 4


def expert_ops(layer, n):
    """Operations (two per multiply-add) of the expert products of one pass."""
    k, e, ff = layer.n_expert_used, layer.n_embd, layer.n_ff_exp
    return 2.0 * n * (k + (1 if layer.has_shared else 0)) * 3 * e * ff


class ClockSampler(threading.Thread):
    """Reads (never sets) SM clocks and throttle reasons through NVML while the
    timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.samples, self.reasons = index, False, [], set()
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if not self.nv:
            return
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
                 "sw_thermal_slowdown": 0x20, "hw_power_brake": 0x80}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.01)

    def finish(self):
        self.stop_flag = True
        self.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        # the median over the samples taken while the GPU was busy (above idle clocks)
        busy = [s for s in self.samples if s > 0.5 * (self.max_mhz or max(self.samples))] or self.samples
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------
# timing

def timed_loops(run_steps, steps, stream, sync, agree=None, min_ms=MIN_TIMED_MS):
    """Device time of `run_steps(steps)` between two events on `stream`, bracketed by
    `sync()` (barrier + device synchronize).  The K-step loop is repeated until the loops
    cover `min_ms` of device time; returns (median ms per loop, all loop times).  `agree`
    makes a figure the same on all ranks (max all-reduce)."""
    import torch

    def one():
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run_steps(steps)
        e1.record(stream)
        sync()
        t = e0.elapsed_time(e1)
        return agree(t) if agree else t

    first = one()
    reps = int(min(400, max(3, math.ceil(min_ms / max(first, 1e-3)))))
    times = [first] + [one() for _ in range(reps - 1)]
    return statistics.median(times), times


# --------------------------------------------------------------------------
# parity against the CPU oracle, outside every timed region

def parity_against_oracle(m, layer, h, got, rows):
    """Rows `rows` of a pass `m` (a `Moe` whose taps hold that pass) against the oracle
    on those rows alone - the layer is token-wise.  Reports what the gates of
    tests/test_gpu_parity.py check: ids, outputs of tokens without a re-quantisation flip
    (gate 1e-3), and the count and worst error of tokens with one (gate 1e-2)."""
    import oracle
    from biv_b200 import capi
    rows = np.asarray(rows)
    k, ff = layer.n_expert_used, layer.n_ff_exp
    ref, tap = oracle.moe_forward(layer, np.ascontiguousarray(h[rows]), level=oracle.host_level(),
                                  threads=oracle.max_threads(), taps=True)
    ids = m.tap(capi.TAP_IDS)[rows]
    same = (ids == tap["ids"]).all(axis=1)
    ties = 0
    for t in np.nonzero(~same)[0]:          # excused only at logit ties closer than 1e-6
        for a, b in zip(ids[t], tap["ids"][t]):
            if a != b and abs(float(tap["logits"][t, a]) - float(tap["logits"][t, b])) >= 1e-6:
                ties += 1
                break
    floor = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    err = (np.abs(got[rows].astype(np.float64) - ref) / np.maximum(np.abs(ref), floor)).max(axis=1)
    flipped_tok = np.zeros(len(rows), bool)
    flipped_int8 = 0
    if tap.get("mid_q") is not None:
        mid = m.tap(capi.TAP_MID).reshape(-1, k, ff)[rows].reshape(-1, ff)
        mq, _, _ = oracle.q8_quantize(mid)
        differ = (mq != tap["mid_q"]).reshape(len(rows), k, ff)
        differ[~same] = False
        flipped_int8 = int(differ.sum())
        flipped_tok = differ.any(axis=(1, 2))
    clean = same & ~flipped_tok
    worst_clean = float(err[clean].max(initial=0.0))
    worst_flipped = float(err[same & flipped_tok].max(initial=0.0))
    # a flip in the shared expert's row shows as a clean token above the gate; they are
    # counted with the flipped ones when their error is what one int8 step explains
    over = clean & (err >= GATE)
    return {"against": "CPU oracle (C restatement of the reference's kernels), same rows",
            "rows": int(len(rows)), "rows_with_equal_ids": int(same.sum()),
            "id_mismatches_beyond_ties": int(ties),
            "rel_err": float(err[clean & ~over].max(initial=0.0)), "gate": GATE,
            "flipped_int8": flipped_int8,
            "flipped_tokens": int(flipped_tok.sum() + over.sum()),
            "worst_flipped_token_err": max(worst_flipped, float(err[over].max(initial=0.0))),
            "flip_gate": FLIP_GATE,
            "metric": "max_i |got - ref| / max(|ref|, rms(ref))",
            "ok": bool(ties == 0 and max(worst_clean, worst_flipped) < FLIP_GATE
                       and float(err[clean & ~over].max(initial=0.0)) < GATE
                       and over.sum() <= max(2, 0.02 * len(rows)))}


def sample_rows(n, count, seed=17):
    if n <= count:
        return np.arange(n)
    return np.sort(np.random.default_rng(seed).choice(n, count, replace=False))


# --------------------------------------------------------------------------
# the CPU arm

def cpu_sample(wl):
    n = min(wl.n, CPU_SAMPLE_TOKENS)
    return np.ascontiguousarray(wl.h[:n]), n


def time_cpu(wl, budget_s=12.0, min_passes=2):
    """The oracle (the C restatement of the reference's CPU kernels) on this host's cores,
    on a bounded sample of the workload's rows; tokens/s of the sample."""
    import oracle
    threads, level = oracle.max_threads(), oracle.host_level()
    h, n = cpu_sample(wl)
    oracle.moe_forward(wl.layer, h[: min(4, n)], level=level, threads=threads)   # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_passes or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        oracle.moe_forward(wl.layer, h, level=level, threads=threads)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": n / med, "unit": UNIT, "cores": threads, "kind": "port",
            "kernels": oracle.LEVEL_NAMES[level],
            "sample": f"{len(times)} passes over the first {n} of the workload's {wl.n} rows, median "
                      f"(tokens/s of the sample: the layer is token-wise, so the figure scales linearly; "
                      f"each pass streams the weights of every expert the sample selects); best "
                      f"{n / min(times):.1f} {UNIT}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload(args.workload, args.tokens)
    import oracle
    threads, level = oracle.max_threads(), oracle.host_level()
    h, n = cpu_sample(wl)
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.moe_forward(wl.layer, h, level=level, threads=threads)
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.moe_forward(wl.layer, h, level=level, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    val = n / dt
    sample = (f"{steps} steps, each one pass over the first {n} of the workload's {wl.n} rows on the host "
              "cores (tokens/s of the sample; the layer is token-wise); C restatement of biv's CPU "
              "kernels (the Rust reference cannot be built here)")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPES.get(wl.name, "f32"),
        "data": "synthetic",
        "config": {"workload": describe(wl), "tokens": wl.n, "sample_tokens": n, "parallelism": "cpu"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "kernels": oracle.LEVEL_NAMES[level], "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------
# one layer on one GPU

def measure_layer(wl, args, local, copies=1, in_flight=1, parity_rows=256, with_e2e=True):
    """One layer object (or `copies` of it, rotated so the working set exceeds L2) on
    this GPU: one pass at a time (the figure), `in_flight` passes on as many streams (a
    side figure), the host-buffer call end to end, the stages with events, parity."""
    import torch
    from biv_b200 import capi
    from biv_b200.moe import Moe, launch_count
    layer, n = wl.layer, wl.n
    ms_ = [Moe(layer, n, device=local) for _ in range(copies)]
    h = torch.from_numpy(wl.h).cuda()
    outs = [torch.empty_like(h) for _ in range(max(1, in_flight))]
    streams = [torch.cuda.Stream() for _ in range(max(1, in_flight))]
    res = {}

    def sync():
        torch.cuda.synchronize()

    def alone(count):
        with torch.cuda.stream(streams[0]):
            for i in range(count):
                ms_[i % copies].moe_(h, outs[0], accumulate=False)

    warm = max(args.warmup, 3) if copies == 1 else max(args.warmup, 3 * copies)
    alone(warm)          # every layer object sees its call twice (the second builds its graph)
    sync()
    experts_hit = int((ms_[0].tap(capi.TAP_COUNTS) > 0).sum())
    l0 = launch_count()
    ms_loop, loops = timed_loops(alone, args.steps, streams[0], sync, min_ms=0.0 if args.quick else MIN_TIMED_MS)
    launches = (launch_count() - l0) // len(loops)
    ms_[0].status()      # no bounded wait gave up on the device
    res.update(ms_per_step=ms_loop / args.steps, loops=len(loops), launches=launches,
               experts_hit=experts_hit, warmup=warm,
               spread=[min(loops) / args.steps, max(loops) / args.steps])
    if args.quick:
        for m in ms_:
            m.close()
        return res
    # ---- parity of the last pass (the taps of the layer object that ran it)
    last = ms_[(args.steps - 1) % copies]
    got = outs[0].cpu().numpy()
    res["parity"] = parity_against_oracle(last, layer, wl.h, got, sample_rows(n, parity_rows))
    # ---- several passes in flight: layer object j on stream j mod in_flight
    if in_flight > 1 and copies % in_flight == 0:
        def flight(count):
            for i in range(count):
                j = i % copies
                with torch.cuda.stream(streams[j % in_flight]):
                    ms_[j].moe_(h, outs[j % in_flight], accumulate=False)
            for st in streams[1:]:
                ev = torch.cuda.Event()
                ev.record(st)
                streams[0].wait_event(ev)
        flight(3 * copies)
        sync()
        fl_ms, _ = timed_loops(flight, args.steps, streams[0], sync)
        res["in_flight"] = {"passes": in_flight, "ms_per_step": fl_ms / args.steps,
                            "value": n / (fl_ms / args.steps * 1e-3), "unit": UNIT,
                            "note": f"{in_flight} independent passes on {in_flight} streams and layer objects "
                                    "(how a host with several micro-batches drives the layers); the figure "
                                    "above it is one pass at a time"}
        alone(3 * copies)      # the graphs go back to stream 0
        sync()
    # ---- end to end through the host-buffer call: rows in from page-locked memory,
    #      the delta out, every step, one pass at a time
    if with_e2e:
        h_pin = torch.from_numpy(wl.h).pin_memory()
        out_pin = torch.empty_like(h_pin).pin_memory()
        for i in range(3 * copies):
            ms_[i % copies].moe_host(h_pin, out_pin)
        sync()
        e2e_steps = max(3, min(args.steps, int(2000.0 / max(res["ms_per_step"], 0.05))))
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            ms_[i % copies].moe_host(h_pin, out_pin)
        sync()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        res["e2e"] = {"value": n / e2e_s, "unit": UNIT, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                      "h2d_bytes_per_step": n * layer.n_embd * 4, "d2h_bytes_per_step": n * layer.n_embd * 4,
                      "call": "bivmoe_forward_host on page-locked buffers, one pass at a time: every step "
                              "copies its rows in and its result out (from 4096 rows on the call works in "
                              "sections whose copies overlap the section at work)"}
        if in_flight > 1 and copies % in_flight == 0:
            hp = [h_pin] + [torch.from_numpy(wl.h).pin_memory() for _ in range(in_flight - 1)]
            op = [out_pin] + [torch.empty_like(h_pin).pin_memory() for _ in range(in_flight - 1)]

            def pipelined(count):
                for i in range(count):
                    j = i % copies
                    if i >= in_flight:
                        ms_[(i - in_flight) % copies].wait()
                    ms_[j].moe_host_async(hp[j % in_flight], op[j % in_flight])
                for i in range(max(0, count - in_flight), count):
                    ms_[i % copies].wait()
            pipelined(3 * copies)
            sync()
            t0 = time.perf_counter()
            pipelined(e2e_steps)
            sync()
            fl_s = (time.perf_counter() - t0) / e2e_steps
            res["e2e"]["in_flight"] = {"passes": in_flight, "value": n / fl_s,
                                       "call": "bivmoe_forward_host_async + bivmoe_host_wait"}
    # ---- the stages with events around each launch (a loop of its own)
    profs = [ms_[i % copies].profile(h, outs[0]) for i in range(min(args.steps, 50))]
    res["stage_ms"] = {k: statistics.median(p[k] for p in profs) for k in profs[0]}
    res["int8_peak"] = ms_[0].int8_peak() if layer.gate.ty == W.Q8_0 else None
    for m in ms_:
        m.close()
    return res


def hbm_roofline(layer, n, r, traffic=None, traffic_source=None):
    hbm_peak, _, kind = load_peaks()
    kbytes = gateup_bytes(layer, n, r["experts_hit"])
    k_ms = r["stage_ms"]["gateup"]
    lbytes = algorithmic_bytes(layer, n, r["experts_hit"])
    roof = {"bound": "hbm", "kernel": "experts_kernel<gate+up>", "achieved": kbytes / (k_ms * 1e-3) / 1e9,
            "peak": hbm_peak, "peak_kind": f"of {kind}", "unit": "GB/s",
            "frac": kbytes / (k_ms * 1e-3) / 1e9 / hbm_peak, "traffic": traffic,
            "bytes_per_launch": kbytes, "kernel_ms": k_ms, "experts_hit": r["experts_hit"],
            "stage_ms": r["stage_ms"], "layer_bytes": lbytes,
            "layer_frac": lbytes / (r["ms_per_step"] * 1e-3) / 1e9 / hbm_peak}
    if traffic_source:
        roof["traffic_source"] = traffic_source
    return roof


def tensor_roofline(layer, n, r, int8):
    _, tf_peak, kind = load_peaks()
    st = r["stage_ms"]
    t_exp = (st["gateup"] + st["down"]) * 1e-3
    ops = expert_ops(layer, n)
    peak = r["int8_peak"] if int8 else tf_peak
    hbm_peak = load_peaks()[0]
    lbytes = algorithmic_bytes(layer, n, r["experts_hit"])
    t_roof = max(lbytes / (hbm_peak * 1e9), ops / (peak * 1e12))
    return {"bound": "tensor",
            "kernel": "experts_prefill_kernel (tcgen05 kind::i8)" if int8
            else "experts_prefill_bf16_gateup_kernel + experts_prefill_bf16_down_kernel (tcgen05 kind::f16)",
            "achieved": ops / t_exp / 1e12, "peak": peak,
            "peak_kind": "int8 tensor pipe measured in this run (back-to-back tcgen05.mma kind::i8, "
                         "bivmoe_int8_peak)" if int8 else f"of {kind}",
            "unit": "TOP/s" if int8 else "TFLOP/s", "frac": ops / t_exp / 1e12 / peak, "traffic": None,
            "kernel_ms": t_exp * 1e3, "stage_ms": st, "experts_hit": r["experts_hit"],
            "whole_layer_frac_of_max_roof": t_roof / (r["ms_per_step"] * 1e-3),
            "note": ("achieved counts the reference's multiply-adds once; every 32-wide block dot is one MMA "
                     "whose int32 result the epilogue warps scale in f32 (exact block dots), which bounds the "
                     "kernel at 12.5 % of the int8 peak" if int8 else
                     "achieved counts the reference's multiply-adds once; the kernel issues two MMAs per "
                     "multiply-add (an f32 row as two bf16 terms: one 11-bit term misses the 1e-3 gate, "
                     "tests/test_operand_precision.py), so 0.5 is the ceiling of this figure")}


def side_object(wl, r, roof):
    o = {"workload": describe(wl), "value": wl.n / (r["ms_per_step"] * 1e-3), "unit": UNIT,
         "ms_per_step": r["ms_per_step"], "timing": f"one pass at a time; median of {r['loops']} loops",
         "dtype": DTYPES.get(wl.name), "roofline": roof, "parity": r.get("parity"), "e2e": r.get("e2e"),
         "gpu_launches_per_loop": r["launches"]}
    if "in_flight" in r:
        o["in_flight"] = r["in_flight"]
    return o


# --------------------------------------------------------------------------
# configs[3]: the 40-layer stack, streamed to the device one layer at a time

def measure_stack(args, local, budget_s):
    import oracle
    import torch
    from biv_b200 import capi
    from biv_b200.moe import Moe, MoeStack, launch_count
    x0, eps, _ = W.mtp_stack_streamed(n_layers=args.layers)
    n = x0.shape[0]

    # layers are independent streams of the generator: build them on host threads, keep a
    # few ahead of the uploads
    def gen_layer(l):
        return W.mtp_stack_layer(l)

    layers, hosts0, t_start = [], None, time.perf_counter()
    with ThreadPoolExecutor(max_workers=6) as pool:
        pending = []
        nxt = 0
        while len(layers) < args.layers:
            while nxt < args.layers and len(pending) < 6:
                pending.append(pool.submit(gen_layer, nxt))
                nxt += 1
            layer, nw = pending.pop(0).result()
            m = Moe(layer, n, device=local)
            m.set_post_norm(nw, eps)
            if not layers:
                hosts0 = (layer, nw)
            layers.append(m)
            if time.perf_counter() - t_start > budget_s and len(layers) >= 8:
                for p in pending:
                    p.cancel()
                break
    nl = len(layers)
    stack = MoeStack(layers)
    xd0 = torch.from_numpy(x0).cuda()
    x = xd0.clone()
    stream = torch.cuda.Stream()

    def sync():
        torch.cuda.synchronize()

    def run(count):
        with torch.cuda.stream(stream):
            for _ in range(count):
                x.copy_(xd0)            # the residual of a fresh pass
                stack.forward_(x)

    run(max(3, min(args.warmup, 5)))
    sync()
    steps = max(3, min(args.steps, 10))
    l0 = launch_count()
    ms_loop, loops = timed_loops(run, steps, stream, sync)
    launches = (launch_count() - l0) // len(loops)
    ms = ms_loop / steps
    for m in layers:
        m.status()      # no bounded wait gave up on the device
    hits = [int((m.tap(capi.TAP_COUNTS) > 0).sum()) for m in layers]
    # parity of the first layer (norm fused into the router, layer, residual add)
    one = xd0.clone()
    with torch.cuda.stream(stream):
        MoeStack(layers[:1]).forward_(one)
    sync()
    want = oracle.moe_stack([hosts0[0]], [hosts0[1]], eps, x0, level=oracle.host_level(),
                            threads=oracle.max_threads())
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    row = np.abs(one.cpu().numpy() - want).max(axis=1) / rms
    hbm_peak, _, kind = load_peaks()
    sizes = hosts0[0]
    bytes_pass = sum(algorithmic_bytes(sizes, n, h_) for h_ in hits)
    out = {"workload": f"mtp_stack: {nl} MoE FFN layers of the 40 (built until the {budget_s:.0f} s set-up budget "
                       f"ran out)" if nl < args.layers else
                       f"mtp_stack: all {nl} MoE FFN layers, {n} tokens (32 sequences x 5), hidden 2048, 256 "
                       "experts top-8 + shared expert, ff 512, gate/up Q5_K down Q6_K, rms_norm fused into "
                       "the router kernel + residual add per layer, seed 3 (one generator stream per layer)",
           "layers": nl, "value": n / (ms * 1e-3) * (40.0 / nl if nl < 40 else 1.0), "unit": UNIT,
           "ms_per_step": ms, "ms_per_layer": ms / nl, "timing": f"median of {len(loops)} loops of {steps} passes",
           "dtype": DTYPES["mtp_stack"],
           "roofline": {"bound": "hbm", "kernel": "whole stack", "achieved": bytes_pass / (ms * 1e-3) / 1e9,
                        "peak": hbm_peak, "peak_kind": f"of {kind}", "unit": "GB/s",
                        "frac": bytes_pass / (ms * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                        "bytes_per_pass": bytes_pass, "experts_hit_per_layer": hits},
           "parity": {"against": "CPU oracle, first layer of the stack on the same rows (norm, layer, residual)",
                      "rows": int(n), "median_row_err": float(np.median(row)), "worst_row_err": float(row.max()),
                      "gate": "median < 2e-4, worst < 1e-2 (a re-quantisation flip or a changed top-8 choice)",
                      "ok": bool(np.median(row) < 2e-4 and row.max() < FLIP_GATE)},
           "gpu_launches_per_loop": launches}
    if nl < 40:
        out["note"] = "value is scaled to 40 layers from the layers that were built"
    for m in layers:
        m.close()
    return out


# --------------------------------------------------------------------------
# expert parallelism: the headline at N > 1

def measure_ep(wl, args, rank, world, local):
    import torch
    import torch.distributed as dist
    from biv_b200.ep import EpMoe
    from biv_b200.moe import Moe, launch_count
    layer = wl.layer
    n_per = wl.n // world
    h_rank = np.ascontiguousarray(wl.h[rank * n_per:(rank + 1) * n_per])
    peer = args.ep_exchange == "peer"
    h = torch.from_numpy(h_rank).cuda()
    out = torch.empty_like(h)

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    def agree(t):
        v = torch.tensor([t], device="cuda", dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v[0])

    def build(parts):
        np_ = n_per // parts
        objs = [EpMoe(layer, np_, rank, world, local, exchange=args.ep_exchange,
                      barrier="lib" if peer and args.ep_barrier == "lib" else "comm") for _ in range(parts)]
        streams = [torch.cuda.Stream() for _ in range(parts)]
        hs = [h[i * np_:(i + 1) * np_] for i in range(parts)]
        os_ = [out[i * np_:(i + 1) * np_] for i in range(parts)]

        def run(count):
            for _ in range(count):
                if peer:
                    for i in range(parts):
                        with torch.cuda.stream(streams[i]):
                            objs[i].moe_(hs[i], os_[i], accumulate=False)
                else:
                    for i in range(parts):
                        with torch.cuda.stream(streams[i]):
                            objs[i].begin(hs[i])
                    for i in range(parts):
                        with torch.cuda.stream(streams[i]):
                            objs[i].finish(os_[i], accumulate=False)
            for st in streams[1:]:
                ev = torch.cuda.Event()
                ev.record(st)
                streams[0].wait_event(ev)
        return objs, streams, run, hs, os_

    # how many micro-batches a rank keeps in flight (each with its own layer object and
    # stream, so that one's stores over NVLink run beside the other's expert kernels): the
    # faster of 1 and 2 on a short trial, unless the command line fixes it
    candidates = [args.ep_in_flight] if args.ep_in_flight else [1, 2]
    candidates = [c for c in candidates if n_per % c == 0] or [1]
    trials, built = {}, {}
    for parts in candidates:
        objs, streams, run, hs, os_ = build(parts)
        run(max(3, args.warmup))
        for o in objs:
            o.status()
        sync()
        t, _ = timed_loops(run, max(2, min(args.steps, 5)), streams[0], sync, agree, min_ms=0.0)
        trials[parts] = t / max(2, min(args.steps, 5))
        built[parts] = (objs, streams, run, hs, os_)
    # the faster; within 2 % the larger count, whose copies the end-to-end steps can overlap
    fastest = min(trials.values())
    best = max(p_ for p_, t_ in trials.items() if t_ <= 1.02 * fastest)
    for parts, (objs, _, _, _, _) in built.items():
        if parts != best:
            sync()
            for o in objs:
                o.close()
    objs, streams, run, hs, os_ = built[best]
    sync()
    l0 = launch_count()
    ms_loop, loops = timed_loops(run, args.steps, streams[0], sync, agree)
    launches = (launch_count() - l0) // len(loops)
    for o in objs:
        o.status()
    res = {"ms_per_step": ms_loop / args.steps, "loops": len(loops), "launches": launches,
           "micro_batches": best, "trial_ms": {str(k_): v for k_, v in trials.items()},
           "spread": [min(loops) / args.steps, max(loops) / args.steps]}
    if args.quick:
        sync()
        for o in objs:
            o.close()
        return res
    got = out.cpu().numpy()
    # ---- where the time goes: the steps of one pass with events (one micro-batch object)
    if peer:
        st0 = streams[0]
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        o0, np0 = objs[0], n_per // best
        bar = o0.steps.peer_barrier if o0.lib_barrier else (lambda: o0.comm.barrier(h.device))
        stage_runs = []
        for _ in range(5):
            sync()
            with torch.cuda.stream(st0):
                evs[0].record(st0)
                o0.steps.peer_dispatch(h[:np0])
                evs[1].record(st0)
                bar()
                evs[2].record(st0)
                o0.steps.shared(h[:np0])
                o0.steps.peer_experts()
                evs[3].record(st0)
                bar()
                evs[4].record(st0)
                o0.steps.peer_combine(out[:np0], False)
                evs[5].record(st0)
            sync()
            stage_runs.append([evs[i].elapsed_time(evs[i + 1]) for i in range(5)])
        med = [statistics.median(r[i] for r in stage_runs) for i in range(5)]
        res["stage_ms"] = dict(zip(["route_and_stores_out", "barrier_a", "experts_and_stores_back", "barrier_b",
                                    "combine"], med))
    # ---- end to end: this rank's rows in from page-locked memory, the pass, the delta out
    h_pin = torch.from_numpy(h_rank).pin_memory()
    out_pin = torch.empty_like(h_pin).pin_memory()

    np_ = n_per // len(objs)
    pipelined = peer and len(objs) > 1

    def e2e_step():
        if pipelined:
            # every micro-batch on its own stream: its rows in, its pass, its delta out - one
            # micro-batch's copies run beside the other's kernels
            for i, o in enumerate(objs):
                with torch.cuda.stream(streams[i]):
                    hs[i].copy_(h_pin[i * np_:(i + 1) * np_], non_blocking=True)
                    o.moe_(hs[i], os_[i], accumulate=False)
                    out_pin[i * np_:(i + 1) * np_].copy_(os_[i], non_blocking=True)
            for st in streams:
                st.synchronize()
            return
        with torch.cuda.stream(streams[0]):
            h.copy_(h_pin, non_blocking=True)
        for st in streams[1:]:
            st.wait_stream(streams[0])
        run(1)
        with torch.cuda.stream(streams[0]):
            out_pin.copy_(out, non_blocking=True)
        streams[0].synchronize()

    for _ in range(3):
        e2e_step()
    sync()
    e2e_steps = max(3, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    sync()
    e2e_ms = agree((time.perf_counter() - t0) * 1e3 / e2e_steps)
    res["e2e"] = {"value": wl.n / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "steps": e2e_steps,
                  "h2d_bytes_per_step": wl.n * layer.n_embd * 4, "d2h_bytes_per_step": wl.n * layer.n_embd * 4,
                  "call": "per rank and step: its rows copied in from page-locked memory, EpMoe.moe_ (the "
                          "bivmoe_ep_peer_* / bivmoe_ep_* steps), the delta copied out; wall clock, max over ranks"
                          + ("; each micro-batch copies, computes and copies out on its own stream" if pipelined
                             else "")}
    # ---- exchange volume (rank 0): a row goes once to every rank owning one of its experts
    ids_rows = None
    sync()
    for o in objs:
        o.close()
    # ---- parity, rank 0: its rows through the whole layer on this GPU alone, and the oracle
    if rank == 0:
        m = Moe(layer, n_per, device=local)
        want = m.moe(torch.from_numpy(h_rank).cuda()).cpu().numpy()
        torch.cuda.synchronize()
        from biv_b200 import capi
        ids_rows = m.tap(capi.TAP_IDS)
        owners = np.unique(np.stack([np.arange(n_per).repeat(layer.n_expert_used),
                                     (ids_rows.reshape(-1) // (layer.n_expert // world))], 1), axis=0)
        sent = int(len(owners))
        delta = float(np.abs(got - want).max() / max(float(np.abs(want).max()), 1e-30))
        par = parity_against_oracle(m, layer, h_rank, got, sample_rows(n_per, 256))
        m.close()
        par["against_single_gpu_layer"] = {"rows": int(n_per), "max_abs_delta_over_max_abs": delta,
                                           "gate": 1e-6, "ok": bool(delta <= 1e-6)}
        par["ok"] = bool(par["ok"] and delta <= 1e-6)
        res["parity"] = par
        res["rows_sent_rank0"] = sent
    dist.barrier()
    return res


# --------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="ep_bf16",
                    help="the headline workload: ep_bf16 (default), decode_q4k, prefill_q8_0, parity_q8_0")
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--side", default="auto", choices=["auto", "none", "all"],
                    help="the decode / prefill / stack side objects: auto = at N = 1 with the default workload")
    ap.add_argument("--layers", type=int, default=40, help="layers of the stack side object")
    ap.add_argument("--stack-budget", type=float, default=150.0,
                    help="seconds the stack side object may spend building layers before it measures what it has")
    ap.add_argument("--copies", type=int, default=4,
                    help="resident copies of the decode layer the timed loop rotates over (working set > L2)")
    ap.add_argument("--ep-exchange", default="peer", choices=["all_to_all", "peer"],
                    help="expert parallelism: rows moved by NCCL all-to-alls, or by the library's "
                         "kernels storing into the peers' memory")
    ap.add_argument("--ep-barrier", default="lib", choices=["lib", "comm"],
                    help="peer exchange: the library's own barrier, or one-element NCCL all-reduces")
    ap.add_argument("--ep-in-flight", type=int, default=0,
                    help="micro-batches a rank keeps in flight (0: the faster of 1 and 2 on a short trial)")
    ap.add_argument("--quick", action="store_true",
                    help="warm-up and timed loop only (the command profilers wrap)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sides = (args.side == "all" or (args.side == "auto" and world == 1 and args.workload == "ep_bf16")) \
        and not args.quick and rank == 0
    # the side workloads are generated on host threads while the headline runs
    pool = ThreadPoolExecutor(max_workers=2)
    side_wl = {name: pool.submit(make_workload, name) for name in ("decode_q4k", "prefill_q8_0")} if sides else {}

    wl = make_workload(args.workload, args.tokens)
    layer, n = wl.layer, wl.n
    sampler = ClockSampler(local)
    sampler.start()
    if world > 1 and layer.n_expert % world == 0 and n % world == 0:
        r = measure_ep(wl, args, rank, world, local)
        parallelism = f"ep{world}"
    else:
        copies = args.copies if args.workload == "decode_q4k" else 1
        r = measure_layer(wl, args, local, copies=copies, in_flight=copies if copies > 1 else 1)
        parallelism = "single" if world == 1 else "replicas"
    clocks = sampler.finish()
    if args.quick:
        if rank == 0:
            print(json.dumps({"quick": True, "workload": wl.name, "ms_per_step": r["ms_per_step"],
                              "steps": args.steps, "loops": r["loops"]}))
        if world > 1:
            dist.destroy_process_group()
        return
    if rank != 0:
        dist.destroy_process_group()
        return

    ms_step = r["ms_per_step"]
    line = {
        "metric": METRIC, "value": n / (ms_step * 1e-3) * (world if parallelism == "replicas" else 1),
        "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak" if parallelism == "replicas" else "strong", "vs_baseline": None,
        "dtype": DTYPES.get(wl.name, "f32"), "data": "synthetic",
        "config": {"workload": describe(wl), "tokens": n, "tokens_per_gpu": n // world if parallelism != "replicas" else n,
                   "parallelism": parallelism,
                   "experts_per_gpu": layer.n_expert // world if parallelism.startswith("ep") else layer.n_expert,
                   "passes": "one pass at a time",
                   "timing": f"CUDA events around K = {args.steps} steps, the loop repeated {r['loops']} times "
                             f"(>= {MIN_TIMED_MS:.0f} ms of device time), median loop; fastest and slowest loop "
                             f"{r['spread'][0]:.4f} / {r['spread'][1]:.4f} ms per step",
                   "l2": "weights and rows of one pass exceed the 126 MB L2, no flush" if args.workload != "decode_q4k"
                         else f"steps rotate over {args.copies} resident copies of the layer (working set > 126 MB L2)"},
        "e2e": r.get("e2e"), "gpu_launches": r["launches"] * 1, "clocks": clocks,
    }
    if parallelism.startswith("ep"):
        _, tf_peak, kind = load_peaks()
        ops = expert_ops(layer, n)
        e = layer.n_embd
        sent = r.get("rows_sent_rank0") or 0
        st = r.get("stage_ms") or {}
        mb = r["micro_batches"]
        line["config"].update(exchange=args.ep_exchange, barrier=args.ep_barrier if args.ep_exchange == "peer" else "nccl",
                              micro_batches=mb)
        line["roofline"] = {"bound": "tensor", "kernel": "whole pass per GPU, exchanges included",
                            "achieved": ops / (ms_step * 1e-3) / 1e12 / world, "peak": tf_peak,
                            "peak_kind": f"of {kind}", "unit": "TFLOP/s",
                            "frac": ops / (ms_step * 1e-3) / 1e12 / world / tf_peak if tf_peak else None,
                            "traffic": None}
        out_b = sent * (e * 4 + 2 * layer.n_expert_used * 4)
        back_b = sent * e * 4
        ep = {"exchange": args.ep_exchange, "micro_batches": mb, "trial_ms_per_step": r["trial_ms"],
              "rows_sent_rank0": sent, "bytes_out_rank0": out_b, "bytes_back_rank0": back_b,
              "transport": ("the library's kernels store rows and tags into the owners' memory and the "
                            "partial sums into the home ranks' memory over NVLink (CUDA IPC mappings); "
                            + ("the library's own barrier (flag words in the ranks' blocks, bounded waits)"
                               if args.ep_barrier == "lib" else "one-element NCCL all-reduces as barriers"))
              if args.ep_exchange == "peer" else "NCCL all_to_all_single over NVLink, counts through the host",
              "stage_ms": st or None, "parity": r.get("parity")}
        if st and sent:
            per = sent / mb     # the staged pass covers one micro-batch
            ep["nvlink"] = {
                "out_gbs_lower_bound": per * (e * 4 + 64) / (st["route_and_stores_out"] * 1e-3) / 1e9,
                "back_gbs_lower_bound": per * e * 4 / (st["experts_and_stores_back"] * 1e-3) / 1e9,
                "barrier_ms": st["barrier_a"] + st["barrier_b"],
                "note": "lower bounds: the stages also hold the router, top-k and the expert kernels; "
                        "measured peer copy 770 GB/s per direction"}
            t_ideal = max(ops / world / (tf_peak * 1e12), per * mb * e * 4 / 770e9)
            ep["limiter"] = max(st, key=st.get)
            ep["roofline_time_ms"] = t_ideal * 1e3
        line["ep"] = ep
        line["parity"] = r.get("parity")
    else:
        if layer.gate.ty in (W.BF16, W.Q8_0) and n >= 512:
            line["roofline"] = tensor_roofline(layer, n, r, int8=layer.gate.ty == W.Q8_0)
        else:
            line["roofline"] = hbm_roofline(layer, n, r)
        line["parity"] = r.get("parity")
        if "in_flight" in r:
            line["in_flight"] = r["in_flight"]

    if not args.no_cpu:
        line["cpu_baseline"] = time_cpu(wl)

    if sides:
        t_side = time.perf_counter()
        a2 = argparse.Namespace(**vars(args))
        a2.steps, a2.warmup = 200, 20
        dw = side_wl["decode_q4k"].result()
        dr = measure_layer(dw, a2, local, copies=args.copies, in_flight=args.copies, parity_rows=64)
        line["decode"] = side_object(dw, dr, hbm_roofline(
            dw.layer, dw.n, dr, traffic=108.0e6,
            traffic_source="dram__bytes_read.sum + dram__bytes_write.sum of one gate+up launch from an ncu "
                           "capture of this workload at commit 86365ed (one weight copy); a recorded figure, "
                           "not produced by this run"))
        a2.steps, a2.warmup = 20, 5
        pw = side_wl["prefill_q8_0"].result()
        pr = measure_layer(pw, a2, local, copies=1, parity_rows=256)
        line["prefill"] = side_object(pw, pr, tensor_roofline(pw.layer, pw.n, pr, int8=True))
        line["stack"] = measure_stack(a2, local, args.stack_budget)
        line["side_objects_s"] = time.perf_counter() - t_side
    pool.shutdown(wait=False, cancel_futures=True)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
