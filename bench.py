#!/usr/bin/env python
"""Benchmark of the qwen35moe MoE feed-forward layer on B200.

One "step" is one pass of the layer over one batch of synthetic rows.  The
workload at any N is the decode configuration (64 single-token sequences,
Q4_K experts, skewed routing): inputs are generated from a seed, there is no
dataset.  Prints ONE JSON line (rank 0).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
  python bench.py --impl reference ...   # the CPU restatement of the reference's kernels
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from biv_b200 import workloads as W  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
WEIGHT_COPIES = 4   # the timed loop rotates over this many resident copies of the layer


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"], d.get("bf16_tflops"), "measured"
    return 6650.0, 1590.0, "fallback"


def make_workload(name, args):
    if name == "decode_q4k":
        return W.decode_q4k(n=args.tokens or 64)
    if name == "parity_q8_0":
        return W.parity_q8_0(n=args.tokens or 16)
    if name == "prefill_q8_0":
        return W.prefill_q8_0(n=args.tokens or 4096)
    if name == "ep_bf16":
        return W.ep_bf16(n=args.tokens or 16384)
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(layer, n, experts_hit):
    """Bytes one pass must move at least: every selected expert's weights once,
    the shared expert, the router and gate vector, the rows in and out."""
    return layer.weight_bytes(experts_hit) + 2 * n * layer.n_embd * 4


def gateup_bytes(layer, n, experts_hit):
    """The dominant kernel (gate+up with SwiGLU): gate and up matrices of every
    selected expert and of the shared expert once, the Q8 rows of h once per
    (token, expert) pair, the f32 mid rows written."""
    k, e, ff = layer.n_expert_used, layer.n_embd, layer.n_ff_exp
    w = experts_hit * (layer.gate.matrix_bytes + layer.up.matrix_bytes)
    pairs = n * k
    if layer.has_shared:
        w += layer.sh_gate.matrix_bytes + layer.sh_up.matrix_bytes
        pairs += n
    quant = layer.gate.ty not in (W.F32, W.BF16)
    act = n * (e + e // 32 * 8) if quant else n * e * 4
    return w + act + pairs * ff * 4


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

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def time_cpu(wl, budget_s=12.0, min_passes=2):
    """The oracle (the C restatement of the reference's CPU kernels) on this
    host's cores, same inputs; returns tokens/s and what was timed."""
    import oracle
    threads = oracle.max_threads()
    level = oracle.host_level()
    oracle.moe_forward(wl.layer, wl.h[: min(4, wl.n)], level=level, threads=threads)   # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_passes or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        oracle.moe_forward(wl.layer, wl.h, level=level, threads=threads)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": wl.n / med, "unit": UNIT, "cores": threads, "kind": "port",
            "kernels": oracle.LEVEL_NAMES[level],
            "sample": f"{len(times)} passes of the full workload ({wl.n} tokens), median; "
                      f"best {wl.n / min(times):.1f} {UNIT}"}, med


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload(args.workload, args)
    import oracle
    threads, level = oracle.max_threads(), oracle.host_level()
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.moe_forward(wl.layer, wl.h, level=level, threads=threads)
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.moe_forward(wl.layer, wl.h, level=level, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    val = wl.n / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 block dots, f32 scales",
        "data": "synthetic",
        "config": config_of(wl, args, 1),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "kernels": oracle.LEVEL_NAMES[level],
                         "sample": f"{steps} passes of the full workload ({wl.n} tokens) on the "
                                   "host cores; C restatement of biv's CPU kernels (the Rust "
                                   "reference cannot be built here)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def time_ep(layer, h_rank, steps, warmup, rank, world, local, in_flight=1, exchange="all_to_all",
            graph=False):
    """Expert-parallel passes of the layer: this rank's rows in, experts sharded
    n_expert / world per GPU, rows exchanged over NCCL.  Device time of `steps`
    passes, max over ranks; also this rank's output of the last pass.  With
    `in_flight` = 2 the rank's rows are two micro-batches, each with its own layer
    object and stream, begun together so that one's exchanges overlap the other's
    kernels; a step is still all of the rank's rows.  `exchange` "peer": the rows move by
    the library's own kernels (stores into the peers' memory), one pass at a time."""
    import torch
    import torch.distributed as dist
    from biv_b200.ep import EpMoe
    n = h_rank.shape[0]
    peer = exchange == "peer"
    parts = in_flight if (in_flight > 1 and n % in_flight == 0 and not peer) else 1
    n_part = n // parts
    ms_ = [EpMoe(layer, n_part, rank, world, local, exchange=exchange) for _ in range(parts)]
    streams = [torch.cuda.Stream() for _ in range(parts)]
    h = torch.from_numpy(h_rank).cuda()
    out = torch.empty_like(h)
    hs = [h[i * n_part:(i + 1) * n_part] for i in range(parts)]
    outs = [out[i * n_part:(i + 1) * n_part] for i in range(parts)]
    torch.cuda.synchronize()

    def one_step():
        if peer:
            with torch.cuda.stream(streams[0]):
                ms_[0].moe_(hs[0], outs[0], accumulate=False)
            return
        for i in range(parts):
            with torch.cuda.stream(streams[i]):
                ms_[i].begin(hs[i])
        for i in range(parts):
            with torch.cuda.stream(streams[i]):
                ms_[i].finish(outs[i], accumulate=False)

    for _ in range(max(3, warmup)):
        one_step()
    for m in ms_:
        m.status()
    dist.barrier()
    torch.cuda.synchronize()
    if peer and graph:      # the pass has no host step: replay it as one graph launch
        with torch.cuda.stream(streams[0]):
            g = ms_[0].capture(hs[0], outs[0], accumulate=False)

            def one_step():     # noqa: F811
                with torch.cuda.stream(streams[0]):
                    g.replay()
            for _ in range(3):
                one_step()
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(streams[0])
    for _ in range(steps):
        one_step()
    for st in streams[1:]:
        joined = torch.cuda.Event()
        joined.record(st)
        streams[0].wait_event(joined)
    e1.record(streams[0])
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    for m in ms_:
        m.status()
    recv = sum(m.last_plan.m for m in ms_) if not peer else 0
    res = out.cpu().numpy()
    for m in ms_:
        m.close()
    return float(t[0]) / steps, recv, res


def run_ep_workload(args, wl, rank, world, local):
    """`--workload ep_bf16` on more than one GPU: the configuration's rows split
    over the ranks (strong scaling), one JSON line."""
    import torch
    import torch.distributed as dist
    layer = wl.layer
    n_per = wl.n // world
    h_rank = np.ascontiguousarray(wl.h[rank * n_per:(rank + 1) * n_per])
    sampler = ClockSampler(local)
    sampler.start()
    ms, recv, _ = time_ep(layer, h_rank, args.steps, args.warmup, rank, world, local,
                          in_flight=args.ep_in_flight, exchange=args.ep_exchange, graph=args.ep_graph)
    sampler.stop_flag = True
    sampler.join()
    if rank == 0:
        _, tf_peak, peak_kind = load_peaks()
        k, e, ff = layer.n_expert_used, layer.n_embd, layer.n_ff_exp
        flops = 2.0 * wl.n * (k + 1) * 3 * e * ff
        row_bytes = e * 4
        line = {
            "metric": METRIC, "value": n_per * world / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 weights x f32 activations, f32 accumulation", "data": "synthetic",
            "config": {"workload": f"{wl.name}: {wl.n} tokens over {world} GPUs, hidden {e}, "
                                   f"{layer.n_expert} experts top-{k} + shared expert, ff {ff}, "
                                   f"BF16, seed {wl.seed}",
                       "tokens_per_gpu": n_per, "parallelism": f"ep{world}",
                       "exchange": args.ep_exchange,
                       "graph_replay": bool(args.ep_graph and args.ep_exchange == "peer"),
                       "in_flight": ("1 pass" if args.ep_exchange == "peer" else
                                     f"{args.ep_in_flight} micro-batch(es) of "
                                     f"{n_per // max(1, args.ep_in_flight)} rows per GPU"),
                       "experts_per_gpu": layer.n_expert // world,
                       "l2": "weights and rows of one pass exceed the 126 MB L2, no flush"},
            "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12 / world,
                         "peak": tf_peak, "peak_kind": f"of {peak_kind}", "unit": "TFLOP/s",
                         "frac": flops / (ms * 1e-3) / 1e12 / world / tf_peak if tf_peak else None,
                         "traffic": None, "scope": "whole pass per GPU, exchanges included"},
            "exchange": {"rows_received_rank0": recv, "bytes_each_way_rank0": recv * row_bytes,
                         "transport": ("the library's kernels store into the peers' memory over NVLink "
                                       "(CUDA IPC mappings), two one-element all-reduces per pass as "
                                       "barriers" if args.ep_exchange == "peer" else
                                       "NCCL all_to_all_single over NVLink") +
                                      "; an f32 row once per owning rank out, one f32 partial sum per "
                                      "row back"},
            "gpu_launches": None, "clocks": sampler.summary(),
        }
        print(json.dumps(line))
    dist.destroy_process_group()


def run_stack_workload(args, rank, world, local):
    """`--workload mtp_stack` (the MTP-verify shape): the 40-layer MoE FFN stack over
    32 sequences x 5 tokens, gate/up Q5_K and down Q6_K, rms_norm before each layer and
    the residual carried; a step is one pass of the whole stack (`--layers` of it)."""
    import torch
    from biv_b200.moe import Moe, MoeStack, launch_count
    wl = W.mtp_stack(n_layers=args.layers)
    n, nl = wl.n, len(wl.layers)
    layers = [Moe(l, n, device=local) for l in wl.layers]
    for m, nw in zip(layers, wl.norm_w):
        m.set_post_norm(nw, wl.eps)
    stack = MoeStack(layers)
    x0 = torch.from_numpy(wl.h).cuda()
    x = x0.clone()
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()

    def step():
        with torch.cuda.stream(stream):
            x.copy_(x0)                 # the residual of a fresh pass
            stack.forward_(x)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    launches = launch_count() - l0
    sampler.stop_flag = True
    sampler.join()
    ms = e0.elapsed_time(e1) / args.steps
    hits = [int((m.tap(3) > 0).sum()) for m in layers]          # TAP_COUNTS of the last pass
    hbm_peak, _, peak_kind = load_peaks()
    bytes_pass = sum(algorithmic_bytes(l, n, h_) for l, h_ in zip(wl.layers, hits))
    l = wl.layers[0]
    line = {
        "metric": METRIC, "value": world * n / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 block dots, f32 scales",
        "data": "synthetic",
        "config": {"workload": f"mtp_stack: {nl} MoE FFN layers, {n} tokens (32 sequences x 5), hidden "
                               f"{l.n_embd}, {l.n_expert} experts top-{l.n_expert_used} + shared expert, ff "
                               f"{l.n_ff_exp}, gate/up Q5_K down Q6_K, rms_norm + residual per layer, seed {wl.seed}",
                   "tokens_per_gpu": n, "layers": nl, "parallelism": "single" if world == 1 else "replicas",
                   "l2": f"{nl} layers of weights ({sum(x_.weight_bytes() for x_ in wl.layers) / 1e9:.1f} GB) "
                         "stream through the 126 MB L2 once per pass, no flush"},
        "roofline": {"bound": "hbm", "kernel": "whole stack", "achieved": bytes_pass / (ms * 1e-3) / 1e9,
                     "peak": hbm_peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                     "frac": bytes_pass / (ms * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                     "bytes_per_pass": bytes_pass, "experts_hit_per_layer": hits},
        "gpu_launches": launches, "clocks": sampler.summary(),
    }
    for m in layers:
        m.close()
    if rank == 0:
        print(json.dumps(line))


def config_of(wl, args, world):
    l = wl.layer
    return {"workload": f"{wl.name}: {wl.n} tokens per GPU, hidden {l.n_embd}, {l.n_expert} experts "
                        f"top-{l.n_expert_used} + shared expert, ff {l.n_ff_exp}, "
                        f"gate/up {W.TYPE_NAMES[l.gate.ty]} down {W.TYPE_NAMES[l.down.ty]}, seed {wl.seed}",
            "tokens_per_gpu": wl.n, "parallelism": "replicas" if world > 1 else "single",
            "l2": f"steps rotate over {max(1, args.copies)} resident copies of the layer's weights "
                  "(working set > 126 MB L2), no flush",
            "streams": f"passes rotate over {args.streams} streams, {args.streams} in flight"
            if getattr(args, "streams", 2) != 1 else "one stream, one pass at a time"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode_q4k")
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--copies", type=int, default=WEIGHT_COPIES,
                    help="resident copies of the layer the timed loop rotates over")
    ap.add_argument("--streams", type=int, default=WEIGHT_COPIES,
                    help="passes in flight: the timed passes rotate over this many streams, layer object "
                         "j on stream j mod streams (must divide --copies; 1: one pass at a time)")
    ap.add_argument("--layers", type=int, default=40, help="layers of the mtp_stack workload")
    ap.add_argument("--ep-exchange", default="peer", choices=["all_to_all", "peer"],
                    help="expert parallelism: rows moved by NCCL all-to-alls, or by the library's "
                         "kernels storing into the peers' memory")
    ap.add_argument("--ep-graph", action="store_true",
                    help="with --ep-exchange peer: replay each pass, barriers included, as one CUDA "
                         "graph instead of launching it kernel by kernel")
    ap.add_argument("--ep-in-flight", type=int, default=1,
                    help="micro-batches a rank keeps in flight in the expert-parallel workload (two "
                         "measured slower than one at 2 GPUs: 2.65 against 2.50 ms)")
    ap.add_argument("--quick", action="store_true",
                    help="warm-up and timed loop only (the command profilers wrap)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from biv_b200 import capi
    from biv_b200.moe import Moe, launch_count

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    warmup = max(args.warmup, 3)

    if args.workload == "mtp_stack":
        return run_stack_workload(args, rank, world, local)
    wl = make_workload(args.workload, args)
    if world > 1 and args.workload == "ep_bf16":
        return run_ep_workload(args, wl, rank, world, local)
    layer, n = wl.layer, wl.n
    ncopies = max(1, args.copies)
    copies = [Moe(layer, n, device=local) for _ in range(ncopies)]
    h = torch.from_numpy(wl.h).cuda()
    out = torch.empty_like(h)
    h_pin = torch.from_numpy(wl.h).pin_memory()
    out_pin = torch.empty_like(h_pin).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # a side stream: the library replays its launch sequence as a CUDA graph, which the
    # legacy default stream cannot capture
    # Passes rotate over `--streams` streams (layer object j on stream j mod streams): the
    # latency-bound routing kernels and the ramp and tail of one pass's expert kernels
    # overlap another's, as with a host that keeps several micro-batches in flight.
    # Measured at the decode shape: 94 us per pass alone, 77 with two in flight, 57 with
    # four.  `--quick` (the command profilers wrap) keeps one stream.
    nstreams = args.streams if (args.streams >= 1 and ncopies % max(1, args.streams) == 0 and not args.quick) else 1
    streams = [torch.cuda.Stream() for _ in range(nstreams)]
    outs = [out] + [torch.empty_like(h) for _ in range(nstreams - 1)]
    side = streams[0]
    torch.cuda.synchronize()
    torch.cuda.set_stream(side)

    def step(i):
        j = i % ncopies
        with torch.cuda.stream(streams[j % nstreams]):
            copies[j].moe_(h, outs[j % nstreams], accumulate=False)

    # every layer object needs three passes before it is warm (the second builds its graph)
    warmup = max(warmup, 3 * ncopies)
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    experts_hit = int((copies[0].tap(capi.TAP_COUNTS) > 0).sum())

    sampler = ClockSampler(local)
    sampler.start()
    # ---- timed region: exactly K steps between events on the launching stream
    barrier()
    l0 = launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(streams[0])
    for i in range(args.steps):
        step(i)
    for st in streams[1:]:      # the second event closes after both streams' work
        joined = torch.cuda.Event()
        joined.record(st)
        streams[0].wait_event(joined)
    e1.record(streams[0])
    barrier()
    launches = launch_count() - l0
    ms = e0.elapsed_time(e1)
    if args.quick:
        if rank == 0:
            print(json.dumps({"quick": True, "ms_per_step": ms / args.steps, "steps": args.steps}))
        return
    # ---- the same K steps one pass at a time on one stream (the latency figure)
    def step_alone(i):
        with torch.cuda.stream(streams[0]):
            copies[i % ncopies].moe_(h, outs[0], accumulate=False)

    for i in range(3 * ncopies):     # the layers' graphs are rebuilt for the new stream
        step_alone(i)
    barrier()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record(streams[0])
    for i in range(args.steps):
        step_alone(i)
    a1.record(streams[0])
    barrier()
    ms_alone = a0.elapsed_time(a1)
    # ---- end to end: host rows in, host delta out, through the host-buffer call.  Every
    #      step copies its rows in from page-locked memory and its result out.  First one
    #      pass at a time; then with two passes in flight on different layer objects
    #      (bivmoe_forward_host_async / bivmoe_host_wait), which lets the copies of one
    #      pass overlap the kernels of another - how a host with several micro-batches
    #      drives the layers.
    for i in range(3):
        copies[i % ncopies].moe_host(h_pin, out_pin)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        copies[i % ncopies].moe_host(h_pin, out_pin)
    torch.cuda.synchronize()
    e2e_sync_s = time.perf_counter() - t0
    depth = nstreams
    h_pins = [h_pin] + [torch.from_numpy(wl.h).pin_memory() for _ in range(depth - 1)]
    out_pins = [out_pin] + [torch.empty_like(h_pin).pin_memory() for _ in range(depth - 1)]

    def pipelined(count):
        for i in range(count):
            j = i % ncopies
            if i >= depth:
                copies[(i - depth) % ncopies].wait()
            copies[j].moe_host_async(h_pins[j % depth], out_pins[j % depth])
        for i in range(max(0, count - depth), count):
            copies[i % ncopies].wait()

    pipelined(3 * ncopies)      # each layer object sees its buffers twice: the graphs exist
    barrier()
    t0 = time.perf_counter()
    pipelined(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    # ---- the dominant kernel alone, events around each launch (separate loop so
    #      the events do not perturb the number above)
    k_ms, stage_ms = [], []
    for i in range(min(args.steps, 100)):
        prof = copies[i % ncopies].profile(h, out)
        k_ms.append(prof["gateup"])
        stage_ms.append(prof)
    # keep the clocks sampler fed for long enough to see the load
    t_end = time.perf_counter() + 0.5
    i = 0
    while time.perf_counter() < t_end:
        step(i)
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    sampler.stop_flag = True
    sampler.join()

    t = torch.tensor([ms, e2e_s * 1e3, e2e_sync_s * 1e3, ms_alone], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_sync_ms, ms_alone = float(t[0]), float(t[1]), float(t[2]), float(t[3])
    # ---- the same shape with the experts sharded over the GPUs instead of replicated:
    #      every rank passes its own n rows, rows travel to the experts' owners and back
    ep = None
    if world > 1 and layer.n_expert % world == 0:
        torch.cuda.set_stream(torch.cuda.default_stream())
        h_rank = np.random.default_rng(1000 + rank).standard_normal((n, layer.n_embd), dtype=np.float32)
        ep_ms, ep_recv, _ = time_ep(layer, h_rank, min(args.steps, 100), 5, rank, world, local,
                                    exchange=args.ep_exchange, graph=args.ep_graph)
        ep = {"value": world * n / (ep_ms * 1e-3), "unit": UNIT, "ms_per_step": ep_ms,
              "parallelism": f"ep{world}", "experts_per_gpu": layer.n_expert // world,
              "tokens_per_gpu": n, "exchange": args.ep_exchange,
              "graph_replay": bool(args.ep_graph and args.ep_exchange == "peer"),
              "note": ("experts sharded; rows and tags out and partial sums back as stores of the "
                       "library's kernels into the peers' memory, two one-element all-reduces per "
                       "pass as barriers" if args.ep_exchange == "peer" else
                       "experts sharded; per pass one count all-gather read by the host, rows and "
                       "tags out and partial sums back as NCCL all-to-alls") +
                      "; `value` above is the replicated (no-exchange) arrangement"}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak, tf_peak, peak_kind = load_peaks()
    ms_step = ms / args.steps
    value = world * n * args.steps / (ms * 1e-3)
    kbytes = gateup_bytes(layer, n, experts_hit)
    k_med = statistics.median(k_ms) if k_ms else None
    achieved = kbytes / (k_med * 1e-3) / 1e9 if k_med else None
    lbytes = algorithmic_bytes(layer, n, experts_hit)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32 block dots, f32 scales",
        "data": "synthetic", "config": config_of(wl, args, world),
        "one_pass_at_a_time": {"value": world * n * args.steps / (ms_alone * 1e-3), "unit": UNIT,
                               "ms_per_step": ms_alone / args.steps,
                               "note": "the same steps on one stream, each pass after the previous"},
        "roofline": {"bound": "hbm", "kernel": "experts_kernel<gate+up>", "achieved": achieved,
                     "peak": hbm_peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                     "frac": achieved / hbm_peak if achieved else None, "traffic": None,
                     "bytes_per_launch": kbytes, "kernel_ms": k_med, "experts_hit": experts_hit,
                     "stage_ms": {k: statistics.median(p[k] for p in stage_ms)
                                  for k in stage_ms[0]} if stage_ms else None,
                     "layer_bytes": lbytes,
                     "layer_frac": lbytes / (ms_step * 1e-3) / 1e9 / hbm_peak},
        "e2e": {"value": world * n * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": n * layer.n_embd * 4, "d2h_bytes_per_step": n * layer.n_embd * 4,
                "passes_in_flight": depth,
                "one_pass_at_a_time": world * n * args.steps / (e2e_sync_ms * 1e-3),
                "call": "bivmoe_forward_host_async + bivmoe_host_wait on page-locked buffers; every "
                        "step copies its rows in and its result out"},
        "gpu_launches": launches,
        "clocks": sampler.summary(),
    }
    if args.workload in ("prefill_q8_0", "ep_bf16") and stage_ms:
        # prefill-sized groups: the expert products are the dense contraction; report the
        # tensor-pipe roofline of the expert kernels (gate+up, SwiGLU, down) together
        st = line["roofline"]["stage_ms"]
        t_exp = (st["gateup"] + st["down"]) * 1e-3
        k, e, ff = layer.n_expert_used, layer.n_embd, layer.n_ff_exp
        ops = 2.0 * n * (k + (1 if layer.has_shared else 0)) * 3 * e * ff
        int8 = args.workload == "prefill_q8_0"
        peak = copies[0].int8_peak() if int8 else tf_peak
        line["roofline"] = {
            "bound": "tensor", "kernel": "experts_prefill_kernel (tcgen05 kind::i8)" if int8
            else "experts_prefill_bf16_kernel (tcgen05 kind::f16)",
            "achieved": ops / t_exp / 1e12, "peak": peak,
            "peak_kind": "int8 tensor pipe measured in this run (back-to-back tcgen05.mma kind::i8, "
                         "bivmoe_int8_peak)" if int8 else f"of {peak_kind}",
            "unit": "TOP/s" if int8 else "TFLOP/s", "frac": ops / t_exp / 1e12 / peak, "traffic": None,
            "kernel_ms": t_exp * 1e3, "stage_ms": st, "experts_hit": experts_hit,
            "note": "achieved counts the reference's multiply-adds once; the BF16 kernel issues "
                    "two MMAs per multiply-add (f32 rows as two bf16 terms)" if not int8 else
                    "every 32-wide block dot is one MMA whose int32 result is scaled in f32 by the "
                    "epilogue warps, which bound the kernel",
        }
        line["dtype"] = ("int8 x int8 -> int32 block dots, f32 scales" if int8
                         else "bf16 weights x f32 activations (two bf16 terms), f32 accumulation")
    if args.workload == "decode_q4k" and n == 64:
        # dram__bytes_read.sum + dram__bytes_write.sum of this kernel on this workload
        # (profiles/experts_kernel_decode_q4k.md)
        line["roofline"]["traffic"] = 108.0e6
        line["roofline"]["traffic_source"] = "ncu capture of the same command with one weight copy"
    if ep:
        line["ep"] = ep
    if not args.no_cpu:
        cpu, _ = time_cpu(wl)
        line["cpu_baseline"] = cpu
    for m in copies:
        m.close()
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
