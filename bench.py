#!/usr/bin/env python
"""Benchmark of the FP8 block-scaled MoE layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one pass of the whole layer (routing, dispatch, permute, GEMM1+SwiGLU+requant,
GEMM2, combine, and for N > 1 the NCCL sum of the partial outputs: reduce-scatter by default,
--collective all_reduce for replicated outputs) over one synthetic batch.
The default workload is the large-prefill configuration: T = 12288 tokens, all 256 experts,
split evenly over the N GPUs (N = 1 holds all 256 on one GPU).  Rank 0 prints ONE JSON line.

Timed on the device with CUDA events after W warm-up steps, max over ranks; the weights
(11.3 GB over all ranks) and activations are far larger than the 126 MB L2, so no explicit
flush is needed between iterations.  Seeded synthetic inputs stand in for recorded traces.

--impl reference runs the UNMODIFIED reference operator (oracle/_ref/libref_moe.so, built
from the reference's own sources by oracle/build_ref.sh) on the same GPU(s), workload and
metric: 32 experts per call, so (256/N)/32 sequential calls per rank whose bf16 outputs are
added, then the same NCCL sum.  If that library cannot be loaded, the CPU oracle port of the
layer is timed on the host cores instead and the line says so.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

H, I, N1, NE = 7168, 2048, 4096, 256
RSF = 2.5
FLOPS_PER_ROW = 2 * (H * N1 + I * H)          # 88,080,384
GEMM1_FLOPS_PER_ROW = 2 * H * N1              # 58,720,256
GEMM2_FLOPS_PER_ROW = 2 * I * H               # 29,360,128
FP8_NOMINAL_TFLOPS = 4500.0

WORKLOADS = {
    # name: (T, skew, experts in the layer, description)
    "t12288_e256": (12288, False, 256, "T=12288 prefill, 256 experts split over the GPUs, uniform routing"),
    "t16384_e256_skew": (16384, True, 256, "T=16384, 256 experts split over the GPUs, Zipf-like skewed routing"),
    "t1024_e256": (1024, False, 256, "T=1024 prefill, 256 experts split over the GPUs"),
    # single 32-expert shard (offset 0) on one GPU: the reference's native shape; also the small
    # cases used for ncu captures (1.4 GB of weights, well above the 126 MB L2)
    "t12288_e32": (12288, False, 32, "T=12288, one 32-expert shard (offset 0), 1 GPU"),
    "t1024_e32": (1024, False, 32, "T=1024, one 32-expert shard (offset 0), 1 GPU"),
    "t16_e32": (16, False, 32, "T=16, one 32-expert shard (offset 0), 1 GPU"),
}

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the dominant kernel
# (GEMM1) from the ncu capture summarised in profiles/gemm_t12288_e32_ncu_full.md: 928 MB for
# T = 12288 on one 32-expert shard.  Weights are 97 % of that traffic and are read exactly once,
# so for the other workloads the figure is scaled by (experts on the GPU) / 32.
NCU_GEMM1_DRAM_BYTES_32_EXPERTS_T12288 = 928.0e6


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def clocks_suspect(c) -> bool:
    if {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"} & set(c["reasons"]):
        return True
    return bool(c["sm_mhz"] and c["sm_max_mhz"] and c["sm_mhz"] < 0.85 * c["sm_max_mhz"] and not c["reasons"])


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def workload_config(name: str, experts_per_gpu: int) -> dict:
    """What was measured, in the same words for both arms (everything specific to an arm goes elsewhere)."""
    T, skew, experts_total, desc = WORKLOADS[name]
    return {"workload": name, "description": desc, "tokens": T, "experts_total": experts_total,
            "experts_per_gpu": experts_per_gpu, "routing": "skewed (Zipf-like)" if skew else "uniform",
            "reference_pruning": True,
            "l2": f"inputs larger than L2 (weights {experts_per_gpu * 44.04e-3:.1f} GB per GPU), no flush"}


def make_workload(name: str, rank: int, world: int):
    entry.load_package()
    from fp8_moe_dev_b200 import gen
    from fp8_moe_dev_b200.dist import expert_range
    T, skew, experts_total, _ = WORKLOADS[name]
    if experts_total == NE:
        offset, E = expert_range(rank, world)
    else:
        if world != 1:
            raise SystemExit(f"workload {name} is a single-shard case: run it with --gpus 1")
        offset, E = 0, experts_total
    logits, bias = gen.make_routing(T, seed=0, skew=skew)           # CPU streams: identical on every rank
    hidden, hscale = gen.make_hidden(T, seed=1)
    weights = gen.make_shard(offset, E, base_seed=1000, device="cuda", out_device="cuda")
    return T, offset, E, (logits, bias, hidden, hscale), weights


def time_steps(step, steps, warmup, world, drain=None):
    """`drain`: called after the warm-up and after the last timed step, for steps that return
    before their work is finished (it must block the host until everything issued is done)."""
    for _ in range(warmup):
        step()
    if drain:
        drain()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    if drain:
        drain()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world) / steps  # ms per step


def _event_times_us(fn, n):
    """Per-call device time of n calls of fn, each bracketed by its own pair of events."""
    times = []
    for _ in range(n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    return times


def small_config_latencies(pkg, weights, bias_dev, reference_mod=None):
    """Latency of the small single-shard configurations (rank 0, N = 1; 32 experts, offset 0) at
    T = 1, 16, 1024.  Ours: the whole layer (routing included) captured once into a CUDA graph,
    median of 1000 (T = 1) / 200 replays, plus the mean of back-to-back eager calls.  Reference:
    median of the same number of calls on identical pointers, i.e. its own steady state, in
    which it replays an internal CUDA graph and skips routing (kernel/moe_fp8.cu:2696-2702,
    2881-2916)."""
    from fp8_moe_dev_b200 import gen
    w1, s1, w2, s2 = [x[:32] for x in weights]
    out = []
    for T in (1, 16, 1024):
        logits, _ = gen.make_routing(T, seed=0)
        hidden, hscale = gen.make_hidden(T, seed=1)
        dev = [logits.cuda(), bias_dev, hidden.cuda(), hscale.cuda()]
        o = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
        reps = 1000 if T == 1 else 200
        # the shard (local_expert_offset) that holds the first token's best expert, so that
        # the T = 1 case has routed rows to compute; same weights tensor for every offset
        sb = torch.sigmoid(logits[0]) + bias_dev.float().cpu()
        gs = sb.view(8, 32).topk(2, dim=-1).values.sum(-1)
        keep = torch.zeros(8, dtype=torch.bool)
        keep[gs.topk(4).indices] = True
        off = int(sb.masked_fill(~keep.repeat_interleave(32), -1e30).argmax()) // 32 * 32 if T == 1 else 0
        if reference_mod is not None:
            run = lambda: reference_mod.run(*dev, w1, s1, w2, s2, off, RSF, o)  # noqa: E731
            for _ in range(5):
                run()
            torch.cuda.synchronize()
            lat = statistics.median(_event_times_us(run, reps))
            # fresh inputs: the same values in three rotating buffer sets, so that the
            # reference's pointer-keyed caches miss and it runs routing, its host read-back
            # and its descriptor set-up, as it must whenever the activations change
            sets = [[x.clone() for x in (dev[0], dev[2], dev[3])] + [torch.zeros_like(o)] for _ in range(3)]
            state = {"i": 0}

            def run_fresh():
                lg, hd, hs, oo = sets[state["i"] % 3]
                state["i"] += 1
                reference_mod.run(lg, dev[1], hd, hs, w1, s1, w2, s2, off, RSF, oo)
            for _ in range(6):
                run_fresh()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            n_fresh = 100
            for _ in range(n_fresh):
                run_fresh()
            torch.cuda.synchronize()
            fresh = (time.perf_counter() - t0) / n_fresh * 1e6
            out.append({"workload": f"T={T}, 32 experts, offset {off}", "latency_us": round(lat, 2),
                        "tokens_per_s": round(T / lat * 1e6, 1),
                        "fresh_inputs_latency_us": round(fresh, 2),
                        "how": f"median of {reps} calls on identical pointers (reference steady state: cached "
                               "routing, internal graph replay); fresh_inputs = mean wall time per call over "
                               f"{n_fresh} calls rotating three input buffer sets (its caches miss)"})
            continue
        layer = pkg.MoeLayer(T, 32, 0)
        run = lambda: layer.run(*dev, w1, s1, w2, s2, off, RSF, o)  # noqa: E731
        for _ in range(5):
            run()
        layer.check()
        rows = int(layer.read("pair_count", T).sum())
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                run()
        torch.cuda.current_stream().wait_stream(s)
        lat = statistics.median(_event_times_us(g.replay, reps))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(50):
            run()
        b.record()
        b.synchronize()
        eager = a.elapsed_time(b) * 1e3 / 50
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(100):
            run()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / 100 * 1e6
        timeline = None
        if T <= 8:
            # the decode kernel's own phase clock (CTA 0, ns), median over 20 eager runs
            import numpy as np
            names = ("tables", "phase1_gemm1_swiglu", "barrier1_wait", "phase2_requant_gemm2", "barrier2_wait", "combine")
            acc = []
            for _ in range(20):
                run()
                layer.check()
                tl = layer.read("decode_timeline", 8).astype(np.int64)
                acc.append(np.diff(tl[:7]))
            med = np.median(np.array(acc), axis=0)
            timeline = {n: round(float(v) / 1e3, 2) for n, v in zip(names, med)}
        active = int((layer.read("expert_count", 32) > 0).sum())
        wbytes = active * (N1 * H + H * I)
        gbs = wbytes / (lat * 1e-6) / 1e9
        pk = peaks()
        out.append({"workload": f"T={T}, 32 experts, offset {off}", "latency_us": round(lat, 2),
                    "eager_wall_us_per_call": round(wall, 2),
                    "tokens_per_s": round(T / lat * 1e6, 1), "routed_rows": rows, "active_experts": active,
                    "weight_bytes": wbytes,
                    "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                                 "frac": round(gbs / pk["hbm_gbs"], 4),
                                 "note": "algorithmic bytes = weights of the experts that received a row (44.04 MB "
                                         "each), each read once per call; whole-layer latency, routing included; "
                                         f"peak = copy bandwidth of MEASURED_PEAKS.json ({pk['source']})"},
                    "decode_kernel_timeline_us": timeline,
                    "eager_latency_us": round(eager, 2),
                    "how": f"median of {reps} CUDA-graph replays of the whole layer (routing included)"})
        layer.close()
    return out


def adjacent_ops(layer, T, dev, weights, offset):
    """The operators either side of the layer, timed alone on the bench workload: quantise-on-entry
    (HBM-bound: 2 B read + 1 B written per element, 4 B per 128-block) and the layer without its
    final combine (what a caller that finalises elsewhere pays)."""
    pk = peaks()
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    q = torch.empty(T, H, dtype=torch.float8_e4m3fn, device="cuda")
    sc = torch.empty(H // 128, T, dtype=torch.float32, device="cuda")
    qt = sorted(_event_times_us(lambda: layer.quantize_hidden(x, q, sc), 30)[5:])
    q_us = qt[len(qt) // 2]
    q_bytes = T * H * 3 + 4 * (H // 128) * T
    gbs = q_bytes / (q_us * 1e-6) / 1e9
    w1, s1, w2, s2 = weights
    ut = sorted(_event_times_us(lambda: layer.run_unfinalized(*dev, w1, s1, w2, s2, offset, RSF), 12)[3:])
    layer.check()
    return {"quantize_hidden": {"tokens": T, "latency_us": round(q_us, 2), "bytes": q_bytes,
                                "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"],
                                             "unit": "GB/s", "frac": round(gbs / pk["hbm_gbs"], 4)},
                                "note": "working set (3 B/element) fits L2 only below ~5800 tokens"},
            "run_unfinalized": {"tokens": T, "latency_us": round(ut[len(ut) // 2], 1)}}


def parity_vs_reference(got_rows, token_ids, inputs_dev, T, world, n_sample=256):
    """Outside the timed region: the rows `got_rows` (bf16 [n, 7168], this rank's output for the tokens
    `token_ids`) against the reference operator -- the fp32 sum of its eight 32-expert `run` calls on the
    same inputs, weights regenerated shard by shard -- for up to n_sample / world of those tokens.
    Returns the gate quantities of the parity tests; reduced over ranks by the caller."""
    sys.path.insert(0, str(ROOT / "tests"))
    import helpers as hp
    from fp8_moe_dev_b200 import gen
    try:
        mod = hp.reference_module()
    except Exception as ex:
        return {"unavailable": f"reference library not loadable: {ex}"[:200]}
    n = min(max(1, n_sample // world), len(token_ids))
    pick = torch.linspace(0, len(token_ids) - 1, n).round().long()
    toks = token_ids[pick].cuda()
    total = torch.zeros(n, H, device="cuda")
    rows_ref = 0
    logits, bias, hidden, hscale = inputs_dev
    part = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    keep_alive = []   # the reference caches a transposed copy of the weight scales BY POINTER: every shard's
    for s_ in range(NE // 32):   # scale tensors must keep their own addresses while it is in use
        w = gen.make_shard(32 * s_, 32, base_seed=1000, device="cuda", out_device="cuda")
        keep_alive.append((w[1], w[3]))
        mod.run(logits, bias, hidden, hscale, *w, 32 * s_, RSF, part)
        torch.cuda.synchronize()
        total += part[toks].float()
        rows_ref += int(hp.reference_dispatch_arrays(logits, bias, 32 * s_)["pair_n"].sum())
        del w
    got = got_rows[pick.cuda()].float()
    diff = (got - total).abs()
    return {"tokens_compared": n, "ratio": float((diff <= 1.0 + 0.3 * total.abs()).float().mean()),
            "rel_l2": float((got - total).norm() / (total.norm() + 1e-30)), "max_abs": float(diff.max()),
            "mean_abs": float(diff.mean()), "rows_ref": rows_ref}


def cpu_baseline(inputs, weights, sample_tokens=64):
    """Host fp32 dequantise-and-compute baseline (the layer's definition, oracle port), timed on
    a bounded sample: the first `sample_tokens` tokens against the first 32-expert shard."""
    orc = entry.load_oracle()
    logits, bias, hidden, hscale = inputs
    S = min(sample_tokens, logits.shape[0])
    w1, s1, w2, s2 = [x[:32] for x in weights]
    args = (logits[:S].numpy(), bias.view(torch.uint16).numpy(), hidden[:S].view(torch.uint8).numpy(),
            hscale[:, :S].contiguous().numpy(), w1.view(torch.uint8).cpu().numpy(), s1.cpu().numpy(),
            w2.view(torch.uint8).cpu().numpy(), s2.cpu().numpy(), 0, RSF)
    t0 = time.perf_counter()
    _, rows = orc.layer(*args, mode="fp32")
    dt = time.perf_counter() - t0
    rows_per_s = rows / dt if dt > 0 else 0.0
    return {"value": round(rows_per_s / 8.0, 3), "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"fp32 definition of the layer on the host: first {S} tokens x experts 0..31 "
                      f"({rows} routed rows, {dt:.2f} s incl. dequantising the touched experts); "
                      "tokens/s = rows/s / 8 rows per token"}


def run_ours(args, rank, world, local):
    pkg = entry.load_package()
    from fp8_moe_dev_b200.dist import ShardedMoe, combine_partials
    T, offset, E, inputs, weights = make_workload(args.workload, rank, world)
    dev = [x.cuda() for x in inputs]
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    per = (T + world - 1) // world
    scat = torch.empty(per, H, dtype=torch.bfloat16, device="cuda")
    moe, placement_ms = None, None
    if world > 1:
        # expert placement: the reference's contiguous blocks, or every world-th expert per rank (an equal
        # share of every routing group on every rank), or experts dealt by measured load; "auto" times
        # them and keeps the fastest
        from fp8_moe_dev_b200 import gen
        cands = {}
        # calibration of the load-aware placement: routed rows per expert of ANOTHER batch (same
        # distribution and routing bias, different seed), never of the batch that is timed
        cal_logits, _ = gen.make_routing(4096, seed=12345, skew=WORKLOADS[args.workload][1], skew_seed=0)
        loads = pkg.expert_loads(cal_logits.cuda(), dev[1], RSF)
        for place in (("contiguous", "balanced") if args.placement == "auto" else (args.placement,)):
            m = ShardedMoe(T, rank, world, local, placement=place, loads=loads)
            w = weights if place == "contiguous" else gen.make_experts(m.expert_ids, base_seed=1000, device="cuda",
                                                                         out_device="cuda")
            cands[place] = (m, w)
        if len(cands) > 1:
            placement_ms = {}
            for place, (m, w) in cands.items():
                try:
                    # both candidates are timed like the headline (same steps and warm-up), so that the
                    # contiguous figure stands beside the chosen one as a number of the same kind
                    placement_ms[place] = round(time_steps(lambda: m.run(*dev, *w, RSF, out, mode=args.collective,
                                                                          scatter_out=scat), args.steps, args.warmup, world), 4)
                    m.layer.check()
                except Exception as ex:   # a candidate that does not run is not a candidate
                    sys.stderr.write(f"placement {place} failed on rank {rank}: {ex}\n")
                    placement_ms[place] = float("inf")
            # every rank must take the same decision: a failure anywhere disqualifies the candidate everywhere
            for place in placement_ms:
                placement_ms[place] = max_over_ranks(placement_ms[place], world)
            best = min(placement_ms, key=placement_ms.get)
            placement_ms = {k: (None if v == float("inf") else v) for k, v in placement_ms.items()}
            for place in list(cands):
                if place != best:
                    cands[place][0].layer.close()
                    del cands[place]
            torch.cuda.empty_cache()
        (place, (moe, weights)), = cands.items()
        offset = moe.local_expert_offset
    w1, s1, w2, s2 = weights
    layer = moe.layer if moe else pkg.MoeLayer(T, E, local)

    def step(mode=args.collective):
        if mode == "fused" and moe:
            return moe.run_fused(*dev, w1, s1, w2, s2, RSF, scatter_out=scat)
        layer.run(*dev, w1, s1, w2, s2, offset, RSF, out)
        return combine_partials(out, mode, scatter_out=scat)

    contiguous_ms = placement_ms.get("contiguous") if placement_ms else None
    step()
    layer.check()
    rows_local = int(layer.read("pair_count", T).sum())
    rows_total = int(sum_over_ranks(rows_local, world))
    rows_max = int(max_over_ranks(rows_local, world))

    # A clock record that shows a thermal / hardware slowdown, or SM clocks well below the maximum with no
    # reason reported, does not count: the timed region is taken once more (all ranks decide together).
    remeasured = False
    for attempt in range(2):
        layer.set_stage_timing(True)
        with ClockSampler(local) as clk:
            ms = time_steps(step, args.steps, args.warmup, world)
        stages, timed_runs = layer.stage_times()
        layer.set_stage_timing(False)
        if attempt == 1 or max_over_ranks(1.0 if clocks_suspect(clk.summary()) else 0.0, world) == 0.0:
            break
        remeasured = True
    layer.check()
    if moe is not None and moe.placement == "contiguous":
        contiguous_ms = ms
    # the fused exchange's own clock (last timed step): how long this rank pushed, waited for its peers, reduced
    exchange = None
    if moe is not None and args.collective == "fused":
        import numpy as np
        tl = layer.read("exchange_timeline", 8).astype(np.int64)
        pc = layer.read("pair_count", T)
        lo_t, hi_t = min(rank * per, T), min(rank * per + per, T)
        remote_rows = int((pc > 0).sum() - (pc[lo_t:hi_t] > 0).sum())
        push_us, wait_us, reduce_us = (tl[1] - tl[0]) / 1e3, (tl[3] - tl[2]) / 1e3, (tl[4] - tl[3]) / 1e3
        gbs = remote_rows * H * 2 / max(push_us, 1e-3) / 1e3
        exchange = {"push_us_max": round(max_over_ranks(push_us, world), 1),
                    "wait_for_peers_us_max": round(max_over_ranks(wait_us, world), 1),
                    "wait_for_peers_us_min": round(-max_over_ranks(-wait_us, world), 1),
                    "reduce_us_max": round(max_over_ranks(reduce_us, world), 1),
                    "remote_rows_pushed_max": int(max_over_ranks(remote_rows, world)),
                    "nvlink_gbs_while_pushing_min": round(-max_over_ranks(-gbs, world), 1),
                    "note": "per rank from %globaltimer stamps inside combine_push_kernel / reduce_owned_kernel; the "
                            "wait is the time the owner step spent before every peer's rows had arrived (load imbalance "
                            "between the ranks shows up here, on the fast ranks)"}


    # end to end: per-step inputs start in pinned host memory, the result ends in host memory
    pin = [x.pin_memory() for x in (inputs[0], inputs[2], inputs[3])]
    host_out = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    host_out2 = torch.empty(T, H, dtype=torch.bfloat16).pin_memory() if world == 1 else None
    pipe = {"i": 0, "tickets": []}
    if world == 1:
        def e2e_sync_step():
            layer.run_host(pin[0], dev[1], pin[1], pin[2], w1, s1, w2, s2, offset, RSF, host_out)

        def e2e_step():
            # pipelined host path, two calls in flight: every step copies its inputs from pinned host
            # memory and lands its output in host memory.  Step i first waits for (reads) the output of
            # step i-2, whose host buffer it reuses, then issues its own call: while step i-1 computes,
            # step i's inputs come in and step i-2's output has gone out.
            i = pipe["i"]
            if i >= 2:
                layer.host_wait(pipe["tickets"][i - 2])
            pipe["tickets"].append(layer.run_host_async(pin[0], dev[1], pin[1], pin[2], w1, s1, w2, s2, offset, RSF,
                                                        host_out if i % 2 == 0 else host_out2))
            pipe["i"] = i + 1

        def e2e_drain():
            for t in pipe["tickets"][-2:]:
                layer.host_wait(t)
    else:
        host_outs = [host_out] + [torch.empty(T, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]

        def e2e_step():
            # every rank copies only its token slice over PCIe, the slices are replicated over NVLink; three
            # calls outstanding over three host output buffers: step i is issued, then the output of step
            # i-2 is awaited (read) -- one call copies in, one computes, one copies out
            i = pipe["i"]
            pipe["tickets"].append(moe.run_host_async(pin[0], dev[1], pin[1], pin[2], w1, s1, w2, s2, RSF,
                                                      host_outs[i % 3], mode=args.collective))
            if i >= 2:
                moe.host_wait(pipe["tickets"][i - 2])
            pipe["i"] = i + 1

        def e2e_drain():
            for t in pipe["tickets"][-2:]:
                moe.host_wait(t)
    e2e_sync_ms = None
    if args.skip_e2e:
        e2e_ms = float("nan")
    elif world == 1:
        e2e_ms = time_steps(e2e_step, max(10, args.steps // 2), 3, world, drain=e2e_drain)
        e2e_sync_ms = time_steps(e2e_sync_step, max(3, args.steps // 3), 2, world)
    else:
        try:
            e2e_ms = time_steps(e2e_step, max(10, args.steps // 2), 3, world, drain=e2e_drain)
        except Exception as ex:   # the device-resident number must not be lost to a host-path failure
            sys.stderr.write(f"end-to-end leg failed on rank {rank}: {ex}\n")
            e2e_ms = float("nan")
            args.skip_e2e = True
    h2d = sum(x.numel() * x.element_size() for x in pin) // world   # per rank: its token slice
    d2h = (host_out if (world == 1 or args.collective == "all_reduce") else scat).numel() * 2
    other_ms = None
    if world > 1:
        other_ms = {m: round(time_steps(lambda: step(m), max(5, args.steps // 2), 3, world), 4)
                    for m in ("fused", "reduce_scatter", "all_reduce") if m != args.collective}
        layer.check()

    # parity with the reference operator on the very tensors that were timed (outside the timed region)
    parity = None
    if not args.skip_parity:
        result = step()
        layer.check()
        if world == 1:
            rows_got, ids = out, torch.arange(T)
        else:
            lo = min(rank * per, T)
            hi = min(lo + per, T)
            rows_got = (result if args.collective != "all_reduce" else out[lo:hi])[:hi - lo]
            ids = torch.arange(lo, hi)
        par = parity_vs_reference(rows_got, ids, dev, T, world)
        if "unavailable" in par:
            parity = par
        else:
            parity = {"vs": "fp32 sum of the reference's eight 32-expert run() calls, same inputs",
                      "tokens_compared": int(sum_over_ranks(par["tokens_compared"], world)),
                      "ratio_atol1_rtol0.3": round(-max_over_ranks(-par["ratio"], world), 6),
                      "rel_l2": round(max_over_ranks(par["rel_l2"], world), 6),
                      "max_abs": round(max_over_ranks(par["max_abs"], world), 5),
                      "mean_abs": round(max_over_ranks(par["mean_abs"], world), 6),
                      "rows_ours": rows_total, "rows_ref": par["rows_ref"],
                      "reduction": "min ratio / max error over ranks; each rank compares tokens of its own output slice"}

    pk = peaks()
    g1_ms = max_over_ranks(stages["gemm1"], world)
    g1_flops = rows_max * GEMM1_FLOPS_PER_ROW  # the slowest rank's launch
    achieved = g1_flops / (g1_ms * 1e-3) / 1e12 if g1_ms > 0 else 0.0
    fp8_peak = 2.0 * pk["bf16_tflops_sustained"]
    line = {
        "metric": "moe_layer_tokens_per_s", "value": round(T / ms * 1e3, 1), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "latency_us": round(ms * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3 x e4m3 -> f32 accumulate, bf16 out", "data": "synthetic",
        "config": workload_config(args.workload, E),
        "run": {"routed_rows_total": rows_total, "routed_rows_max_rank": rows_max,
                "ideal_scaling_bound": round(rows_total / rows_max, 3) if rows_max else None,
                "collective": None if world == 1 else args.collective,
                "expert_placement": None if world == 1 else moe.placement,
                "expert_placement_note": None if world == 1 else
                    "contiguous = blocks of 256/N experts per rank (local_expert_offset = 256/N * rank, the "
                    "partition the layer's interface names); balanced = experts dealt by the routed rows of a "
                    "calibration batch drawn with another seed; auto keeps the faster of the two in a short trial",
                "placement_trial_ms": placement_ms, "contiguous_ms_per_step": contiguous_ms,
                "contiguous_tokens_per_s": round(T / contiguous_ms * 1e3, 1) if contiguous_ms else None,
                "other_collective_ms_per_step": other_ms, "exchange": exchange},
        # the same metric with the partition the layer's interface names (local_expert_offset = 256/N * rank),
        # whatever placement `value` was measured with
        "value_contiguous_placement": (round(T / contiguous_ms * 1e3, 1) if contiguous_ms else None) if world > 1
                                       else round(T / ms * 1e3, 1),
        "parity": parity,
        "clocks": dict(clk.summary(), remeasured=remeasured),
        "e2e": None if args.skip_e2e else {"value": round(T / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "sync_call_ms_per_step": None if e2e_sync_ms is None else round(e2e_sync_ms, 4),
                "path": "moe_fp8_b200_run_host_async + host_wait (C ABI, pinned host buffers, two calls in flight: copy-in of step "
                        "i+1 and copy-out of step i-1 overlap the compute of step i); sync_call_ms_per_step = one blocking "
                        "moe_fp8_b200_run_host per step" if world == 1
                        else ("ShardedMoe.run_host_async + host_wait (three calls in flight): pinned H2D of the rank's token slice, copy-engine "
                              "replication of the slice into every peer's input staging over NVLink (bounded flag hand-shake) + "
                              + ("moe_fp8_b200_run_reduce_scatter (peer stores)" if args.collective == "fused"
                                 else f"moe_fp8_b200_run + NCCL {args.collective}") + " + D2H of the rank's output slice; "
                              "bytes are per rank")},
        "gpu_launches": (6 if (world > 1 and args.collective == "fused") else 5) * args.steps * world,
        "stage_ms": {k: round(max_over_ranks(v, world), 4) for k, v in stages.items()},
        "layer_tflops": round(rows_max * FLOPS_PER_ROW / (ms * 1e-3) / 1e12, 1),
        "roofline": {"kernel": "grouped_gemm_kernel<1> (GEMM1 + SwiGLU + requant)", "bound": "tensor",
                     "achieved": round(achieved, 1), "peak": round(fp8_peak, 1), "unit": "TFLOP/s",
                     "frac": round(achieved / fp8_peak, 4) if fp8_peak else None,
                     "peak_note": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({pk['source']}); "
                                  f"nominal dense fp8 {FP8_NOMINAL_TFLOPS:.0f}",
                     "frac_of_nominal": round(achieved / FP8_NOMINAL_TFLOPS, 4),
                     "flops_per_launch": g1_flops, "avg_launch_ms": round(g1_ms, 4), "timed_launches": timed_runs,
                     "traffic": (NCU_GEMM1_DRAM_BYTES_32_EXPERTS_T12288 * E / 32) if T >= 8192 else None,
                     "traffic_note": "SCALED, not measured at this size: ncu dram bytes of GEMM1 at T=12288 on one "
                                     "32-expert shard (928 MB, weights 96 % of it and read once) x experts/32"},
    }
    if rank == 0 and world == 1:
        if not args.skip_small:
            line["configs"] = small_config_latencies(pkg, weights, dev[1])
        if not args.skip_small:
            line["adjacent_ops"] = adjacent_ops(layer, T, dev, weights, offset)
        if not args.skip_cpu:
            line["cpu_baseline"] = cpu_baseline(inputs, weights)
    layer.close()
    return line


def run_reference(args, rank, world, local):
    sys.path.insert(0, str(ROOT / "tests"))
    entry.load_package()
    from fp8_moe_dev_b200.dist import combine_partials
    import helpers as hp
    T, offset, E, inputs, weights = make_workload(args.workload, rank, world)
    try:
        mod = hp.reference_module()
    except Exception as ex:  # library missing or not loadable: time the CPU port instead
        if rank != 0:
            return None
        cb = cpu_baseline(inputs, weights)
        return {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
                "n_gpus": world, "steps": 1, "warmup": 0, "ms_per_step": None, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(args.workload, E),
                "run": {"note": f"reference GPU library unavailable ({ex}); CPU port timed"},
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    dev = [x.cuda() for x in inputs]
    w1, s1, w2, s2 = weights
    shards = E // 32
    parts = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(shards)]
    scat = torch.empty((T + world - 1) // world, H, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")

    def step():
        for s in range(shards):
            sl = slice(32 * s, 32 * s + 32)
            mod.run(dev[0], dev[1], dev[2], dev[3], w1[sl], s1[sl], w2[sl], s2[sl], offset + 32 * s, RSF, parts[s])
        out.copy_(parts[0])
        for s in range(1, shards):
            out.add_(parts[s])
        combine_partials(out, "reduce_scatter" if args.collective == "fused" else args.collective, scatter_out=scat)

    with ClockSampler(local) as clk:
        ms = time_steps(step, args.steps, args.warmup, world)
    val = round(T / ms * 1e3, 1)
    small = None
    if rank == 0 and world == 1 and not args.skip_small:
        small = small_config_latencies(None, weights, dev[1], reference_mod=mod)
    return {"impl": "reference", "configs": small, "metric": "moe_layer_tokens_per_s", "value": val, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
            "latency_us": round(ms * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "e4m3 x e4m3 -> f32 accumulate, bf16 out", "data": "synthetic",
            "config": workload_config(args.workload, E),
            "run": {"how": f"{shards} sequential reference calls of 32 experts per rank on identical pointers "
                           "(its pointer-keyed caches may hit), bf16 adds, then NCCL "
                           + ("reduce_scatter" if args.collective == "fused" else args.collective),
                    "expert_placement": "contiguous"},
            "clocks": clk.summary(),
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": 0, "kind": "reference",
                             "sample": "the reference's own GPU build (oracle/_ref/libref_moe.so) on the same "
                                       "B200(s), full workload; the reference has no CPU implementation"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="t12288_e256")
    ap.add_argument("--collective", choices=["fused", "reduce_scatter", "all_reduce"], default="fused",
                    help="how the ranks' partial outputs are summed for N > 1: reduce_scatter leaves rank r "
                         "with tokens [r*T/N, (r+1)*T/N) (the inverse of the all-gather that replicated the "
                         "inputs); all_reduce leaves every rank with all T tokens; fused gives the reduce_scatter "
                         "result with the exchange done by the combine kernel's own peer stores (the reference "
                         "arm uses NCCL reduce_scatter for it)")
    ap.add_argument("--placement", choices=["auto", "contiguous", "strided", "balanced"], default="auto",
                    help="N > 1: which experts a rank holds -- the reference's contiguous blocks of 256/N, every N-th "
                         "expert, experts dealt longest-first by the routed rows of the first 4096 tokens "
                         "(balanced), or the faster of contiguous and balanced in a short trial (auto; strided never won one)")
    ap.add_argument("--skip-small", action="store_true", help="skip the T=1/16/1024 single-shard latencies")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the host fp32 baseline")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--skip-parity", action="store_true", help="skip the comparison with the reference operator")
    args = ap.parse_args()
    if not args.skip_e2e:
        args.warmup = max(args.warmup, 3)
    rank, world, local = dist_setup(args.gpus)
    line = run_ours(args, rank, world, local) if args.impl == "ours" else run_reference(args, rank, world, local)
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
