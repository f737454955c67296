#!/usr/bin/env python3
"""Benchmark of the MOD-DiT attention layer (mask prediction + block-sparse attention) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload hunyuan]

One "step" is one attention-layer call at the workload's shape: pooled mask prediction (Q/K block
pooling, pooled map, M^T S, solve, line selection, mask, work lists) followed by the block-sparse
forward, all through the public `SparseAttentionWithMap` API.  Rank 0 prints one JSON line.

  value      kept-block TFLOP/s of the whole job with q/k/v resident in HBM (inputs, 2.1 GB at the
             HunyuanVideo shape, are far larger than L2, so nothing stays cached between steps)
  e2e        the same metric with q/k/v in pinned host memory: every step copies them to the device
             and copies the output back, inside the timed region
  roofline   the block-sparse forward kernel alone (CUDA events around its launches in the timed
             region) against the measured bf16 tensor peak
  cpu_baseline  the CPU oracle (`oracle/`) timed on the host cores on a bounded sample of the workload

With N > 1 (torchrun) heads are sharded over ranks: every rank holds a sequence shard of q/k/v, an
exchange over NVLink (this library's copy kernel storing straight into peer-mapped buffers) turns it into
a head shard, the path runs on the local heads and the output goes back the same way; total work is fixed
("strong" scaling).

`--impl reference` times the reference's own CPU path for this hot path (the oracle port of it: the
reference itself is Python that needs its checkout, which does not exist on the benchmark box).

`--sweep mass|reference` runs the specification's step-adaptive sweep instead: 50 denoising steps at the
workload's shape whose positional gain rises linearly from 0.2 to 1.0 of `--gain` (inputs regenerated per step
from seed 4000 + step, outside the timed regions), every step timed on its own.  `mass`: mean-pooled producer
and cumulative-mass selector every step, so the block sparsity follows the locality (about 60 % to 90 % with
the defaults, `--sweep-tau 0.4 --gain 1.1`).  `reference`: the reference's own schedule (dense warm-up steps,
exact replay map on the two collecting steps and on every predict_T-th step after them, top-k lines), which
gives the amortised cost of its refresh steps.  The line carries per-step arrays in `sweep`.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "mod-dit_b200"))

import torch  # noqa: E402

METRIC = "MOD-DiT attn layer effective TFLOP/s on kept blocks @115k tok bf16 (ms_per_step = layer ms; mask_pred_pct = mask-pred overhead %)"
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []               # (arrival time, line)
        self.thread = None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def mark_begin(self):
        self.t_begin = time.monotonic()

    def mark_end(self):
        self.t_end = time.monotonic()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        # samples inside the timed region; when the region is shorter than the sampling interval, the samples
        # taken under the same load since the sampler started (the warm-up steps directly before it)
        t0 = self.t_begin if self.t_begin is not None else 0.0
        t1 = self.t_end if self.t_end is not None else float("inf")
        inside = [line for t, line in self.lines if t0 <= t <= t1 + 0.05]
        window = "timed region"
        if not inside:
            inside = [line for t, line in self.lines if t <= t1 + 0.05]
            window = "warm-up + timed region (timed region shorter than the sampling interval)"
        for line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "window": window,
                "reasons": sorted(reasons)}


def make_state(cfg, heads_local, warmup_steps=2, producer="pooled", selector="topk_lines", tau=0.9):
    from MoD.mod.state import create_adaptive_mask_state
    T, Hh, Ww = cfg["grid"]
    video = T * Hh * Ww
    state = create_adaptive_mask_state(cfg["model_type"], heads_local, video, cfg["text_tokens"], Hh * Ww, T,
                                       warmup_steps=warmup_steps, top_k=cfg["top_k"], predict_T=cfg["predict_T"],
                                       threshold=1e-4, block_size=cfg["block_size"])
    state["score_producer"] = producer
    state["selector"] = selector
    state["mass_threshold"] = tau
    return state


def kept_flops(mask: torch.Tensor, block_size: int, head_dim: int) -> float:
    return float(mask.sum().item()) * 4.0 * block_size * block_size * head_dim


def bind_to_gpu_numa_node(local_rank: int):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, before any pinned buffer exists, so that
    the pinned pages (first touched here) are local to the GPU's PCIe root.  Returns what it found, for the record."""
    info = {"numa_node": None, "cpus": None}
    try:
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev_id = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev_id:02x}.0/numa_node"
        with open(path) as fh:
            node = int(fh.read().strip())
        info["numa_node"] = node
        if node >= 0:
            with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
                cpus = set()
                for part in fh.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = cpus & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["cpus"] = len(allowed)
    except Exception as exc:            # sysfs layout differs or affinity is not ours to set: leave things as they are
        info["error"] = repr(exc)[:120]
    return info


class Harness:
    """What both the default run and the sweep need: ranks, the workload, the re-shard plumbing and one layer call."""

    def __init__(self, args):
        import torch.distributed as dist
        from moddit_b200 import dist as mdist
        from moddit_b200 import ops, synth
        self.dist, self.mdist, self.ops, self.synth, self.args = dist, mdist, ops, synth, args
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if args.gpus > 1 else 1
        self.rank = int(os.environ.get("RANK", "0")) if self.world > 1 else 0
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0")) if self.world > 1 else 0
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.numa = bind_to_gpu_numa_node(self.local_rank) if self.world > 1 else {"numa_node": None}
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.cfg = synth.WORKLOADS[args.workload]
        self.H, self.D, self.bs = self.cfg["heads"], self.cfg["head_dim"], self.cfg["block_size"]
        if self.H % self.world:
            raise SystemExit(f"{self.H} heads do not divide over {self.world} GPUs")
        self.hb, self.he = mdist.shard_bounds(self.H, self.world, self.rank)
        self.gain = args.gain if args.gain is not None else self.cfg.get("gain", 2.0)
        self.logger = logging.getLogger("bench")
        self.logger.setLevel(logging.WARNING)
        T, Hh, Ww = self.cfg["grid"]
        self.N = T * Hh * Ww + self.cfg["text_tokens"]
        self.comm_stream = torch.cuda.Stream(device=self.dev) if self.world > 1 else None
        self.qk_stream = torch.cuda.Stream(device=self.dev) if self.world > 1 else None
        self.stepped = False            # a step has run: the re-shard buffers were last used before a closing barrier
        self.timeline = None            # a list while --timeline steps run: one dict of timing events per step
        self.resharder, self.value_group, self.reshard = None, None, "none"
        if self.world > 1:
            self._setup_resharder()

    def _setup_resharder(self):
        mdist, dist, dev = self.mdist, self.dist, self.dev
        if self.N % self.world:
            raise SystemExit(f"{self.N} tokens do not divide over {self.world} sequence shards")
        try:
            self.resharder = mdist.PeerResharder(self.H, self.N, self.D, torch.bfloat16, dev,
                                                 bulk_copy=self.args.bulk_copy)
            if self.args.narrow_ctas > 0:
                self.resharder.NARROW_CTAS = self.args.narrow_ctas
            if self.args.copy_streams > 0:
                self.resharder.COPY_STREAMS = self.args.copy_streams
            self.resharder.enable_pooling(self.bs)
            self.reshard = ("peer-memory copies (%s) + fused output scatter; query/key pooled on the sequence shards"
                            % {"dma": "copy engines", "kernel": "copy kernel", "narrow": "copy kernel on few CTAs"}[
                                self.args.bulk_copy])
            try:                   # one exchange up front: a box without peer DMA fails here, on every rank alike
                probe = torch.zeros(1, self.H, self.N // self.world, self.D, device=dev, dtype=torch.bfloat16)
                self.resharder.seq_to_head(probe, 2, channel=1)
                torch.cuda.synchronize(dev)
            except RuntimeError as exc:
                print(f"[bench] copy-engine peer copies unavailable ({exc!r}); using the copy kernel", file=sys.stderr)
                self.resharder.bulk_copy = "kernel"
                self.reshard = ("peer-memory copies (copy kernel) + fused output scatter; query/key pooled on the "
                                "sequence shards")
        except Exception as exc:   # symmetric memory unavailable on this box: NCCL all-to-all does the same exchange
            print(f"[bench] peer-memory re-shard unavailable ({exc!r}); using NCCL all-to-all", file=sys.stderr)
            self.resharder = None
            self.value_group = dist.new_group(backend="nccl")
            self.reshard = "NCCL all-to-all"

    def inputs(self, seed, gain):
        """What the caller of the layer holds: q, k, v of the local heads (one GPU) or its sequence shard of all
        heads (several GPUs, as a sequence-parallel pipeline would)."""
        q, k, v = self.synth.make_workload_qkv(self.args.workload, seed=seed, gain=gain, device=self.dev,
                                               head_begin=self.hb, head_end=self.he)
        if self.world > 1:
            out = tuple(self.mdist.head_to_seq(t) for t in (q, k, v))
            del q, k, v
            return out
        return q, k, v

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def layer(self, qs, ks, vs, step, state, use_dense=False):
        from MoD.mod.attn_mask import SparseAttentionWithMap
        world, dev, resharder, mdist = self.world, self.dev, self.resharder, self.mdist
        ready, scatter, qk_ready, pooled = None, None, None, None
        pooled_mode = state.get("score_producer") == "pooled" and not use_dense
        groups = 0
        if world > 1 and resharder is not None and pooled_mode and state.get("mask") is not None:
            groups = self.head_groups()
        if groups > 1:
            # query, key and value travel together, group of heads by group of heads, and the sparse forward is
            # launched per group behind that group's event: all but the first group's share of the exchange
            # runs beside the attention kernel
            main = torch.cuda.current_stream(dev)
            self.qk_stream.wait_stream(main)
            with torch.cuda.stream(self.qk_stream):
                (qh, kh, vh), group_ready = resharder.seq_to_head_groups([qs, ks, vs], [0, 1, 2], groups, channel=0,
                                                                         quiesced=self.stepped)
            pooled = resharder.pool_to_head(qs, ks, channel=0, quiesced=self.stepped)
            scatter = resharder.begin_output(channel=0, consumed=self.stepped)
            state["_head_groups"] = groups
            out, _ = SparseAttentionWithMap(qh, kh, vh, state, self.logger, current_step=step, pooled_qk=pooled,
                                            head_group_ready=group_ready, output_scatter=scatter)
            out = resharder.finish_output(channel=0) if out is None else resharder.head_to_seq(out, channel=0)
            self.stepped = True
            return out
        state.pop("_head_groups", None)
        marks = None
        if world > 1 and self.timeline is not None:
            marks = {k: torch.cuda.Event(enable_timing=True) for k in ("in", "v", "qk", "pool", "out")}
            marks["in"].record(torch.cuda.current_stream(dev))
        if world > 1:
            main = torch.cuda.current_stream(dev)
            self.comm_stream.wait_stream(main)
            with torch.cuda.stream(self.comm_stream):
                # value is not needed until the attention kernel: it travels while the mask is predicted
                # after the first call every rank has passed the barrier that closed the previous step (the output
                # exchange) with all its kernels done, so the barriers that would open this step's exchanges are skipped
                vs_h = (resharder.seq_to_head(vs, 2, channel=1, quiesced=self.stepped) if resharder is not None
                        else mdist.seq_to_head(vs, group=self.value_group))
                ready = marks["v"] if marks else torch.cuda.Event()
                ready.record(self.comm_stream)
            if resharder is not None:
                # the mask needs only block means of query and key: they are pooled on the sequence shards and
                # sent to the head owners, so the prediction runs while the rows themselves still travel
                self.qk_stream.wait_stream(main)
                with torch.cuda.stream(self.qk_stream):
                    qh, kh = resharder.seq_to_head_many([qs, ks], [0, 1], channel=0, quiesced=self.stepped)
                    qk_ready = marks["qk"] if marks else torch.cuda.Event()
                    qk_ready.record(self.qk_stream)
                if pooled_mode:
                    pooled = resharder.pool_to_head(qs, ks, channel=0, quiesced=self.stepped)
                    if marks:
                        marks["pool"].record(main)
                else:
                    main.wait_event(qk_ready)
                    qk_ready = None
                qs, ks = qh, kh
                # the pooling exchange above ended with a barrier on this stream: the previous output is consumed
                scatter = resharder.begin_output(channel=0, consumed=pooled_mode and self.stepped)
            else:
                qs, ks = mdist.seq_to_head(qs), mdist.seq_to_head(ks)
            vs = vs_h
            vs.record_stream(main)
        kw = {}
        if pooled is not None or qk_ready is not None:
            kw = dict(qk_ready=qk_ready, pooled_qk=pooled)
        out, _ = SparseAttentionWithMap(qs, ks, vs, state, self.logger, current_step=step, value_ready=ready,
                                        output_scatter=scatter, use_dense=use_dense, **kw)
        if world > 1:
            if resharder is None:
                out = mdist.head_to_seq(out)
            else:
                # sparse steps wrote their rows straight into the peers' buffers; dense steps did not
                out = resharder.finish_output(channel=0) if out is None else resharder.head_to_seq(out, channel=0)
                self.stepped = True
            if marks and resharder is not None and pooled_mode:
                marks["out"].record(main)
                self.timeline.append(marks)
        return out

    def head_groups(self):
        """Groups the local heads are delivered (and attended) in.  --head-groups 0 picks: two when a rank holds at
        least six heads (measured at 4 GPUs: 6.14 ms against 6.26 ms with one), else one - with fewer heads the
        pieces of the exchange get so small that their fixed cost outweighs the overlap (six groups of one head at
        4 GPUs: 6.71 ms)."""
        hp = self.H // self.world
        want = self.args.head_groups if self.args.head_groups > 0 else (2 if hp >= 6 else 1)
        return max(1, min(want, hp))

    def reduce(self, maxed, summed):
        vals = torch.tensor(maxed, device=self.dev, dtype=torch.float64)
        sums = torch.tensor(summed, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(vals, op=self.dist.ReduceOp.MAX)
            self.dist.all_reduce(sums, op=self.dist.ReduceOp.SUM)
        return vals.tolist(), sums.tolist()

    def workload_string(self):
        cfg = self.cfg
        return (f"{self.args.workload}: B=1 H={self.H} D={self.D} N={self.N} block={self.bs} top_k={cfg['top_k']} "
                f"pooled mask prediction every step")

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def run_ours(args):
    hx = Harness(args)
    ops, dev, world, rank = hx.ops, hx.dev, hx.world, hx.rank
    cfg, H, D, bs, N = hx.cfg, hx.H, hx.D, hx.bs, hx.N
    q_in, k_in, v_in = hx.inputs(1, hx.gain)
    state = make_state(cfg, hx.he - hx.hb)
    layer = lambda qs, ks, vs, step: hx.layer(qs, ks, vs, step, state)     # noqa: E731
    barrier = hx.barrier

    # two untimed priming steps fill the feature history (the first one runs dense attention)
    for step in range(2):
        layer(q_in, k_in, v_in, step)
    sampler = ClockSampler(hx.local_rank)
    if rank == 0:
        sampler.start()               # running before the warm-up so that short timed regions still get samples
    for i in range(args.warmup):
        layer(q_in, k_in, v_in, 2 + i)
    ops.raise_on_status(dev)

    # ---- value: inputs resident in HBM ------------------------------------------------------------
    # The timed region (exactly `steps` steps between a barrier + synchronize on both sides, maximum over ranks)
    # is run `repeats` times back to back - as many as make about a second of work, so that short multi-GPU
    # steps are not at the mercy of one scheduling hiccup and the clock sampler sees the load - and the median
    # repeat is the reported one; minimum and maximum are printed beside it.
    # Inside the timed regions only the dominant kernel is bracketed by events (its launches feed the roofline)
    # and every launch is counted; the per-stage breakdown comes from a few untimed steps afterwards, so that
    # two event records per entry-point call do not load the host while short multi-GPU steps are timed.
    step_no = 2 + args.warmup
    repeat_ms, repeat_attn, repeat_host, launches = [], [], [], 0
    repeats = 1
    r = 0
    sampler.mark_begin()
    while r < repeats:
        barrier()
        ops.stage_timing(True, only=("moddit_sparse_attn_fwd",))
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        host0 = time.perf_counter()
        for i in range(args.steps):
            layer(q_in, k_in, v_in, step_no)
            step_no += 1
        host_ms = (time.perf_counter() - host0) * 1e3       # what the host needed to queue the steps (no waiting)
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        attn = sum(t for _, t in ops.stage_records()) / args.steps
        launches = ops.launches_recorded()
        (ms_max, attn_max, host_max), _ = hx.reduce([ms, attn, host_ms], [0.0])
        repeat_ms.append(ms_max)
        repeat_attn.append(attn_max)
        repeat_host.append(host_max)
        if r == 0:
            want = args.repeats if args.repeats > 0 else int(min(25, max(1, -(-1000.0 // max(ms_max, 1e-3)))))
            repeats = max(1, want)
        r += 1
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    order = sorted(range(repeats), key=lambda i: repeat_ms[i])
    mid = order[(repeats - 1) // 2]
    total_ms, attn_ms = repeat_ms[mid], repeat_attn[mid]
    breakdown_steps = max(1, min(args.steps, 5))
    # one more step goes first, unrecorded: its attention kernel keeps the GPU busy while the host enqueues the
    # recorded steps, so that the events bracket kernels waiting in the queue and not the host's launch latency
    layer(q_in, k_in, v_in, step_no)
    ops.stage_timing(True)
    for i in range(breakdown_steps):
        layer(q_in, k_in, v_in, step_no + 1 + i)
    records = ops.stage_records()
    ops.stage_timing(False)
    ops.check_health(dev)
    timeline = None
    if args.timeline and world > 1 and hx.head_groups() == 1 and hx.resharder is not None:
        # where a step's time goes on this rank: milliseconds from the layer's first operation to the arrival of
        # value / query+key, to the end of the pooling exchange, and to the end of the output barrier
        hx.timeline = []
        ops.stage_timing(True, only=("moddit_sparse_attn_fwd",))
        for i in range(10):
            layer(q_in, k_in, v_in, step_no + 10 + i)
        torch.cuda.synchronize(dev)
        attn_tl = sum(t for _, t in ops.stage_records()) / 10
        ops.stage_timing(False)
        tl = {k: statistics.median(m["in"].elapsed_time(m[k]) for m in hx.timeline) for k in ("v", "qk", "pool", "out")}
        hx.timeline = None
        timeline = {"value_arrived_ms": round(tl["v"], 3), "query_key_arrived_ms": round(tl["qk"], 3),
                    "pooled_means_exchanged_ms": round(tl["pool"], 3), "output_barrier_done_ms": round(tl["out"], 3),
                    "attention_kernel_ms": round(attn_tl, 3),
                    "attention_started_ms": round(tl["out"] - attn_tl, 3), "rank": rank,
                    "note": "medians over 10 steps on rank 0, from the layer's first operation; attention_started "
                            "= output_barrier_done - attention_kernel, an upper bound (it includes the output barrier)"}

    mask = state["mask"]
    flops_local = kept_flops(mask, bs, D)
    per_head = 1.0 - mask.float().mean(dim=(1, 2))
    sparsity_local = float(per_head.mean().item())
    stage_ms = {}
    for name, ms in records:
        stage_ms[name] = stage_ms.get(name, 0.0) + ms
    copies = ("moddit_copy_rows", "moddit_copy_rows_dma")               # re-shard copies (N > 1 only)
    comm_ms = sum(stage_ms.get(name, 0.0) for name in copies) / breakdown_steps
    pred_ms = sum(ms for name, ms in stage_ms.items()
                  if name not in ("moddit_sparse_attn_fwd",) + copies) / breakdown_steps

    # ---- e2e: inputs in pinned host memory, output copied back ----------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    e2e_ms, h2d, d2h, h2d_gbs, d2h_gbs = 0.0, 0, 0, 0.0, 0.0
    if not args.no_e2e:
        # Double-buffered pipeline, as a serving loop would run it: step i's inputs are copied host->device
        # on one stream while step i-1 computes on the main stream and step i-2's output is copied back on
        # a third; every step still moves all of its inputs and its output inside the timed region.
        host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in (q_in, k_in, v_in)]
        host_out = [torch.empty(q_in.shape, dtype=q_in.dtype, pin_memory=True) for _ in range(2)]
        dev_in = [[torch.empty_like(t) for t in (q_in, k_in, v_in)] for _ in range(2)]
        h2d = sum(t.numel() * t.element_size() for t in host_in)
        d2h = host_out[0].numel() * host_out[0].element_size()
        main = torch.cuda.current_stream(dev)
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        out_done = [torch.cuda.Event() for _ in range(2)]
        for ev in in_free + out_done:
            ev.record(main)

        # the two copy directions alone, all ranks at once (what the host side of this box gives each GPU)
        barrier()
        c0, c1, c2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        c0.record()
        for d, h in zip(dev_in[0], host_in):
            d.copy_(h, non_blocking=True)
        c1.record()
        host_out[0].copy_(dev_in[0][0], non_blocking=True)
        c2.record()
        barrier()
        h2d_gbs = h2d / (c0.elapsed_time(c1) * 1e-3) / 1e9
        d2h_gbs = d2h / (c1.elapsed_time(c2) * 1e-3) / 1e9

        def e2e_step(i, step):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(in_free[b])                 # the step that last used this buffer has computed
                for d, h in zip(dev_in[b], host_in):
                    d.copy_(h, non_blocking=True)
                in_ready[b].record(s_in)
            main.wait_event(in_ready[b])
            if world > 1:
                # the output lives in the re-shard's own buffer, which the next step's kernels on the peers write
                # again: the copy of the previous output to the host has to be out of it first
                main.wait_event(out_done[1 - b])
            out = layer(dev_in[b][0], dev_in[b][1], dev_in[b][2], step)
            in_free[b].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                s_out.wait_event(out_done[b])               # host buffer b is free again
                host_out[b].copy_(out, non_blocking=True)
                out_done[b].record(s_out)
            out.record_stream(s_out)

        def drain():
            main.wait_stream(s_in)
            main.wait_stream(s_out)

        e2e_step(0, 100)
        e2e_step(1, 101)
        drain()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(e2e_steps):
            e2e_step(i, 102 + i)
        drain()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)

    # ---- the processors' prologue (norm + rotary + head-major layout + block means), timed on its own ------
    prologue = None
    if world == 1 and not args.no_e2e:
        prologue = time_prologue(ops, dev, H, D, N, cfg, bs)

    # ---- reduce over ranks ------------------------------------------------------------------------
    (e2e_ms, pred_ms, comm_ms, h2d_slow, d2h_slow, sp_max), sums = hx.reduce(
        [e2e_ms, pred_ms, comm_ms, -h2d_gbs, -d2h_gbs, float(per_head.max().item())],
        [flops_local, sparsity_local, float(launches), float(h2d), float(d2h), h2d_gbs, d2h_gbs])
    (_, sp_min_neg), _ = hx.reduce([0.0, -float(per_head.min().item())], [0.0])
    flops_total, sparsity_sum, launches_total, h2d_total, d2h_total, h2d_gbs_sum, d2h_gbs_sum = sums

    if rank == 0:
        peaks = load_peaks()
        ms_per_step = total_ms / args.steps
        value = flops_total / (ms_per_step * 1e-3) / 1e12
        e2e_value = flops_total / (e2e_ms / e2e_steps * 1e-3) / 1e12 if e2e_ms > 0 else None
        # roofline of the dominant kernel: kept flops of one launch on this rank / its average duration
        achieved = flops_local / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else 0.0
        peak = float(peaks["bf16_tflops"])
        roof = {"bound": "tensor", "kernel": "sparse_attn_fwd_kernel", "achieved": round(achieved, 2), "peak": peak,
                "peak_source": f"of {peaks['_source']} (burst)", "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                "frac_of_sustained": round(achieved / float(peaks["bf16_tflops_sustained"]), 4),
                "frac_of_nominal_2250": round(achieved / 2250.0, 4), "kernel_ms": round(attn_ms, 3),
                "flops_per_launch": flops_local, "traffic": load_traffic(args.workload, (hx.he - hx.hb) / H)}
        if world > 1 and hx.head_groups() > 1:
            roof["note"] = (f"{hx.head_groups()} launches per step, one per group of heads, overlapping at their ends "
                            "on streams of their own: kernel_ms spans them, from the first launch to the end of the "
                            "last, and flops_per_launch is the whole step's")
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(args.workload, cfg, N, hx.gain, world),
            "sparsity": round(sparsity_sum / world, 4),
            "sparsity_per_head": {"min": round(-sp_min_neg, 4), "max": round(sp_max, 4)},
            "reshard": hx.reshard,
            "timeline": timeline,
            "host_queue_ms_per_step": round(sorted(repeat_host)[len(repeat_host) // 2] / args.steps, 3),
            "repeats": {"n": repeats, "reported": "median", "ms_per_step_min": round(min(repeat_ms) / args.steps, 3),
                        "ms_per_step_max": round(max(repeat_ms) / args.steps, 3)},
            "mask_pred_ms": round(pred_ms, 3), "mask_pred_pct": round(100.0 * pred_ms / max(pred_ms + attn_ms, 1e-9), 2),
            "attn_ms": round(attn_ms, 3), "reshard_copy_ms": round(comm_ms, 3),
            "stage_ms_per_step": {n: round(ms / breakdown_steps, 4) for n, ms in sorted(stage_ms.items())},
            "clocks": clocks,
            "e2e": None if e2e_value is None else {
                "value": round(e2e_value, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms / e2e_steps, 3),
                "steps": e2e_steps, "h2d_bytes_per_step": int(h2d_total), "d2h_bytes_per_step": int(d2h_total),
                "copy_only_gbs_per_rank": {"h2d_slowest": round(-h2d_slow, 1), "h2d_mean": round(h2d_gbs_sum / world, 1),
                                           "d2h_slowest": round(-d2h_slow, 1), "d2h_mean": round(d2h_gbs_sum / world, 1),
                                           "note": "all ranks copying at once, no compute; pinned buffers allocated "
                                                   "after binding to the GPU's NUMA node"},
                "numa": hx.numa},
            "gpu_launches": int(launches_total),
            "roofline": roof,
        }
        if prologue is not None:
            peak_gbs = float(peaks["hbm_gbs"])
            prologue["peak"] = peak_gbs
            prologue["frac"] = round(prologue["achieved"] / peak_gbs, 4)
            line["prologue"] = prologue
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload, hx.gain, blocks=args.cpu_blocks)
        emit(line)
    hx.close()


def bench_config(workload, cfg, N, gain, world):
    """The `config` object both arms print: the workload, nothing that depends on which arm ran it."""
    return {"workload": f"{workload}: B=1 H={cfg['heads']} D={cfg['head_dim']} N={N} block={cfg['block_size']} "
                        f"top_k={cfg['top_k']} pooled mask prediction every step",
            "parallelism": f"head-sharded x{world}", "l2": "inputs larger than L2", "gain": gain, "seed": 1}


def run_sweep(args):
    """The specification's step-adaptive sweep (see the module docstring)."""
    hx = Harness(args)
    ops, dev, world, rank, cfg = hx.ops, hx.dev, hx.world, hx.rank, hx.cfg
    D, bs = hx.D, hx.bs
    steps = args.sweep_steps
    ref_mode = args.sweep == "reference"
    warm = 12 if ref_mode else 1
    state = make_state(cfg, hx.he - hx.hb, warmup_steps=max(warm, 2) if ref_mode else 2,
                       producer="replay" if ref_mode else "pooled",
                       selector="topk_lines" if ref_mode else "cumulative_mass", tau=args.sweep_tau)
    predict_T = cfg["predict_T"]
    sampler = ClockSampler(hx.local_rank)
    if rank == 0:
        sampler.start()
    # untimed: load every kernel once (a dense call and, in mass mode, a predicted call on the first step's input)
    g0 = hx.gain * 0.2
    q_in, k_in, v_in = hx.inputs(4000, g0)
    scratch = make_state(cfg, hx.he - hx.hb, producer=state["score_producer"], selector=state["selector"],
                         tau=args.sweep_tau)
    for s_ in range(3):
        hx.layer(q_in, k_in, v_in, s_, scratch)
    del scratch
    ops.check_health(dev)
    rows = []
    sampler.mark_begin()
    for step in range(steps):
        frac = 0.2 + 0.8 * step / max(steps - 1, 1)
        del q_in, k_in, v_in
        q_in, k_in, v_in = hx.inputs(4000 + step, hx.gain * frac)
        if ref_mode:
            regime = ("dense" if step < warm - 2 else "collect" if step < warm else
                      "refresh" if (step - warm) % predict_T == predict_T - 1 else "sparse")
        else:
            regime = "dense" if step == 0 else "sparse"      # the first call has no feature history yet
        hx.barrier()
        ops.stage_timing(True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # A step is timed alone (its inputs are new), so the GPU would sit idle while the host enqueues the step's
        # launches one by one and the events would measure the host.  A few milliseconds of busy-waiting on the
        # device go first, untimed: the step's kernels queue up behind them as they would behind the previous
        # layer of a running pipeline.
        torch.cuda._sleep(int(args.sweep_lead_ms * 1.0e-3 * 1.5e9))
        e0.record()
        hx.layer(q_in, k_in, v_in, step, state, use_dense=(ref_mode and regime == "dense"))
        e1.record()
        hx.barrier()
        ms = e0.elapsed_time(e1)
        stage = {}
        for name, t in ops.stage_records():
            stage[name] = stage.get(name, 0.0) + t
        ops.stage_timing(False)
        attn = stage.get("moddit_sparse_attn_fwd", 0.0)
        copies = stage.get("moddit_copy_rows", 0.0) + stage.get("moddit_copy_rows_dma", 0.0)
        replay = stage.get("moddit_replay_map", 0.0)
        pred = sum(stage.values()) - attn - copies
        mask = state.get("mask")
        if regime in ("dense", "collect", "refresh") or mask is None:
            nb = -(-hx.N // bs)
            flops = float(hx.he - hx.hb) * nb * nb * 4.0 * bs * bs * D       # these steps run dense attention
            sparsity = 0.0
        else:
            flops = kept_flops(mask, bs, D)
            sparsity = 1.0 - float(mask.float().mean().item())
        (ms, attn, pred, replay), (flops, sparsity) = hx.reduce([ms, attn, pred, replay], [flops, sparsity])
        rows.append(dict(step=step, gain=round(hx.gain * frac, 4), regime=regime, ms=round(ms, 3),
                         sparsity=round(sparsity / world, 4), tflops=round(flops / (ms * 1e-3) / 1e12, 1),
                         attn_ms=round(attn, 3), mask_pred_ms=round(pred, 3), replay_ms=round(replay, 3),
                         mask_pred_pct=round(100.0 * pred / max(pred + attn, 1e-9), 2)))
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    ops.check_health(dev)
    if rank == 0:
        def stats(key, pick):
            vals = sorted(r_[key] for r_ in rows if pick(r_))
            if not vals:
                return None
            return {"min": vals[0], "median": vals[len(vals) // 2], "max": vals[-1], "n": len(vals)}
        sparse = lambda r_: r_["regime"] == "sparse"          # noqa: E731
        total_ms = sum(r_["ms"] for r_ in rows)
        kept_tf = sum(r_["tflops"] * r_["ms"] * 1e-3 for r_ in rows)
        line = {
            "metric": METRIC, "value": round(kept_tf / (total_ms * 1e-3), 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": steps, "warmup": 3, "ms_per_step": round(total_ms / steps, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload} sweep: B=1 H={hx.H} D={D} N={hx.N} block={bs}, {steps} steps, "
                                   f"positional gain {hx.gain} x lerp(0.2, 1.0), seed 4000 + step",
                       "mode": ("reference schedule: dense warm-up, exact replay map on collecting and refresh steps, "
                                f"top_k={cfg['top_k']} lines, predict_T={predict_T}, warmup_steps={warm}") if ref_mode else
                               f"mean-pooled producer + cumulative-mass selector (tau={args.sweep_tau}) every step",
                       "parallelism": f"head-sharded x{world}", "l2": "inputs larger than L2 and regenerated per step"},
            "reshard": hx.reshard, "clocks": clocks,
            "sweep": {"total_ms": round(total_ms, 2),
                      "sparse_steps": {"sparsity": stats("sparsity", sparse), "ms": stats("ms", sparse),
                                       "tflops": stats("tflops", sparse), "mask_pred_pct": stats("mask_pred_pct", sparse),
                                       "mask_pred_ms": stats("mask_pred_ms", sparse)},
                      "ms_by_regime": {name: stats("ms", lambda r_, name=name: r_["regime"] == name)
                                       for name in ("dense", "collect", "refresh", "sparse")},
                      "per_step": {key: [r_[key] for r_ in rows] for key in
                                   ("gain", "regime", "sparsity", "ms", "tflops", "mask_pred_pct", "attn_ms",
                                    "mask_pred_ms", "replay_ms")}},
        }
        if ref_mode:
            by = {name: [r_["ms"] for r_ in rows if r_["regime"] == name] for name in ("dense", "collect", "refresh", "sparse")}
            mean = lambda xs: sum(xs) / len(xs) if xs else 0.0          # noqa: E731
            after = [r_ for r_ in rows if r_["step"] >= warm]
            line["sweep"]["after_warmup"] = {
                "steps": len(after), "ms_per_step": round(mean([r_["ms"] for r_ in after]), 3),
                "sparse_ms_mean": round(mean(by["sparse"]), 3), "refresh_ms_mean": round(mean(by["refresh"]), 3),
                "refresh_share_of_time_pct": round(100.0 * sum(by["refresh"]) / max(sum(r_["ms"] for r_ in after), 1e-9), 2)}
        emit(line)
    hx.close()


def time_prologue(ops, dev, H, D, N, cfg, bs, reps=10):
    """Times moddit_qkv_prologue at the workload's shape (RMS norm per head, rotary on the video tokens, block
    means as a by-product) on synthetic token-major projections: not part of the timed step, reported beside
    it as an HBM-bound kernel (algorithmic bytes = q, k, v read once and written once)."""
    g = torch.Generator(device=dev).manual_seed(7)
    fused = torch.randn(1, N, 3 * H * D, device=dev, dtype=torch.bfloat16, generator=g)
    qi, ki, vi = fused.split(H * D, dim=2)
    weights = [torch.ones(D, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    text = cfg["text_tokens"]
    lo, hi = (text, N) if cfg["text_first"] else (0, N - text)
    ang = torch.rand(hi - lo, D // 2, device=dev, generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()        # one value per rotated pair
    pool_bs = bs if lo % bs == 0 else 0
    kw = dict(num_heads=H, norm="rms_head", q_weight=weights[0], k_weight=weights[1], rope_cos=cos, rope_sin=sin,
              rope_form="pair", rope_range=(lo, hi), pool_block_size=pool_bs)
    out, pools = ops.qkv_prologue(qi, ki, vi, **kw)

    def call():
        ops.qkv_prologue(qi, ki, vi, out=out, pools=pools, **kw)
    for _ in range(3):
        call()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / reps
    nbytes = 2 * 3 * N * H * D * 2 + 2 * (hi - lo) * (D // 2) * 4        # q, k, v in and out + the tables once
    return {"kernel": "qkv_prologue_kernel", "bound": "hbm", "ms": round(ms, 4), "bytes_per_launch": nbytes,
            "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
            "workload": f"norm=rms_head rotary=[{lo},{hi}) block means={'yes' if pool_bs else 'no'}; inputs "
                        f"{3 * N * H * D * 2 / 1e9:.2f} GB (larger than L2)"}


def load_traffic(workload, head_share=1.0):
    """DRAM bytes per launch of the sparse forward from the committed ncu summary (all heads of the workload;
    a rank holding `head_share` of the heads moves that share: traffic follows tensor bytes), or None."""
    path = os.path.join(ROOT, "profiles", f"sparse_attn_fwd_{workload}_traffic.json")
    if os.path.exists(path):
        with open(path) as fh:
            total = json.load(fh).get("dram_bytes_per_launch")
        return None if total is None else float(total) * head_share
    return None


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference path on the host cores
# ---------------------------------------------------------------------------------------------

def _load_synth():
    """The synthetic generator alone (pure torch), without importing the kernel package."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "moddit_synth_standalone", os.path.join(ROOT, "mod-dit_b200", "moddit_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_CPU_INPUTS = {}


def cpu_sample(workload: str, gain: float, blocks: int):
    """One head of the workload on the CPU: full mask prediction, then `blocks` query blocks of fp32
    block-masked attention.  Returns (kept flops of those blocks, seconds, description)."""
    synth = _load_synth()
    from oracle import moddit_oracle as orc
    cfg = synth.WORKLOADS[workload]
    D, bs = cfg["head_dim"], cfg["block_size"]
    T, Hh, Ww = cfg["grid"]
    key = (workload, gain)
    if key not in _CPU_INPUTS:      # inputs are made once, outside every timed region
        _CPU_INPUTS[key] = synth.make_workload_qkv(workload, seed=1, gain=gain, device="cpu", head_begin=0, head_end=1)
    q, k, v = _CPU_INPUTS[key]
    N = q.shape[2]
    video = T * Hh * Ww
    bpf = (Hh * Ww) // bs
    _, n, off = orc.block_geometry(cfg["model_type"], bs, video, cfg["text_tokens"], N)
    t0 = time.perf_counter()
    feats = []
    for rep in range(2):   # two feature sets are needed before a mask exists; both are part of the path
        dark = orc.pooled_darkness_map(orc.pool_blocks(q, bs), orc.pool_blocks(k, bs), q_block_offset=off,
                                       k_block_offset=off, video_blocks=n, scale=D ** -0.5)[0]
        f = orc.solve_features(orc.compute_mts(dark, bpf), n, bpf, 1.0)
        feats.append({key: f[key] for key in ("c", "d", "b_d")})
    lines = orc.choose_topk_lines(feats[0], feats[1], cfg["top_k"], cfg["predict_T"])
    mask = orc.generate_mask_from_lines(model_type=cfg["model_type"], block_size=bs, video_token_num=video,
                                        text_token_num=cfg["text_tokens"], seq_len=N, blocks_per_frame=bpf,
                                        selected_lines=lines, mode=orc.check_bd_values(feats[1]["b_d"], 1.0))
    t_pred = (time.perf_counter() - t0) / 2.0          # one prediction per step
    nbt = mask.shape[-1]
    rows = [int(i * nbt / blocks) for i in range(blocks)]
    t1 = time.perf_counter()
    orc.masked_attention(q, k, v, mask, bs, row_blocks=rows)
    t_attn = time.perf_counter() - t1
    flops = float(mask[0, rows].sum().item()) * 4.0 * bs * bs * D
    seconds = t_attn + t_pred * blocks / nbt
    desc = (f"1 of {cfg['heads']} heads: mask prediction ({t_pred:.2f} s per head, charged {blocks}/{nbt}) + {blocks} of "
            f"{nbt} query blocks of fp32 block-masked attention ({t_attn:.2f} s); oracle port of the reference CPU path")
    return flops, seconds, desc


def cpu_baseline(workload, gain, blocks):
    torch.set_num_threads(os.cpu_count() or 1)
    flops, seconds, desc = cpu_sample(workload, gain, blocks)
    return {"value": round(flops / seconds / 1e12, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "port", "sample": desc, "seconds": round(seconds, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = _load_synth().WORKLOADS[args.workload]
    gain = args.gain if args.gain is not None else cfg.get("gain", 2.0)
    for _ in range(args.warmup):
        cpu_sample(args.workload, gain, 1)
    tot_f, tot_s, desc = 0.0, 0.0, ""
    for _ in range(args.steps):
        f, s, desc = cpu_sample(args.workload, gain, args.ref_blocks)
        tot_f += f
        tot_s += s
    value = tot_f / tot_s / 1e12
    T, Hh, Ww = cfg["grid"]
    N = T * Hh * Ww + cfg["text_tokens"]
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(tot_s / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.workload, cfg, N, gain, args.gpus),
        "note": "each step is a bounded sample of the workload on the host cores (see cpu_baseline.sample)",
        "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": desc},
        "e2e": {"value": round(value, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


_RESULT_OUT = None


def keep_stdout_for_the_result():
    """The result line must be the only thing on standard output, but libraries write there too (NCCL prints
    its version on the first collective): point file descriptor 1 at standard error for everybody else and
    keep a private handle on the real standard output for `emit`."""
    global _RESULT_OUT
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(record) -> None:
    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(record) + "\n")
    out.flush()


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", default="hunyuan")
    ap.add_argument("--gain", type=float, default=None,
                    help="strength of the positional term of the synthetic q/k (default: the workload's, 2.0; 1.1 "
                         "for --sweep mass)")
    ap.add_argument("--repeats", type=int, default=0,
                    help="how often the timed region runs (0: as often as makes about a second, at most 25)")
    ap.add_argument("--sweep", choices=("mass", "reference"), default=None,
                    help="run the 50-step locality sweep instead of the fixed-input benchmark")
    ap.add_argument("--sweep-steps", type=int, default=50)
    ap.add_argument("--sweep-lead-ms", type=float, default=6.0,
                    help="device busy-wait before each timed sweep step, so that its launches are queued, not awaited")
    ap.add_argument("--sweep-tau", type=float, default=0.4, help="cumulative-mass threshold of --sweep mass")
    ap.add_argument("--e2e-steps", type=int, default=20,
                    help="steps of the host-buffer leg (at most --steps); the two-deep copy pipeline fills and drains "
                         "inside its timed region, about one step's worth of time whatever the count")
    ap.add_argument("--cpu-blocks", type=int, default=480, help="query blocks in the cpu_baseline sample")
    ap.add_argument("--ref-blocks", type=int, default=32, help="query blocks per step of --impl reference")
    ap.add_argument("--bulk-copy", choices=("dma", "kernel", "narrow"), default="dma",
                    help="several GPUs: how the sequence->head pieces travel, copy engines (no SM taken) or this "
                         "library's copy kernel (plain peer stores)")
    ap.add_argument("--narrow-ctas", type=int, default=0, help="CTAs of one exchange with --bulk-copy narrow")
    ap.add_argument("--timeline", action="store_true",
                    help="several GPUs, one head group: ten extra steps with events at the arrival of the inputs and the "
                         "end of the step")
    ap.add_argument("--copy-streams", type=int, default=0, help="side streams of one exchange with --bulk-copy dma")
    ap.add_argument("--head-groups", type=int, default=0,
                    help="several GPUs: the sequence->head exchange delivers the local heads in this many groups and "
                         "the sparse forward is launched per group as it arrives (1: one exchange, one launch; "
                         "0: two when a rank holds six heads or more, else one)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--prologue-only", action="store_true",
                    help="time only the processors' prologue kernel at the workload's shape and print its record")
    args = ap.parse_args()
    if args.prologue_only:
        from moddit_b200 import ops, synth
        cfg = synth.WORKLOADS[args.workload]
        torch.cuda.set_device(0)
        N = cfg["grid"][0] * cfg["grid"][1] * cfg["grid"][2] + cfg["text_tokens"]
        rec = time_prologue(ops, torch.device("cuda", 0), cfg["heads"], cfg["head_dim"], N, cfg, cfg["block_size"],
                            reps=max(args.steps, 1))
        peak = float(load_peaks()["hbm_gbs"])
        rec.update(peak=peak, frac=round(rec["achieved"] / peak, 4))
        emit(rec)
    elif args.impl == "reference":
        run_reference(args)
    elif args.sweep:
        if args.gain is None and args.sweep == "mass":
            args.gain = 1.1
        run_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
