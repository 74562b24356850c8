#!/usr/bin/env python
"""Benchmark of the Q4(+LoRA) linear hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (config.workload): the large-layer decode set
- per "layer" the four projections 5120->5120, 5120->1024, 5120->17408, 17408->5120 with Q4
weights quantized from N(0, 0.02^2) and a LoRA adapter of rank 16 on every projection, one
token (M = 1) - repeated over `--layers` layers with distinct weights (4 x 131 MB by default,
several times the 126 MB L2, so every launch streams its weights from HBM).  One step is one
pass over all of them.  metric = weight-streaming rate in GB/s on ALGORITHMIC bytes
(payload + LoRA factors + x + y, each once); with N GPUs the output rows of every projection
are sharded over the ranks and every rank ends the step with all ranks' columns (published
into every rank's step buffer by the step kernel itself; `--gather nccl` uses an NCCL
all-gather per set instead).

A step is ONE lq4_decode_step launch (`--launch step`, the default).  The device-timed leg
issues the K steps back to back as replays of a CUDA graph of up to `--graph-steps`
consecutive steps (a decode loop's queue: a step's weight stream starts while the step before
it drains); the end-to-end leg replays one step per graph through lq4_decode_step_host
(pinned inputs staged in by a kernel, results stored to pinned memory by the step kernel) and
waits for it every step.

Data are seeded synthetic tensors of those shapes (no dataset exists for this path).
The reference arm (--impl reference) times the CPU restatement of the reference's own
path (pre-dequantized f32 weights -> matmul_bt -> apply_lora) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

METRIC = "Q4 linear weight GB/s at M=1 (large-layer decode set, LoRA r=16)"
UNIT = "GB/s"
LORA_RANK, LORA_ALPHA = 16, 32.0
SHAPES = [(5120, 5120), (5120, 1024), (5120, 17408), (17408, 5120)]      # (k, n)
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu capture of
# `python bench.py --only decode-set` / `--only decode-step` (None: not captured for the current kernel).
# A capture belongs to the kernel source it was taken on: the entry carries the hash of the kernel files
# (kernel_source_hash below) at capture time, and the figure is reported only while that still matches.
NCU_TRAFFIC = {
    "grouped": {"bytes_per_launch": 138.64e6, "kernel": "decode_kernel<1, 8>", "source_hash": None},
    "per-projection": {"bytes_per_launch": None, "kernel": "decode_kernel<1, 1>", "source_hash": None},
    "step": {"bytes_per_launch": 553.74e6, "kernel": "decode_step_kernel<false>", "source_hash": "ed2396357ff09d6d"},
}


def kernel_source_hash(files=("lq4_decode.cu", "lq4_decode_common.cuh", "lq4_step.cu", "lq4_step.cuh", "lq4_common.cuh")):
    import hashlib
    h = hashlib.sha256()
    for f in files:
        p = os.path.join(ROOT, "lattice_b200", "csrc", f)
        if os.path.exists(p):
            h.update(open(p, "rb").read())
    return h.hexdigest()[:16]


def ncu_traffic(launch):
    """(bytes per launch or None, note): the captured DRAM traffic if it was taken on the current kernel source."""
    e = NCU_TRAFFIC.get(launch) or {}
    if e.get("bytes_per_launch") is None:
        return None, "not captured"
    if e.get("source_hash") != kernel_source_hash():
        return None, f"captured on an earlier version of {e['kernel']} ({e['bytes_per_launch'] / 1e6:.2f} MB per launch then)"
    return e["bytes_per_launch"], f"ncu capture of {e['kernel']} on this kernel source"


def algorithmic_bytes(m, n, k, rank):
    return n * (k // 32) * 20 + 4 * rank * (k + n) + m * k * 4 + m * n * 4


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0)), float(d.get("bf16_tflops_sustained", 0)), "measured"
    return FALLBACK_HBM_GBS, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons (every 100 ms, with the host time each sample was read)
    while the process measures; `window(t0, t1)` summarises the samples that fall into a timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.samples = []          # (host time, sm MHz, max sm MHz, set of active reasons)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            reasons = {n for n, v in zip(self.NAMES, f[5:9]) if v.lower().startswith("active")}
            self.samples.append((time.time(), sm, mx, reasons))

    def window(self, t0: float, t1: float):
        """Clocks seen in the host-time window [t0, t1] (widened by one sampling period on both sides, since a
        timed region may be shorter than the period)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if time.time() < t1 + 0.12:
            time.sleep(max(0.0, t1 + 0.12 - time.time()))
        pick = [x for x in self.samples if t0 - 0.11 <= x[0] <= t1 + 0.11]
        if not pick:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        reasons = set()
        for x in pick:
            reasons |= x[3]
        sm = [x[1] for x in pick]
        return {"sm_mhz": float(np.median(sm)), "sm_min_mhz": float(min(sm)), "sm_max_mhz": float(max(x[2] for x in pick)),
                "reasons": sorted(reasons), "samples": len(pick)}

    def stop(self):
        if not self.proc:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()


# ----------------------------------------------------------------------------- reference arm
def cpu_token_set(threads: int, layer):
    """One token-set on the CPU oracle: per projection matmul_bt over pre-dequantized f32 weights
    followed by apply_lora, output rows split over `threads` host threads."""
    import oracle
    from concurrent.futures import ThreadPoolExecutor

    def part(job):
        x, w, a, b, scale, n0, n1, k = job
        y = oracle.matmul_bt(x, w[n0:n1], 1, k, n1 - n0)
        out = np.ascontiguousarray(y[0])
        oracle.apply_lora(a, b[n0:n1], LORA_RANK, k, n1 - n0, scale, x[0], out)
        return out

    jobs = []
    for (k, n), (x, w, a, b, scale) in zip(SHAPES, layer):
        for t in range(threads):
            jobs.append((x, w, a, b, scale, n * t // threads, n * (t + 1) // threads, k))
    if threads == 1:
        return [part(j) for j in jobs]
    with ThreadPoolExecutor(threads) as ex:
        return list(ex.map(part, jobs))


def make_cpu_layer(seed: int):
    import oracle
    rng = np.random.default_rng(seed)
    layer = []
    for (k, n) in SHAPES:
        w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        wd = oracle.dequantize_q4_to_f32(oracle.quantize_f32_to_q4(w)).reshape(n, k)   # load-time, untimed
        x = rng.standard_normal((1, k), dtype=np.float32)
        a = rng.standard_normal((LORA_RANK, k), dtype=np.float32) * np.float32(0.02)
        b = rng.standard_normal((n, LORA_RANK), dtype=np.float32) * np.float32(0.02)
        layer.append((x, wd, a, b, oracle.effective_scale(LORA_RANK, LORA_ALPHA)))
    return layer


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = os.cpu_count() or 1
    layer = make_cpu_layer(1)
    set_bytes = sum(algorithmic_bytes(1, n, k, LORA_RANK) for k, n in SHAPES)
    for _ in range(args.warmup):
        cpu_token_set(threads, layer)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_token_set(threads, layer)
    dt = time.perf_counter() - t0
    val = set_bytes * args.steps / dt / 1e9
    sample = (f"each step = one token-set (4 projections, M=1, LoRA r=16) of the workload's {args.layers} layers; "
              f"weights pre-dequantized to f32 at load as the reference's CPU path holds them; "
              f"matmul_bt kernel {oracle.matmul_bt_kernel(1, 5120, 5120)}; output rows split over {threads} threads")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, 1),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(args, world):
    return {"workload": "configs[2] large-layer decode set: (5120->5120, 5120->1024, 5120->17408, 17408->5120) "
                        f"x {args.layers} layers, M={args.m}, Q4 weights ~N(0,0.02^2), LoRA r={LORA_RANK} alpha={LORA_ALPHA:g}",
            "m": args.m, "layers": args.layers, "lora_rank": LORA_RANK,
            "launch": {"grouped": "one lq4_linear_group call per set: the four independent projections share one persistent launch",
                       "per-projection": "one lq4_linear call per projection",
                       "step": "one lq4_decode_step call per step: the sets are the groups of ONE persistent launch" +
                               (", chained (a set's 5120- and 17408-wide inputs are the previous set's gathered down/up outputs, "
                                "read through the mailbox as they arrive)" if args.chained else
                                ", all sixteen projections as one group (nothing links the sets)" if args.flat else
                                ", the sets in order, nothing links them (every set reads the step's external inputs)")}[args.launch],
            "parallelism": (f"N-sharded column-parallel x{world}, " +
                            (("outputs published to every rank's mailbox from the kernel's epilogue (8-byte tagged stores over NVLink), "
                              "gathered to plain f32 at the end of the same launch" +
                              ("" if args.chained else "; no set waits for another set's exchange")) if args.launch == "step" else
                             "all-gather fused into the decode kernel's epilogue (peer stores over NVLink + arrival counters)"
                             if args.gather == "peer" else "one NCCL all-gather per set")) if world > 1 else "single GPU",
            "l2": "inputs larger than L2: every launch streams distinct weights, "
                  f"{args.layers * 131.072:.0f} MB of Q4 payload per step per job"}


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    # The one JSON line is the only thing that may reach stdout: libraries loaded below (NCCL prints its version
    # there) get stderr as their file descriptor 1, and the line is written to the saved descriptor at the end.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    import torch
    import torch.distributed as dist
    from lattice_b200 import CudaQ4Backend, Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    from lattice_b200.sharded import shard_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    def note(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    note("process group ready")
    dev = torch.device("cuda", local_rank)
    be = CudaQ4Backend(local_rank)
    m = args.m
    scale = LORA_ALPHA / LORA_RANK

    # ---- build the synthetic model: every rank holds its row range of every projection
    layers = []
    gen = torch.Generator(device=dev)
    for li in range(args.layers):
        projs = []
        for si, (k, n) in enumerate(SHAPES):
            n0, n1, _ = shard_plan(n, k, world, rank)
            nl = n1 - n0
            gen.manual_seed(1000003 * li + 101 * si + 7 * rank + 1)
            w = torch.randn((nl, k), generator=gen, device=dev, dtype=torch.float32) * 0.02
            payload = be.quantize(w.reshape(-1))
            del w
            gen.manual_seed(5000011 * li + 211 * si + 3)          # A is replicated: same seed on every rank
            a = torch.randn((LORA_RANK, k), generator=gen, device=dev) * 0.02
            gen.manual_seed(7000003 * li + 307 * si + 13 * rank + 5)
            b = torch.randn((nl, LORA_RANK), generator=gen, device=dev) * 0.02
            projs.append(dict(k=k, n=n, nl=nl, n0=n0, qw=Q4WeightBuf.from_device_payload(payload, nl, k), a=a, b=b,
                              lora=LoraDesc(a.data_ptr(), b.data_ptr(), LORA_RANK, scale)))
        layers.append(projs)
    gen.manual_seed(99)
    xs = {k: torch.randn((m, k), generator=gen, device=dev) for k in (5120, 17408)}
    step_mode = args.launch == "step"
    if step_mode and m != 1:
        raise SystemExit("--launch step takes one token (--m 1)")
    # The outputs of one set sit side by side in one buffer, each projection writing its column range
    # (ldy = row pitch).  One GPU: [m, sum(n)].  Several GPUs: the same [m, sum(n)] buffer exists on
    # every rank as a peer buffer, a rank computes the columns of its N-shards and the decode kernels'
    # epilogue writes them into every rank's copy (--gather peer); or, the plain way, the local slices
    # are exchanged with ONE NCCL all-gather per set (--gather nccl).
    from lattice_b200.sharded import PeerGather
    peer_mode = world > 1 and args.gather in ("peer", "peer-nowait") and not step_mode
    peer_wait = args.gather == "peer"
    nls = [layers[0][si]["nl"] for si in range(len(SHAPES))]
    offs = [sum(nls[:si]) for si in range(len(SHAPES))]
    full_n = [n for _, n in SHAPES]
    full_offs = [sum(full_n[:si]) for si in range(len(SHAPES))]
    pg = PeerGather(m, sum(full_n), device=local_rank) if peer_mode else None
    gdesc = pg.desc if peer_mode else None
    if peer_mode:
        y_cat = pg.full
        y_local = {si: y_cat[:, full_offs[si] + layers[0][si]["n0"]:full_offs[si] + layers[0][si]["n0"] + nls[si]]
                   for si in range(len(SHAPES))}
        y_full = y_cat
    else:
        y_cat = torch.empty((m, sum(nls)), device=dev)
        y_local = {si: y_cat[:, offs[si]:offs[si] + nls[si]] for si in range(len(SHAPES))}
        y_full = torch.empty((world * m, sum(nls)), device=dev)
    torch.cuda.synchronize()
    note("synthetic model built")
    grouped = args.launch == "grouped"

    prepared = {}

    def run_set(projs, x_of, grouped=grouped):
        if grouped:
            # one persistent launch for the set's four projections; the argument block is built once
            # per (set, input buffers)
            key = (id(projs), id(x_of))
            if key not in prepared:
                prepared[key] = be.prepare_group([(x_of[p["k"]], p["qw"], p["lora"]) for p in projs],
                                                 [y_local[si] for si in range(len(projs))], gather=gdesc,
                                                 wait_gather=gdesc if peer_wait else None)
            prepared[key]()
        else:
            for si, p in enumerate(projs):
                be.dispatch_gemm_q4(x_of[p["k"]], 0, p["qw"], y_local[si], 0, m, p["nl"], p["k"], lora=p["lora"],
                                    ldy=y_cat.stride(0), gather=gdesc, wait_gather=gdesc if si == 0 and peer_wait else None)
        if world > 1 and args.gather == "nccl":
            dist.all_gather_into_tensor(y_full, y_cat)
        # peer mode: every set's kernel waits itself for the arrivals of the sets before it (as a layer
        # that consumes gathered activations does); the last set of a step is waited for in step()

    if peer_mode:
        # check the fused gather once against NCCL: every rank must hold every rank's columns
        run_set(layers[0], xs)
        be.gather_wait(gdesc)
        torch.cuda.synchronize()
        dist.barrier()
        for si, p in enumerate(layers[0]):
            mine = y_local[si].contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            if len({shard_plan(p["n"], p["k"], world, r)[1] - shard_plan(p["n"], p["k"], world, r)[0] for r in range(world)}) == 1:
                dist.all_gather(parts, mine)
                want = torch.cat(parts, dim=1)
                got = y_cat[:, full_offs[si]:full_offs[si] + p["n"]]
                if not torch.equal(want, got):
                    raise SystemExit(f"fused all-gather mismatch on rank {rank}, projection {si}")
        dist.barrier()
        note("fused all-gather checked against NCCL")

    def step():
        for projs in layers:
            run_set(projs, xs)
        if peer_mode and peer_wait:
            be.gather_wait(gdesc)                  # stream-ordered: the last set's peer columns have arrived

    step_check = None
    step_variants = {}
    if step_mode:
        # ONE launch per step: the sets are the ordered groups of a single lq4_decode_step call and every set's
        # full output row (all ranks' columns side by side) lives in the step buffer.
        #   independent: every set reads the step's external inputs (the workload as it is defined: four
        #                projections per set, nothing links the sets); with several GPUs no set waits for another,
        #                and when the launch completes every rank holds every rank's columns.
        #   chained:     set li > 0 takes its 5120-wide input from set li-1's 17408->5120 output and its 17408-wide
        #                input from set li-1's 5120->17408 output, so a set can only start when the previous set's
        #                columns of ALL ranks have arrived - the dependency a real decode step has.
        from lattice_b200.sharded import StepBuffer
        S = sum(full_n)

        def make_step_variant(chained, flat=False):
            sbuf = StepBuffer(args.layers * S, device=local_rank)
            pay = sbuf.payload

            def row_of(li, si):
                return pay[li * S + full_offs[si]: li * S + full_offs[si] + full_n[si]]

            def y_of(li, si):
                b0 = li * S + full_offs[si] + layers[li][si]["n0"]
                return pay[b0: b0 + nls[si]]

            def build(x_ext, host=False, y_host=None):
                # host: lq4_decode_step_host (x_ext may be pinned host memory); y_host: a pinned [layers * S] buffer
                # the outputs are stored to directly (one GPU, independent sets: nothing reads them on the device)
                groups = []
                for li, projs in enumerate(layers):
                    grp = []
                    for si, p in enumerate(projs):
                        if li == 0 or not chained:
                            x = x_ext[p["k"]]
                        else:
                            x = row_of(li - 1, 3) if p["k"] == 5120 else row_of(li - 1, 2)
                        y = y_of(li, si)
                        if y_host is not None:
                            y = y_host[li * S + full_offs[si]: li * S + full_offs[si] + full_n[si]]
                        grp.append((x, p["qw"], p["lora"], y))
                    groups.append(grp)
                if flat:                          # nothing links the sets: the caller may as well hand them over as ONE group
                    groups = [[pr for grp in groups for pr in grp]]
                if y_host is not None:
                    return be.prepare_step(groups, host=True)
                return be.prepare_step(groups, sbuf, gathered=[pay[li * S:(li + 1) * S] for li in range(args.layers)], host=host)

            run = build(xs)

            # checked once before timing against the same work issued set by set (one grouped launch per set, the
            # slices exchanged by NCCL between the sets)
            def reference():
                x_of = dict(xs)
                rows = []
                for li, projs in enumerate(layers):
                    outs = [torch.empty((1, p["nl"]), device=dev) for p in projs]
                    be.linear_group([(x_of[p["k"]], p["qw"], p["lora"]) for p in projs], outs)
                    full = []
                    for o in outs:
                        if world > 1:
                            parts = [torch.empty_like(o) for _ in range(world)]
                            dist.all_gather(parts, o)
                            full.append(torch.cat(parts, dim=1))
                        else:
                            full.append(o)
                    rows.append(torch.cat(full, dim=1))
                    if chained:
                        x_of = {5120: full[3].contiguous(), 17408: full[2].contiguous()}
                return torch.cat(rows, dim=1).reshape(-1)

            run()
            torch.cuda.synchronize()
            be.check_device_status()
            ref = reference()
            torch.cuda.synchronize()
            rms = float(ref.double().pow(2).mean().sqrt())
            ratio = float(((pay - ref).abs().double() / (1e-3 * (ref.abs().double() + rms))).max())
            if not (ratio <= 1.0) or not bool(torch.isfinite(pay).all()):
                raise SystemExit(f"step launch differs from the set-by-set form on rank {rank}: tolerance ratio {ratio}")
            if world > 1:
                lo, hi = pay.clone(), pay.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                if not torch.equal(lo, hi):
                    raise SystemExit("ranks hold different gathered rows after the step launch")
            check = {"against": "the same work issued as one grouped launch per set" + (" + NCCL all-gather between sets" if world > 1 else ""),
                     "max_tolerance_ratio": ratio, "all_ranks_identical": True}
            return dict(run=run, build=build, sbuf=sbuf, pay=pay, check=check)

        head_name = "chained" if args.chained else ("flat" if args.flat else "independent")
        step_variants[head_name] = make_step_variant(args.chained, args.flat and not args.chained)
        head = step_variants[head_name]
        step, pay, step_check = head["run"], head["pay"], head["check"]
        build_step = head["build"]
        note(f"step launch checked, tolerance ratio {step_check['max_tolerance_ratio']:.3g}")

    # pinned host buffers for the end-to-end variant
    hx = {k: torch.randn((m, k)).pin_memory() for k in (5120, 17408)}
    hy = torch.empty((args.layers,) + tuple(y_full.shape)).pin_memory()      # one result per set
    dx = {k: torch.empty((m, k), device=dev) for k in (5120, 17408)}

    # One GPU: the inputs of the step's sets sit in one pinned buffer and go in with ONE copy, every set
    # has its own device inputs and output, and the results come back with ONE copy: a copy-engine
    # operation costs several microseconds however small it is.
    batched = world == 1 and not step_mode
    if step_mode:
        # one pinned buffer in (the step's external inputs), one launch, one pinned buffer out (every set's rows)
        # The public call is lq4_decode_step_host: the pinned inputs are staged in by a kernel chained in front of
        # the step kernel, and (one GPU, independent sets) the step kernel stores the results straight into the
        # pinned output buffer, so no copy-engine operation is left in the step.  Chained sets and N-sharded steps
        # keep their outputs in the step buffer (later sets and the peers read them there) and copy them out.
        hx_cat = torch.randn(5120 + 17408).pin_memory()
        hy_step = torch.empty(args.layers * S).pin_memory()
        e2e_host_out = world == 1 and not args.chained
        hx_views = {5120: hx_cat[:5120], 17408: hx_cat[5120:]}
        e2e_step_call = build_step(hx_views, host=True, y_host=hy_step if e2e_host_out else None)
        # checked once: the host call gives the bits of the device-buffer call on the same inputs
        dx_chk = hx_cat.to(dev)
        chk_call = build_step({5120: dx_chk[:5120].view(1, -1), 17408: dx_chk[5120:].view(1, -1)})
        chk_call()
        torch.cuda.synchronize()
        want = pay.clone()
        hy_step.fill_(float("nan"))
        e2e_step_call()
        if not e2e_host_out:
            hy_step.copy_(pay, non_blocking=True)
        torch.cuda.synchronize()
        be.check_device_status()
        if not torch.equal(want.cpu(), hy_step):
            raise SystemExit("the host-buffer step differs from the device-buffer step")
        step()                                    # the step buffer holds the timed variant's results again
        torch.cuda.synchronize()
    if batched:
        xw = 5120 + 17408
        hx_all = torch.randn((args.layers, m, xw)).pin_memory()
        dx_all = torch.empty((args.layers, m, xw), device=dev)
        y_all = torch.empty((args.layers, m, sum(nls)), device=dev)
        hy_all = torch.empty((args.layers, m, sum(nls))).pin_memory()
        e2e_groups = {}

    def e2e_set(li, projs):
        """The public call for set li on the batched buffers (inputs are [m, k] slices with row pitch xw)."""
        x_of = {5120: dx_all[li, :, :5120], 17408: dx_all[li, :, 5120:]}
        outs = [y_all[li][:, offs[si]:offs[si] + nls[si]] for si in range(len(projs))]
        if m == 1 and grouped:
            if li not in e2e_groups:
                e2e_groups[li] = be.prepare_group([(x_of[p["k"]], p["qw"], p["lora"]) for p in projs], outs)
            e2e_groups[li]()
        else:
            for si, p in enumerate(projs):
                be.dispatch_gemm_q4(x_of[p["k"]].contiguous(), 0, p["qw"], outs[si], 0, m, p["nl"], p["k"], lora=p["lora"],
                                    ldy=y_all[li].stride(0))

    def e2e_body():
        # host activations in (pinned -> device), the public call per set, host results out
        if step_mode:
            e2e_step_call()                       # reads the pinned inputs; writes the pinned outputs itself ...
            if not e2e_host_out:
                hy_step.copy_(pay, non_blocking=True)      # ... or leaves them in the step buffer
            return
        if batched:
            dx_all.copy_(hx_all, non_blocking=True)
            for li, projs in enumerate(layers):
                e2e_set(li, projs)
            hy_all.copy_(y_all, non_blocking=True)
            return
        for li, projs in enumerate(layers):
            for k in dx:
                dx[k].copy_(hx[k], non_blocking=True)
            run_set(projs, dx)
            if peer_mode and peer_wait:
                be.gather_wait(gdesc)
            hy[li].copy_(y_full if world > 1 else y_cat, non_blocking=True)

    # The copies and kernels of one step are captured in a CUDA graph too when the step holds no NCCL
    # call; a step is then one graph launch and one wait for the results on the host.
    e2e_info = {"mode": "plain calls, one wait per step"}
    e2e_graph = None
    if not args.eager and not (world > 1 and args.gather == "nccl"):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                e2e_body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph, stream=side):
                e2e_body()
            e2e_info["mode"] = ("cuda-graph replay of the step's copies and kernels" +
                                (" (one copy in, one copy out per step)" if batched else "") +
                                (" (lq4_decode_step_host: stage-in kernel + step kernel" +
                                 (", results stored to pinned host memory by the step kernel)" if e2e_host_out else ", one copy out)")
                                 if step_mode else "") + ", one wait per step")
        except Exception as e:
            e2e_graph = None
            e2e_info["mode"] = "plain calls, one wait per step (graph capture failed: %r)" % (e,)
            torch.cuda.synchronize()

    def e2e_step():
        if e2e_graph is not None:
            e2e_graph.replay()
        else:
            e2e_body()
        torch.cuda.current_stream().synchronize()        # the host reads the step's results

    # The device-timed leg replays a CUDA graph of one step (the launch-bound inner loop is captured
    # once; replay removes the per-call host cost).  --eager times plain calls instead.
    graph_info = {"mode": "eager"}

    # steps per captured graph of the headline leg: the largest divisor of --steps that is at most --graph-steps
    head_graph_steps = max(d for d in range(1, max(1, args.graph_steps) + 1) if args.steps % d == 0)
    graph_info["steps_per_replay"] = 1

    def make_graphed(fn, graph_steps=1):
        if args.eager or (world > 1 and args.gather == "nccl"):
            # with NCCL collectives inside the step, capture is left out: a captured all-gather did
            # not complete on this pool, so such steps are timed as plain calls
            if world > 1:
                graph_info["mode"] = "eager (multi-GPU step with NCCL all-gather)"
            return fn, None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            l0 = be.launch_count
            with torch.cuda.graph(g, stream=side):
                for _ in range(graph_steps):
                    fn()
            per_step = (be.launch_count - l0) // graph_steps
            graph_info["mode"] = ("cuda-graph replay of one captured step" if graph_steps == 1 else
                                  f"cuda-graph replay of {graph_steps} consecutive captured steps (programmatic launch edges "
                                  "between them: a step's weight stream starts while the step before it drains; its "
                                  "activations are read after that step has completed)")
            graph_info["steps_per_replay"] = graph_steps
            return g.replay, per_step
        except Exception as e:                      # capture not possible: fall back to plain calls
            graph_info["mode"] = "eager (graph capture failed: %r)" % (e,)
            torch.cuda.synchronize()
            return fn, None

    def timed(fn, steps, warmup, launches_per_step=None):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = be.launch_count
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        n_launch = be.launch_count - l0
        if launches_per_step is not None:
            n_launch = launches_per_step * steps
        return ms, n_launch

    per_step_bytes = args.layers * sum(algorithmic_bytes(m, n, k, LORA_RANK) for k, n in SHAPES)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)                    # the first sample is there before the timed region starts
    step_fn, per_step_launches = make_graphed(step, head_graph_steps)
    note("launch mode: " + graph_info["mode"])
    t_host0 = time.time()
    spr = graph_info["steps_per_replay"]
    ms, launches = timed(step_fn, args.steps // spr, -(-args.warmup // spr), per_step_launches * spr if per_step_launches is not None else None)
    t_host1 = time.time()
    note("device-timed leg done")
    clocks = sampler.window(t_host0, t_host1) if rank == 0 else None
    be.check_device_status()
    e2e_ms, _ = timed(e2e_step, max(1, min(args.steps, 20)), 3)
    e2e_steps = max(1, min(args.steps, 20))
    be.check_device_status()
    # the same step as plain calls (no CUDA graph): the copies are enqueued and the library's entry point is CALLED every
    # step, so its host-side work (argument checks, tensor-map lookups, launch) sits inside the timed region
    def e2e_plain_step():
        e2e_body()
        torch.cuda.current_stream().synchronize()
    e2e_plain_ms, _ = timed(e2e_plain_step, e2e_steps, 3)
    be.check_device_status()
    note("end-to-end leg done")

    value = per_step_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e_value = per_step_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
    hbm_peak, tc_peak, tc_sust, which = measured_peaks()
    n_lin = 1 if step_mode else args.layers * (1 if grouped else len(SHAPES))
    # the step's launches are the decode kernel, one per set when grouped, else one per projection (at
    # M = 1 nothing else runs; at M > 1 a small preparation kernel is chained in front of each), so the
    # average launch duration is the event time over the decode launches, and algorithmic bytes per
    # launch divide the same way; per GPU each rank streams 1/world of the bytes
    avg_launch_us = ms * 1e3 / (args.steps * n_lin)
    achieved = (per_step_bytes / world) * args.steps / (ms * 1e-3) / 1e9
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 codes x int8-limb activations in exact s32, block scales and accumulation in f32", "data": "synthetic",
            "config": workload_config(args, world),
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / e2e_steps,
                    "mode": e2e_info["mode"],
                    "ms_per_step_plain_calls": e2e_plain_ms / e2e_steps,
                    "h2d_bytes_per_step": int((1 if step_mode else args.layers) * sum(m * k * 4 for k in (5120, 17408))),
                    "d2h_bytes_per_step": int(args.layers * sum(m * n * 4 for _, n in SHAPES))},
            "gpu_launches": int(launches), "launch_mode": graph_info["mode"],
            "roofline": {"bound": "hbm", "kernel": ("decode_step_kernel: one persistent launch per step (all sets)" if step_mode else
                                                 "decode_kernel<1, 8>: one persistent launch per set of four projections" if grouped
                                                 else "decode_kernel<1, 1>: one launch per projection") +
                                                ", LoRA projection inside the same launch" if m == 1 else
                                                "dense_kernel + dense_prep_kernel (activation limbs, LoRA projection) per " +
                                                ("set" if grouped else "projection"),
                         "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "peak_source": f"{which} (MEASURED_PEAKS.json hbm_gbs)" if which == "measured" else "fallback 6650 GB/s",
                         "avg_launch_us": avg_launch_us, "algorithmic_bytes_per_launch": per_step_bytes / world / n_lin,
                         "traffic": ncu_traffic(args.launch)[0] if m == 1 and world == 1 else None,
                         "traffic_note": ncu_traffic(args.launch)[1]},
            "clocks": clocks}
    if step_check is not None:
        line["checked_before_timing"] = step_check

    if world == 1 and not args.no_aux:
        # the same STREAM-style copy the measured peak was taken with, on THIS box (the peak in the roofline stays the
        # recorded one): boxes of the pool differ by several percent, and this says how much of a run's figure that is
        try:
            src = torch.empty(1 << 28, dtype=torch.float32, device=dev)
            dst = torch.empty_like(src)
            best = 0.0
            for _ in range(6):
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                dst.copy_(src)
                c1.record()
                torch.cuda.synchronize()
                best = max(best, 2 * src.numel() * 4 / (c0.elapsed_time(c1) * 1e-3) / 1e9)
            del src, dst
            line.setdefault("aux", {})["copy_bandwidth_this_box"] = {"GB/s": best, "vs_recorded_peak": best / hbm_peak,
                                                                       "how": "torch copy of 1 GiB f32, read + write bytes, best of 6"}
        except Exception as e:
            line.setdefault("aux", {})["copy_bandwidth_this_box"] = {"error": repr(e)}
        # the headline step replayed back to back for about two seconds: the rate a decode loop sustains once
        # clocks and power have settled, with the sampled SM clock and the rate binned by clock
        line.setdefault("aux", {})["sustained"] = sustained_run(step_fn, per_step_bytes * spr, sampler, hbm_peak, chunk=max(1, 100 // spr))
        line["aux"]["sustained"]["steps_per_replay"] = spr
    if rank == 0 and world == 1 and not args.no_aux:
        line["aux"].update(aux_measurements(be, dev, hbm_peak, tc_peak, tc_sust, sampler))
        # the same decode set at other token counts and with the other launch mode, timed the same way
        def time_sets(mm, grp):
            xs_m = {k: torch.randn((mm, k), device=dev) for k in (5120, 17408)}
            ycat_m = torch.empty((mm, sum(nls)), device=dev)
            outs = [ycat_m[:, offs[si]:offs[si] + nls[si]] for si in range(len(SHAPES))]

            def fn():
                for projs in layers:
                    if grp:
                        be.linear_group([(xs_m[p["k"]], p["qw"], p["lora"]) for p in projs], outs)
                    else:
                        for si, p in enumerate(projs):
                            be.dispatch_gemm_q4(xs_m[p["k"]], 0, p["qw"], outs[si], 0, mm, p["nl"], p["k"], lora=p["lora"],
                                                ldy=ycat_m.stride(0))
            gfn, gl = make_graphed(fn)
            gms, _ = timed(gfn, min(args.steps, 20), 3, gl)
            nsteps = min(args.steps, 20)
            byts = args.layers * sum(algorithmic_bytes(mm, n, k, LORA_RANK) for k, n in SHAPES)
            v = byts * nsteps / (gms * 1e-3) / 1e9
            return {"GB/s": v, "frac_hbm": v / hbm_peak, "us_per_set": gms * 1e3 / nsteps / args.layers}
        for mm in (1, 4, 16):
            for grp in (True, False):
                if not step_mode and mm == m and grp == grouped:
                    continue
                line["aux"][f"decode_set_M{mm}_" + ("grouped" if grp else "per_projection")] = time_sets(mm, grp)
    if step_mode and not args.no_aux:
        # the other form of the step, timed the same way on every rank (graph replay, max over ranks)
        what = {"chained": "every set's inputs are the previous set's gathered outputs: a set starts when the previous set's "
                           "columns of all ranks have arrived",
                "independent": "the sets in order as four groups, nothing links them",
                "flat": "nothing links the sets, so all sixteen projections are handed over as ONE group: an upper bound, "
                        "not the order a decode step has"}
        for other in ("independent", "chained", "flat"):
            if other in step_variants:
                continue
            var = make_step_variant(other == "chained", other == "flat")
            step_variants[other] = var
            gfn, gl = make_graphed(var["run"], head_graph_steps)      # queued like the headline's steps
            spr_v = graph_info["steps_per_replay"] if gl is not None else 1
            nsteps = max(spr_v, min(args.steps, 50) // spr_v * spr_v)
            gms, _ = timed(gfn, nsteps // spr_v, 3 if spr_v == 1 else 1, gl)
            be.check_device_status()
            v = per_step_bytes * nsteps / (gms * 1e-3) / 1e9
            if rank == 0:
                line.setdefault("aux", {})[f"decode_step_M1_{other}"] = {
                    "GB/s": v, "frac_hbm_per_gpu": v / world / hbm_peak, "us_per_step": gms * 1e3 / nsteps, "steps_per_graph_replay": spr_v,
                    "checked_before_timing": var["check"], "what": what[other]}
    if world > 1 and not args.no_aux:
        sharded = aux_sharded_prefill(be, dev, world, rank, tc_peak, tc_sust)      # every rank takes part
        if rank == 0:
            line.setdefault("aux", {})["config4_prefill_M2048_K5120_N17408_lora64_bf16_sharded"] = sharded
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(layers[0])
    if rank == 0:
        sampler.stop()
        emit(line)
    if step_mode:
        torch.cuda.synchronize()
        for var in step_variants.values():
            var["sbuf"].close()
    if world > 1:
        if pg is not None:
            prepared.clear()
            pg.close()
        dist.barrier()
        dist.destroy_process_group()


def cpu_baseline(gpu_layer):
    """Times the oracle on the host on ONE token-set built from the first layer's own Q4 payload."""
    import oracle
    import torch
    layer = []
    for p in gpu_layer:
        k, n = p["k"], p["nl"]
        payload = p["qw"]._keep.cpu().numpy()
        wd = oracle.dequantize_q4_to_f32(payload).reshape(n, k)           # load-time, untimed
        x = np.random.default_rng(3).standard_normal((1, k), dtype=np.float32)
        layer.append((x, wd, p["a"].cpu().numpy(), p["b"].cpu().numpy(), LORA_ALPHA / LORA_RANK))
    set_bytes = sum(algorithmic_bytes(1, n, k, LORA_RANK) for k, n in SHAPES)
    cpu_token_set(1, layer)
    reps, t0 = 0, time.perf_counter()
    while True:
        cpu_token_set(1, layer)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > 12.0 or reps >= 200:
            break
    # second formulation: the decode shader's fused arithmetic straight from the Q4 payload (dequantization
    # inside the timed region), one thread, followed by the same apply_lora
    fused = None
    try:
        payloads = [p["qw"]._keep.cpu().numpy() for p in gpu_layer]

        def fused_set():
            for (x, wd, a, b, sc), pl, (k, n) in zip(layer, payloads, [(p["k"], p["nl"]) for p in gpu_layer]):
                y = oracle.gemv_q4_decode_form(x[0], pl, n, k)
                oracle.apply_lora(a, b, LORA_RANK, k, n, sc, x[0], y)
        fused_set()
        r2, t2 = 0, time.perf_counter()
        while True:
            fused_set()
            r2 += 1
            d2 = time.perf_counter() - t2
            if d2 > 6.0 or r2 >= 100:
                break
        fused = {"value": set_bytes * r2 / d2 / 1e9, "unit": UNIT, "cores": 1, "ms_per_token_set": d2 / r2 * 1e3,
                 "what": "decode-shader arithmetic on the packed Q4 payload (dequantization timed), 1 thread"}
    except Exception as e:                          # the second formulation must not hide the first
        fused = {"error": repr(e)}
    return {"value": set_bytes * reps / dt / 1e9, "unit": UNIT, "cores": 1, "kind": "port", "fused_dequant_variant": fused,
            "sample": f"{reps} repeats of one token-set (4 projections of layer 0, M=1, LoRA r=16), single thread as "
                      f"the reference's matmul_bt is; kernel {oracle.matmul_bt_kernel(1, 5120, 5120)}; "
                      f"f32 weights pre-dequantized at load (untimed)", "ms_per_token_set": dt / reps * 1e3}


def sustained_run(step_fn, per_step_bytes, sampler, hbm_peak, seconds=2.0, chunk=100):
    """Replays the step back to back for `seconds`, timing every chunk of `chunk` replays with CUDA events (no
    host synchronisation inside), and relates each chunk's rate to the SM clock sampled closest to it."""
    import torch
    step_fn()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True)]
    t0 = time.time()
    evs[0].record()
    while time.time() - t0 < seconds and len(evs) < 4000:
        for _ in range(chunk):
            step_fn()
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        evs.append(e)
        if len(evs) % 8 == 0:
            evs[-1].synchronize()          # keeps the queue a few chunks deep so the host clock tracks the device
    torch.cuda.synchronize()
    t1 = time.time()
    ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(len(evs) - 1)]
    total_ms = sum(ms)
    rates = [per_step_bytes * chunk / (x * 1e-3) / 1e9 for x in ms]
    clk = sampler.window(t0, t1)
    # chunk i ran at about t0 + (time of the chunks before it): pair it with the nearest clock sample
    bins = {}
    acc = 0.0
    for x, r in zip(ms, rates):
        mid = t0 + (acc + x / 2) * 1e-3
        acc += x
        near = min(sampler.samples, key=lambda q: abs(q[0] - mid), default=None)
        if near is not None:
            bins.setdefault(int(round(near[1] / 15.0) * 15), []).append(r)
    return {"seconds": total_ms * 1e-3, "replays": chunk * len(ms), "GB/s": per_step_bytes * chunk * len(ms) / (total_ms * 1e-3) / 1e9,
            "frac_hbm": per_step_bytes * chunk * len(ms) / (total_ms * 1e-3) / 1e9 / hbm_peak,
            "GB/s_first_chunk": rates[0], "GB/s_last_chunk": rates[-1], "GB/s_min_chunk": min(rates),
            "clocks": clk, "GB/s_by_sm_mhz": {str(k): float(np.mean(v)) for k, v in sorted(bins.items())}}


def aux_sharded_prefill(be, dev, world, rank, tc_peak, tc_sust):
    """The prefill GEMM (M=2048, K=5120, N=17408, LoRA r=64, bf16 activations) with its output rows sharded over
    the ranks and the [M, N / world] slices gathered over NCCL through lq4_linear_sharded: plain calls, CUDA events
    from the first launch to the gathered y, MAX over ranks; beside it the local product alone."""
    import torch
    import torch.distributed as dist
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    from lattice_b200.sharded import NcclShardedLinear, shard_plan
    m, k, n, r = 2048, 5120, 17408, 64
    out = {}
    try:
        n0, n1, _ = shard_plan(n, k, world, rank)
        gen = torch.Generator(device=dev)
        gen.manual_seed(4400 + rank)
        w = torch.randn((n1 - n0, k), generator=gen, device=dev) * 0.02
        qw = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), n1 - n0, k)
        del w
        gen.manual_seed(4500)
        a = torch.randn((r, k), generator=gen, device=dev) * 0.02
        x = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
        gen.manual_seed(4600 + rank)
        b = torch.randn((n1 - n0, r), generator=gen, device=dev) * 0.02
        lora = LoraDesc(a.data_ptr(), b.data_ptr(), r, 2.0)
        lin = NcclShardedLinear(be, qw, n, lora=lora)
        y = torch.empty((m, n), device=dev)
        y_local = torch.empty((m, n1 - n0), device=dev)

        def timed_max(fn, reps):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3 / reps], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        us_total = timed_max(lambda: lin.forward(x, out=y), 10)
        be.check_device_status()
        # every rank's columns of the gathered output are what that rank computed
        be.dispatch_gemm_q4(x, 0, qw, y_local, 0, m, n1 - n0, k, lora=lora)
        torch.cuda.synchronize()
        same = torch.tensor([int(torch.equal(y[:, n0:n1], y_local))], device=dev)
        parts = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(parts, y_local)
        same &= int(torch.equal(torch.cat(parts, dim=1), y))
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        us_local = timed_max(lambda: be.dispatch_gemm_q4(x, 0, qw, y_local, 0, m, n1 - n0, k, lora=lora), 10)
        flops = 2 * m * n * k + 2 * m * r * (k + n)
        # the same product with the all-gather fused into the tensor-core kernel's epilogue: every rank's slice is
        # stored straight into every rank's [M, N] buffer over NVLink while the MMAs go on, a signal kernel and a
        # wait kernel close the exchange (no NCCL, no staging, no placement pass)
        from lattice_b200.sharded import PeerGather
        pg = PeerGather(m, n, device=dev.index)
        out_slice = pg.full[:, n0:n1]

        def fused_call():
            be.dispatch_gemm_q4(x, 0, qw, out_slice, 0, m, n1 - n0, k, lora=lora, ldy=n, gather=pg.desc)
            be.gather_wait(pg.desc)

        us_fused = timed_max(fused_call, 10)
        be.check_device_status()
        torch.cuda.synchronize()
        dist.barrier()
        same_fused = torch.tensor([int(torch.equal(pg.full, y))], device=dev)
        dist.all_reduce(same_fused, op=dist.ReduceOp.MIN)
        fused = {"us_per_call": us_fused, "TFLOP/s_aggregate": flops / us_fused / 1e6,
                 "frac_bf16_burst_per_gpu": flops / us_fused / 1e6 / world / tc_peak if tc_peak else None,
                 "us_exchange_not_hidden": us_fused - us_local,
                 "nvlink_bytes_out_per_rank": int(m * (n1 - n0) * 4 * (world - 1)),
                 "gathered_output_checked": bool(int(same_fused.item())),
                 "exchange": "peer stores from the tensor-core kernel's epilogue + signal / wait kernels"}
        pg.close()
        out = {"fused_peer_store": fused, "us_per_call": us_total, "TFLOP/s_aggregate": flops / us_total / 1e6,
               "frac_bf16_burst_per_gpu": flops / us_total / 1e6 / world / tc_peak if tc_peak else None,
               "us_local_product_alone": us_local, "us_exchange_and_placement_not_hidden": us_total - us_local,
               "gathered_bytes_per_rank": int(m * n * 4 * (world - 1) // world),
               "gathered_output_checked": bool(int(same.item())), "timing": "plain calls, CUDA events, max over ranks",
               "exchange": "ncclAllGather per tile-row block on a second stream + placement pass"}
        lin.close()
    except Exception as e:                                   # an aux failure must not hide the headline
        out = {"error": repr(e)}
    return out


def aux_measurements(be, dev, hbm_peak, tc_peak, tc_sust, sampler=None):
    """Secondary configurations, each timed with CUDA events over distinct weight copies; every entry carries
    the SM clock sampled while it was measured."""
    import torch
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    out = {}
    gen = torch.Generator(device=dev)

    def bench_linear(name, m, k, n, rank, copies, reps, rot=False, x_dtype=torch.float32):
        qws, keep = [], []
        for c in range(copies):
            gen.manual_seed(31 * c + k + n)
            w = torch.randn((n, k), generator=gen, device=dev) * 0.02
            payload = be.quantize(w.reshape(-1), symmetric=rot)
            keep.append(payload)
            qws.append(Q4WeightBuf.from_device_payload(payload, n, k))
            del w
        lora = None
        if rank:
            a = torch.randn((rank, k), generator=gen, device=dev) * 0.02
            b = torch.randn((n, rank), generator=gen, device=dev) * 0.02
            keep += [a, b]
            lora = LoraDesc(a.data_ptr(), b.data_ptr(), rank, 2.0)
        rd = None
        if rot:
            signs = be.rot_signs(0xCAFEBABEDEADBEEF, k)
            keep.append(signs)
            rd = be.rot_desc(signs)
        x = torch.randn((m, k), generator=gen, device=dev).to(x_dtype)
        y = torch.empty((m, n), device=dev)
        for i in range(3):
            be.dispatch_gemm_q4(x, 0, qws[i % copies], y, 0, m, n, k, lora=lora, rot=rd)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        mode = "plain calls"
        if m <= 16:
            # decode shapes are launch-bound: time a CUDA-graph replay of `reps` calls, like the headline
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(reps):
                        be.dispatch_gemm_q4(x, 0, qws[i % copies], y, 0, m, n, k, lora=lora, rot=rd)
                g.replay()
                torch.cuda.synchronize()
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                mode = "cuda-graph replay"
            except Exception:
                torch.cuda.synchronize()
                mode = "plain calls"
        if mode == "plain calls":
            e0.record()
            for i in range(reps):
                be.dispatch_gemm_q4(x, 0, qws[i % copies], y, 0, m, n, k, lora=lora, rot=rd)
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        xb = 2 if x_dtype == torch.bfloat16 else 4
        byts = n * (k // 32) * 20 + 4 * rank * (k + n) + m * k * xb + m * n * 4
        flops = 2 * m * n * k + 2 * m * rank * (k + n)
        out[name] = {"us_per_call": us, "GB/s": byts / us / 1e3, "frac_hbm": byts / us / 1e3 / hbm_peak,
                     "TFLOP/s": flops / us / 1e6, "weight_copies": copies, "timing": mode}
        if m >= 64 and tc_peak:
            out[name]["frac_bf16_burst"] = flops / us / 1e6 / tc_peak
            out[name]["frac_bf16_sustained"] = flops / us / 1e6 / tc_sust

    def bench_lm_head(name, vocab, k, top_k, reps):
        """One token's vocabulary projection + exact top-k (the reference's two-stage lm_head path); the
        794 MB of Q4 rows are larger than L2, so one weight copy is a cold read every call."""
        parts = []
        for c0 in range(0, vocab, 31040):
            gen.manual_seed(977 + c0)
            w = torch.randn((min(31040, vocab - c0), k), generator=gen, device=dev) * 0.02
            parts.append(be.quantize(w.reshape(-1)))
            del w
        payload = torch.cat(parts)
        del parts
        qw = Q4WeightBuf.from_device_payload(payload, vocab, k)
        x = torch.randn((1, k), generator=gen, device=dev)
        y = torch.empty((1, vocab), device=dev)
        res = {}
        mode = "cuda-graph replay"
        for what in ("projection", "projection+topk", "topk"):
            def call():
                if what == "projection":
                    be.dispatch_gemm_q4(x, 0, qw, y, 0, 1, vocab, k)
                elif what == "topk":
                    be.logits_topk(y[0], top_k)
                else:
                    be.lm_head_topk(x, qw, top_k)
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for _ in range(reps):
                        call()
                g.replay()
                torch.cuda.synchronize()
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
            except Exception:
                torch.cuda.synchronize()
                mode = "plain calls"
                e0.record()
                for _ in range(reps):
                    call()
                e1.record()
                torch.cuda.synchronize()
            res[what] = e0.elapsed_time(e1) * 1e3 / reps
        byts = vocab * (k // 32) * 20 + k * 4 + vocab * 4
        us = res["projection+topk"]
        out[name] = {"us_per_call": us, "us_projection_only": res["projection"], "us_topk_only": res["topk"],
                     "GB/s": byts / us / 1e3, "frac_hbm": byts / us / 1e3 / hbm_peak, "top_k": top_k, "timing": mode}

    def bench_mlp(name, hidden, inter, rank, copies, reps):
        """One token's dense FFN (gate||up -> silu*up -> down) through lq4_mlp_block, against the same
        three steps as separate calls (grouped gate/up launch, gating pass in torch, down call)."""
        sets = []
        for c in range(copies):
            gen.manual_seed(4242 + c)
            w = torch.randn((2 * inter, hidden), generator=gen, device=dev) * 0.02
            qgu = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), 2 * inter, hidden)
            del w
            w = torch.randn((hidden, inter), generator=gen, device=dev) * 0.02
            qd = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), hidden, inter)
            del w
            sets.append((qgu, qd))
        keep, descs = [], []
        for k_in, n_out in ((hidden, inter), (hidden, inter), (inter, hidden)):
            a = torch.randn((rank, k_in), generator=gen, device=dev) * 0.02
            b = torch.randn((n_out, rank), generator=gen, device=dev) * 0.02
            keep += [a, b]
            descs.append(LoraDesc(a.data_ptr(), b.data_ptr(), rank, 2.0))
        x = torch.randn((1, hidden), generator=gen, device=dev)
        y = torch.empty((1, hidden), device=dev)
        gu = torch.empty((1, 2 * inter), device=dev)
        hbuf = torch.empty((1, inter), device=dev)
        res = {}
        from lattice_b200 import _lib as lq4lib
        for what in ("block", "two_launches", "separate"):
            be.set_option(lq4lib.OPT_MLP_ONE_LAUNCH, 0 if what == "two_launches" else 1)

            def call(i):
                qgu, qd = sets[i % copies]
                if what == "block":              # default: the block as ONE lq4_decode_step launch (row in the library's step buffer)
                    be.mlp_block(x, qgu, qd, lora_gate=descs[0], lora_up=descs[1], lora_down=descs[2], out=y)
                elif what == "two_launches":     # grouped gate/up launch into the caller's row, then down_proj gating its own input
                    be.mlp_block(x, qgu, qd, lora_gate=descs[0], lora_up=descs[1], lora_down=descs[2], gate_up=gu, out=y)
                else:
                    be.dispatch_gemm_q4_at(x, 0, qgu, 0, gu, 0, 1, inter, hidden, lora=descs[0])
                    be.dispatch_gemm_q4_at(x, 0, qgu, inter * (hidden // 32) * 20, gu, inter * 4, 1, inter, hidden, lora=descs[1])
                    torch.mul(torch.nn.functional.silu(gu[:, :inter]), gu[:, inter:], out=hbuf)
                    be.dispatch_gemm_q4(hbuf, 0, qd, y, 0, 1, hidden, inter, lora=descs[2])
            for i in range(3):
                call(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(reps):
                    call(i)
            g.replay()
            torch.cuda.synchronize()
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            res[what] = e0.elapsed_time(e1) * 1e3 / reps
        byts = 3 * inter * (hidden // 32) * 20 + 4 * rank * 3 * (hidden + inter)
        us = res["block"]
        be.set_option(lq4lib.OPT_MLP_ONE_LAUNCH, 1)
        out[name] = {"us_per_block": us, "us_two_launches": res["two_launches"], "us_separate_calls": res["separate"], "GB/s": byts / us / 1e3,
                     "frac_hbm": byts / us / 1e3 / hbm_peak, "weight_copies": copies, "timing": "cuda-graph replay"}

    def clocked(fn, name, *a, **kw):
        t0 = time.time()
        fn(name, *a, **kw)
        if sampler is not None and name in out:
            out[name]["clocks"] = sampler.window(t0, time.time())

    try:
        clocked(bench_mlp, "mlp_block_M1_hidden5120_inter17408_lora16", 5120, 17408, 16, 2, 40)
        clocked(bench_linear, "config1_M1_K1024_N3584_cold", 1, 1024, 3584, 0, 128, 512)
        clocked(bench_linear, "config1_M1_K1024_N3584_warm", 1, 1024, 3584, 0, 1, 512)
        clocked(bench_linear, "config2_M1_lora16_cold", 1, 1024, 3584, 16, 128, 512)
        clocked(bench_linear, "config2_M8_lora16_cold", 8, 1024, 3584, 16, 128, 512)
        clocked(bench_linear, "config5_quarot_M1_K4096_N11008", 1, 4096, 11008, 0, 8, 200, rot=True)
        clocked(bench_linear, "config4_prefill_M2048_K5120_N17408_lora64_bf16", 2048, 5120, 17408, 64, 1, 50,
                x_dtype=torch.bfloat16)
        clocked(bench_linear, "config5_quarot_M512_K4096_N11008", 512, 4096, 11008, 0, 1, 20, rot=True)
        clocked(bench_lm_head, "lm_head_topk50_vocab248320_K5120", 248320, 5120, 50, 20)
    except Exception as e:                                   # an aux failure must not hide the headline
        out["error"] = repr(e)
    return out


def run_only(args):
    """Small single cases for profiler captures (no JSON line): a few launches of one kernel."""
    import torch
    from lattice_b200 import CudaQ4Backend, Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    be = CudaQ4Backend(0)
    dev = torch.device("cuda", 0)
    if args.only == "gemm-slice":          # M=2048, K=5120 on a 2176-row N-shard of the 17408 outputs, bf16, LoRA r=64
        m, k, n, r, dt = 2048, 5120, 2176, 64, torch.bfloat16
    elif args.only == "decode-up":         # M=--m (default 1), 5120 -> 17408, LoRA r=16
        m, k, n, r, dt = args.m, 5120, 17408, 16, torch.float32
    elif args.only == "decode-set":        # M=1, one grouped launch over the four large-layer shapes, LoRA r=16
        probs, keep = [], []
        for k, n in SHAPES:
            w = torch.randn((n, k), device=dev) * 0.02
            qw = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), n, k)
            del w
            a = torch.randn((LORA_RANK, k), device=dev) * 0.02
            b = torch.randn((n, LORA_RANK), device=dev) * 0.02
            keep += [a, b]
            probs.append((torch.randn((1, k), device=dev), qw, LoraDesc(a.data_ptr(), b.data_ptr(), LORA_RANK, 2.0)))
        for _ in range(3):
            be.linear_group(probs)
        torch.cuda.synchronize()
        be.check_device_status()
        print("ok", args.only)
        return
    elif args.only == "decode-step":       # M=1, --layers sets of the four large-layer shapes in ONE launch (--chained: each fed by the one before)
        from lattice_b200.sharded import StepBuffer
        S = sum(n for _, n in SHAPES)
        offs_full = [sum(n for _, n in SHAPES[:i]) for i in range(len(SHAPES))]
        sbuf = StepBuffer(args.layers * S)
        pay = sbuf.payload
        keep, groups = [], []
        x_ext = {k: torch.randn((1, k), device=dev) for k in (5120, 17408)}
        for li in range(args.layers):
            grp = []
            for si, (k, n) in enumerate(SHAPES):
                w = torch.randn((n, k), device=dev) * 0.02
                qw = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), n, k)
                del w
                a = torch.randn((LORA_RANK, k), device=dev) * 0.02
                b = torch.randn((n, LORA_RANK), device=dev) * 0.02
                keep += [a, b]
                if li == 0 or not args.chained:
                    x = x_ext[k]
                else:
                    src = 3 if k == 5120 else 2
                    x = pay[(li - 1) * S + offs_full[src]: (li - 1) * S + offs_full[src] + SHAPES[src][1]]
                grp.append((x, qw, LoraDesc(a.data_ptr(), b.data_ptr(), LORA_RANK, 2.0),
                            pay[li * S + offs_full[si]: li * S + offs_full[si] + n]))
            groups.append(grp)
        step = be.prepare_step(groups, sbuf, gathered=[])
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        be.check_device_status()
        print("ok", args.only, float(pay.abs().max()))
        return
    elif args.only == "mlp-block":         # M=1 dense FFN, hidden 5120, inter 17408, three r=16 adapters
        hidden, inter = 5120, 17408
        w = torch.randn((2 * inter, hidden), device=dev) * 0.02
        qgu = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), 2 * inter, hidden)
        del w
        w = torch.randn((hidden, inter), device=dev) * 0.02
        qd = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), hidden, inter)
        del w
        keep, descs = [], []
        for k_in, n_out in ((hidden, inter), (hidden, inter), (inter, hidden)):
            a = torch.randn((LORA_RANK, k_in), device=dev) * 0.02
            b = torch.randn((n_out, LORA_RANK), device=dev) * 0.02
            keep += [a, b]
            descs.append(LoraDesc(a.data_ptr(), b.data_ptr(), LORA_RANK, 2.0))
        x = torch.randn((1, hidden), device=dev)
        for _ in range(3):
            y = be.mlp_block(x, qgu, qd, lora_gate=descs[0], lora_up=descs[1], lora_down=descs[2])
        torch.cuda.synchronize()
        be.check_device_status()
        print("ok", args.only, float(y.abs().max()))
        return
    elif args.only == "lm-head":           # M=1, vocabulary projection 5120 -> 248320 + exact top-50
        vocab, k = 248320, 5120
        parts = []
        for c0 in range(0, vocab, 31040):
            w = torch.randn((31040, k), device=dev) * 0.02
            parts.append(be.quantize(w.reshape(-1)))
            del w
        payload = torch.cat(parts)
        del parts
        qw = Q4WeightBuf.from_device_payload(payload, vocab, k)
        x = torch.randn((1, k), device=dev)
        for _ in range(3):
            vals, ids = be.lm_head_topk(x, qw, 50)
        torch.cuda.synchronize()
        be.check_device_status()
        print("ok", args.only, ids[:4].tolist())
        return
    else:
        raise SystemExit("unknown --only case")
    w = torch.randn((n, k), device=dev) * 0.02
    qw = Q4WeightBuf.from_device_payload(be.quantize(w.reshape(-1)), n, k)
    del w
    a = torch.randn((r, k), device=dev) * 0.02
    b = torch.randn((n, r), device=dev) * 0.02
    x = torch.randn((m, k), device=dev).to(dt)
    y = torch.empty((m, n), device=dev)
    for _ in range(3):
        be.dispatch_gemm_q4(x, 0, qw, y, 0, m, n, k, lora=LoraDesc(a.data_ptr(), b.data_ptr(), r, 2.0))
    torch.cuda.synchronize()
    be.check_device_status()
    print("ok", args.only)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--launch", default="step", choices=["step", "grouped", "per-projection"],
                    help="step: one persistent launch per step, the sets are its groups (lq4_decode_step); "
                         "grouped: one persistent launch per set of four projections (lq4_linear_group); "
                         "per-projection: one lq4_linear call each")
    ap.add_argument("--flat", action="store_true",
                    help="with --launch step: all projections of the step as ONE group (nothing links the sets)")
    ap.add_argument("--chained", action="store_true",
                    help="with --launch step: every set's inputs are the previous set's gathered outputs (the dependent "
                         "form; reported in aux otherwise)")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl", "peer-nowait", "none"],
                    help="several GPUs: peer = all-gather fused into the kernel epilogue (stores into every "
                         "rank's buffer over NVLink); nccl = one NCCL all-gather per set; peer-nowait and none are "
                         "diagnostics (no waiting for the peers / no exchange at all): their values are not results")
    ap.add_argument("--eager", action="store_true", help="time plain calls instead of a CUDA-graph replay")
    ap.add_argument("--graph-steps", type=int, default=10,
                    help="consecutive steps captured in the replayed CUDA graph of the device-timed leg (1: one step per replay)")
    ap.add_argument("--verbose", action="store_true", help="progress notes on stderr")
    ap.add_argument("--only", default=None, help="gemm-slice | decode-up | decode-set | decode-step | mlp-block | lm-head: three launches of one case, for profiling")
    ap.add_argument("--no-aux", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
