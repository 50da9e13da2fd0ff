#!/usr/bin/env python
"""Benchmark of the mask-packing + fused sparse-mask attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2|3|4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one pass of the hot path over one batch: pack_mask(mask) followed by the attention forward
with the packed mask (the reference times exactly this pair, run.py:147-155, 433).  The default
workload is the headline configuration (B16 H12 N512 D64 fp16, keep probability 0.25, diagonal kept);
with N GPUs every rank runs that batch on its own GPU (B x H sharding, no collective; at N=8 the
whole job is the B=128 multi-GPU configuration).  Rank 0 prints one JSON line.

value      dense-equivalent TFLOP/s (4*B*H*N^2*D flops per step, the reference's convention,
           run.py:198-203) with inputs resident in HBM, summed over ranks.  K steps form one timed region
           (CUDA events, nothing else on the stream); `repeats` such regions run back to back and the
           median region counts, max over ranks: one region of 50 steps lasts 2 ms, too short to stand
           for a rank on a host shared by eight of them
e2e        the same metric through the public API sparse_attention_host() starting from pinned HOST
           tensors and ending with the result in pinned host memory, copies inside the timed region
roofline   the attention kernel: skip-adjusted flops per launch / mean launch time against the measured dense
           bf16 tensor peak; the launch times come from a separate pass over K steps with CUDA events
           around every launch (the timed regions themselves carry no events between their kernels)
other_configs   the block-sparse and the causal bf16 configuration and the keep-probability sweep, a few steps each
comparators     the reference project's own CUDA kernels (recompiled for sm_100a), torch's fused attention and flash-attn on
                the same inputs, launches back to back, outside every timed region
cpu_baseline / --impl reference: the reference's CPU path (PyTorch masked attention on the host cores)
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the ncu captures summarised under
# profiles/ — figures of those captures, not of this run; `traffic_source` in the JSON line names the file.
NCU_TRAFFIC = {
    ("attn", 2): (44_119_040 + 442_112, "profiles/attn_fwd_headline_B16_H12_N512.md"),
    ("pack", 2): (50_335_744 + 84_608, "profiles/pack_flat_headline_B16_H12_N512.md"),
}


def load_workloads():
    """sparse_mask_attention_b200/workloads.py as a plain module, without importing the package (whose __init__
    loads the CUDA library): the CPU reference arm must not map libsma_b200.so."""
    spec = importlib.util.spec_from_file_location(
        "sma_workloads", os.path.join(REPO, "sparse_mask_attention_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["sma_workloads"] = mod
    spec.loader.exec_module(mod)
    return mod


def load_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def config_dict(cfg, sets: int):
    """The `config` object of the JSON line; the same for both arms."""
    set_bytes = 3 * cfg.B * cfg.H * cfg.N * 64 * 2 + cfg.B * cfg.H * cfg.N * cfg.N
    return {"workload": cfg.name, "B_per_gpu": cfg.B, "H": cfg.H, "N": cfg.N, "D": 64, "mask": cfg.mask_kind,
            "keep_prob": cfg.keep_prob, "step": "pack_mask + attention forward",
            "l2": "rotates %d input sets (%d MB in HBM, L2 is 126 MB): every step reads cold inputs"
                  % (sets, sets * set_bytes // 2**20),
            "sharding": "B x H across ranks, no collective"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of the node's GPUs with ONE nvidia-smi while the timed regions run
    (one sampler per node, started by rank 0: eight of them at 10 Hz were a load of their own)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, indices):
        self.indices = set(indices)
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                if int(r[0]) not in self.indices:
                    continue
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "gpus": sorted(self.indices), "reasons": sorted(reasons)}


def cpu_reference_tflops(workloads, cfg, steps: int, warmup: int, sample_B: int, min_seconds: float = 0.0):
    """The reference's CPU path (PyTorch masked attention in fp32, all host threads) on a bounded sample of the
    workload: `steps` passes over `sample_B` batches, repeated until at least `min_seconds` have been spent.
    Returns (TFLOP/s dense-equivalent, seconds per pass, threads, passes)."""
    from oracle import sma_oracle  # the one place outside tests where the oracle runs: the CPU baseline

    # a multi-process launcher pins every rank to one OpenMP thread; this leg runs on one rank and takes the host
    host_threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if torch.get_num_threads() < host_threads:
        torch.set_num_threads(host_threads)
    q, k, v, mask = workloads.make_inputs(cfg, B=sample_B)
    q, k, v = q.float(), k.float(), v.float()  # the reference's CPU branch computes in fp32
    for _ in range(warmup):
        sma_oracle.attention_torch_cpu(q, k, v, mask)
    passes = 0
    t0 = time.perf_counter()
    while passes < steps or (time.perf_counter() - t0 < min_seconds and passes < 1000):
        sma_oracle.attention_torch_cpu(q, k, v, mask)
        passes += 1
    dt = (time.perf_counter() - t0) / passes
    flops = workloads.dense_flops(sample_B, cfg.H, cfg.N)
    return flops / dt / 1e12, dt, torch.get_num_threads(), passes


def run_reference_arm(args, cfg, rank: int):
    """--impl reference: the reference's CPU implementation of the path on this box's host cores, exactly
    `--steps` timed passes after `--warmup` untimed ones, each over a bounded sample of the workload."""
    if rank != 0:
        return
    workloads = load_workloads()
    # a pass over the full headline batch takes 70 ms on 16 cores; larger shapes are sampled down
    sample_B = cfg.B if cfg.N <= 512 else max(1, cfg.B // 4)
    tflops, dt, cores, passes = cpu_reference_tflops(workloads, cfg, args.steps, args.warmup, sample_B)
    sample = "B=%d of %d batches of %s per step, PyTorch CPU masked attention in fp32" % (sample_B, cfg.B, cfg.name)
    line = {
        "impl": "reference", "metric": "effective_tflops_dense_equiv", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": passes, "warmup": args.warmup, "ms_per_step": dt * 1e3 * cfg.B / sample_B,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(cfg, args.sets),
        "note": "ms_per_step is scaled from the sample to the full batch",
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def bind_to_gpu_numa_node(dev_index: int):
    """Pins this process to the CPU cores next to its GPU, so that the pinned host buffers allocated afterwards
    (first touch) and the copy threads sit on the GPU's side of the host.  The cores come from sysfs (the NUMA node of
    the GPU's PCI device) or, where a container hides that, from the driver (NVML's ideal CPU affinity of the device).
    Best effort: returns what it bound to ("node 1", "nvml 48 cpus"), or None when neither source answers (the
    affinity is then left alone)."""
    have = set(os.sched_getaffinity(0))
    try:
        props = torch.cuda.get_device_properties(dev_index)
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/numa_node" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        node = int(open(path).read().strip())
        if node >= 0:
            cpus = set()
            for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            if cpus & have:
                os.sched_setaffinity(0, cpus & have)
                return "node %d" % node
    except Exception:
        pass
    try:
        import pynvml

        pynvml.nvmlInit()
        try:
            props = torch.cuda.get_device_properties(dev_index)
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(
                "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id))
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
            cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        finally:
            pynvml.nvmlShutdown()
        # an affinity that names every core says nothing about the topology
        if cpus & have and len(cpus) < os.cpu_count():
            os.sched_setaffinity(0, cpus & have)
            return "nvml %d cpus" % len(cpus & have)
    except Exception:
        pass
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=25, help="timed regions of --steps steps; the median one counts")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4])
    ap.add_argument("--keep-prob", type=float, default=None,
                    help="keep probability of the mask (the sparsity sweep of the multi-GPU configuration); default: the configuration's own")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip other_configs and comparators")
    ap.add_argument("--sets", type=int, default=4, help="input sets rotated through so that every step reads cold data")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    workloads = load_workloads()
    cfg = workloads.CONFIGS[args.config]
    if args.keep_prob is not None:
        import dataclasses
        cfg = dataclasses.replace(cfg, name="%s_keep%g" % (cfg.name, args.keep_prob), keep_prob=args.keep_prob)
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)

    from sparse_mask_attention_b200 import _capi, sparse_attn_cuda
    from sparse_mask_attention_b200.sparse_attention import sparse_attention_func, sparse_attention_host

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    host_affinity = set(os.sched_getaffinity(0))  # the CPU baseline leg gets the whole host back
    numa_node = bind_to_gpu_numa_node(local_rank)

    peaks, peaks_kind = load_peaks()
    B, H, N, D = cfg.B, cfg.H, cfg.N, 64
    K, R = args.steps, args.repeats

    # ---- inputs: `sets` independent batches per rank (seed differs per rank and set) ------------------
    def device_sets(c, n_sets, seed0):
        out_sets, host0, skip = [], None, None
        for s in range(n_sets):
            cc = workloads.Config(c.name, c.B, c.H, c.N, c.dtype, c.mask_kind, c.keep_prob, seed=seed0 + s)
            q, k, v, mask = workloads.make_inputs(cc)
            if s == 0:
                host0 = (q, k, v, mask)
                skip = workloads.skip_adjusted_flops(mask)
            out_sets.append(tuple(t.to(dev) for t in (q, k, v, mask)))
        return out_sets, host0, skip

    sets, host0, skip_flops = device_sets(cfg, args.sets, 1000 * rank)
    host_sets = [t.pin_memory() for t in host0]
    out = torch.empty_like(sets[0][0])
    scale = 1.0 / D ** 0.5
    dense = workloads.dense_flops(B, H, N)
    stream = torch.cuda.current_stream(dev)

    def make_step(step_sets, step_out):
        n = len(step_sets)

        def step(i, ev=None):
            q, k, v, mask = step_sets[i % n]
            if ev is None:
                # the public call: pack_mask + attention forward (what the reference times, run.py:147-155)
                sparse_attention_func(q, k, v, mask)
                return
            # the same two kernels with an event between them (the instrumented pass)
            packed = sparse_attn_cuda.pack_mask(mask)
            ev[0].record(stream)
            sparse_attn_cuda.forward(q, k, v, packed, step_out, None, scale, False)
            ev[1].record(stream)
        return step

    step = make_step(sets, out)

    def barrier():
        torch.cuda.synchronize(dev)
        if dist:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # the clock sampler (one per node) starts first: the warm-up steps then run directly before the timed regions,
    # so that the GPU does not sit idle (and clock down) between the two
    sampler = None
    if rank == 0:
        sampler = ClockSampler(range(world))
        sampler.start()
    time.sleep(0.25)
    # spin-up (not counted as warm-up steps): keep the GPU busy for some tens of milliseconds so that its clocks
    # are up before the W warm-up steps and the timed regions, however few steps were asked for
    t_spin = time.perf_counter()
    while time.perf_counter() - t_spin < 0.03:
        for i in range(20):
            step(i)
    for i in range(args.warmup):
        step(i)

    # ---- timed: R regions of exactly K steps each, back to back, one event between regions ---------------
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
    barrier()
    host_t0 = time.perf_counter()
    marks[0].record(stream)
    n = 0
    for rep in range(R):
        for i in range(K):
            step(n)
            n += 1
        marks[rep + 1].record(stream)
    host_issue_s = time.perf_counter() - host_t0
    barrier()
    region_ms = [marks[i].elapsed_time(marks[i + 1]) for i in range(R)]
    median_region_ms = statistics.median(region_ms)

    # ---- K steps once more with events around every launch: per-kernel durations for the rooflines.
    # (An event record between two kernels keeps the second from starting its set-up under the tail of the first,
    # so this pass is slower than the timed regions; its step time is reported as instrumented_ms_per_step.)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
            torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    i_start = torch.cuda.Event(enable_timing=True)
    i_end = torch.cuda.Event(enable_timing=True)
    barrier()
    i_start.record(stream)
    for i in range(K):
        evs[i][2].record(stream)
        step(i, evs[i])
    i_end.record(stream)
    barrier()
    instrumented_ms = i_start.elapsed_time(i_end)
    attn_ms = [e[0].elapsed_time(e[1]) for e in evs]
    pack_ms = [e[2].elapsed_time(e[0]) for e in evs]
    _capi.device_status()

    # ---- each kernel alone, launches back to back between one pair of events (rotating input sets): what a
    # launch costs when its set-up overlaps the tail of the launch before it and no event record separates them
    def alone_ms(launch, launches):
        a0 = torch.cuda.Event(enable_timing=True)
        a1 = torch.cuda.Event(enable_timing=True)
        for i in range(max(args.warmup, 3)):
            launch(i)
        a0.record(stream)
        for i in range(launches):
            launch(i)
        a1.record(stream)
        barrier()
        return a0.elapsed_time(a1) / launches

    raw_stream = stream.cuda_stream

    def kernels_alone(k_sets, k_out, launches):
        packed_sets = [sparse_attn_cuda.pack_mask(s[3]) for s in k_sets]
        m = len(k_sets)
        kB, kH, kN = k_sets[0][0].shape[:3]
        # (the pack launch goes through the C ABI with a preallocated output: the Python wrapper's allocation and
        # checks take longer on the host than this kernel runs)
        p_ms = alone_ms(lambda i: _capi.pack_mask(k_sets[i % m][3].data_ptr(), packed_sets[i % m].data_ptr(), kB, kH, kN,
                                                  raw_stream), launches)
        a_ms = alone_ms(lambda i: sparse_attn_cuda.forward(k_sets[i % m][0], k_sets[i % m][1], k_sets[i % m][2],
                                                           packed_sets[i % m], k_out, None, scale, False), launches)
        return p_ms, a_ms

    pack_alone_ms, attn_alone_ms = kernels_alone(sets, out, K)

    # ---- end to end through the public API from pinned host memory ---------------------------------
    hq, hk, hv, hm = host_sets
    h_out = torch.empty_like(hq).pin_memory()
    e2e_steps = max(3, min(K, 20))

    def e2e_step():
        # host tensors in, host tensor out: copies to the device, pack + attention, copy back, pipelined over
        # slices of the batch inside the call
        sparse_attention_host(hq, hk, hv, hm, out=h_out, device=dev, sync=False)

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    clocks = sampler.stop() if sampler else None
    h2d = sum(t.numel() * t.element_size() for t in host_sets)
    d2h = h_out.numel() * h_out.element_size()

    # ---- other configurations and comparators: rank 0 of a single-GPU run only, outside every timed region ----
    other_configs, comparators = None, None
    if world == 1 and not args.no_extras:
        other_configs = {}

        def measure_config(name, c, n_sets, launches):
            c_sets, _, c_skip = device_sets(c, n_sets, 7000)
            c_out = torch.empty_like(c_sets[0][0])
            c_step = make_step(c_sets, c_out)
            step_ms = alone_ms(c_step, launches)
            p_ms, a_ms = kernels_alone(c_sets, c_out, launches)
            _capi.device_status()
            a_tf = c_skip / (a_ms * 1e-3) / 1e12
            other_configs[name] = {
                "workload": c.name, "B": c.B, "H": c.H, "N": c.N, "dtype": "f16" if c.dtype == torch.float16 else "bf16",
                "mask": c.mask_kind, "keep_prob": c.keep_prob, "launches": launches, "ms_per_step": step_ms,
                "value": workloads.dense_flops(c.B, c.H, c.N) / (step_ms * 1e-3) / 1e12,
                "attention_ms": a_ms, "pack_ms": p_ms, "skip_adjusted_flops": c_skip,
                "attention_achieved_tflops": a_tf, "attention_frac": a_tf / peaks["bf16_tflops"],
                "attention_hbm_frac": workloads.attention_bytes(c.B, c.H, c.N) / (a_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "pack_hbm_frac": workloads.pack_bytes(c.B, c.H, c.N) / (p_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "timed": "launches back to back (no event between kernels), %d rotating input sets" % n_sets}
            del c_sets, c_out
            torch.cuda.empty_cache()

        import dataclasses
        for cid in (3, 4):
            if cid != args.config:
                measure_config("config%d" % cid, workloads.CONFIGS[cid], 2, 20)
        base5 = workloads.CONFIGS[2]  # the multi-GPU configuration's per-GPU shard is the headline shape
        for p in (0.05, 0.5, 1.0):
            measure_config("keep_prob_%g" % p, dataclasses.replace(base5, name="cfg5_shard_keep%g" % p, keep_prob=p), 2, 20)

        # ---- the same step as a CUDA graph: what the host pays per step when the caller captures the call ----
        def measure_graph():
            gq, gk, gv, gm = sets[0]
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                for _ in range(3):
                    sparse_attention_func(gq, gk, gv, gm)
            stream.wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                sparse_attention_func(gq, gk, gv, gm)
            ms = alone_ms(lambda i: graph.replay(), 50)
            t0 = time.perf_counter()
            for _ in range(200):
                graph.replay()
            host_us = (time.perf_counter() - t0) / 200 * 1e6
            torch.cuda.synchronize(dev)
            _capi.device_status()
            return {"ms_per_step": ms, "host_issue_us_per_step": host_us,
                    "what": "sparse_attention_func captured once into a torch.cuda.CUDAGraph and replayed on one input set "
                            "(inputs stay in L2 between replays, unlike the timed regions above)"}

        try:
            other_configs["cuda_graph_replay"] = measure_graph()
        except Exception as e:
            other_configs["cuda_graph_replay"] = {"error": repr(e)[:200]}

        # ---- the backward pass at the bench workload (not part of the headline metric, which is forward only) ----
        def measure_backward():
            q0, k0, v0, m0 = sets[0]
            packed0 = sparse_attn_cuda.pack_mask(m0)
            out0 = torch.empty_like(q0)
            lse0 = torch.empty((B, H, N), dtype=torch.float32, device=dev)
            scale = 64 ** -0.5
            sparse_attn_cuda.forward(q0, k0, v0, packed0, out0, lse0, scale, True)
            dout = torch.randn_like(q0)
            dq, dk, dv = (torch.empty_like(q0) for _ in range(3))
            ms = alone_ms(lambda i: sparse_attn_cuda.backward(dout, q0, k0, v0, out0, lse0, packed0, dq, dk, dv, scale), 20)
            _capi.device_status()
            flops = 2.5 * skip_flops  # five products per visited tile against the forward pass's two
            res = {"ms_per_call": ms, "kernels": "bwd_prepare_kernel + attn_bwd_kernel + bwd_finish_kernel",
                   "skip_adjusted_flops": flops, "achieved_tflops": flops / (ms * 1e-3) / 1e12,
                   "frac": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], "timed": "20 calls back to back"}
            try:  # the PyTorch formulation that the reference's autograd function falls back to (dense [B,H,N,N] fp32)
                def dense(i):
                    s_ = (q0.float() @ k0.float().transpose(-1, -2)) * scale
                    a_ = torch.nan_to_num(torch.softmax(s_.masked_fill(~m0, float("-inf")), dim=-1), nan=0.0)
                    dv_ = a_.transpose(-1, -2) @ dout.float()
                    da_ = (dout.float() @ v0.float().transpose(-1, -2)).masked_fill(~m0, 0.0)
                    ds_ = a_ * (da_ - (da_ * a_).sum(dim=-1, keepdim=True)) * scale
                    return ds_ @ k0.float(), ds_.transpose(-1, -2) @ q0.float(), dv_
                res["torch_dense_recompute_ms"] = alone_ms(dense, 5)
            except Exception as e:
                res["torch_dense_recompute_ms"] = repr(e)[:120]
            return res

        try:
            other_configs["backward"] = measure_backward()
        except Exception as e:
            other_configs["backward"] = {"error": repr(e)[:200]}
        torch.cuda.empty_cache()

        comparators = {}
        q0, k0, v0, m0 = sets[0]
        try:
            from oracle import ref_cuda  # the reference's own kernels, recompiled for sm_100a (test infrastructure)

            if not ref_cuda.available():
                comparators["reference_cuda_sm100"] = {"unavailable": "oracle/_ref/libsma_ref.so not built"}
            elif not (cfg.dtype == torch.float16 and ref_cuda.mask_ok(m0)):
                comparators["reference_cuda_sm100"] = {
                    "unavailable": "not run: the reference kernels stop on masks with empty 16x16 blocks; fp16 i.i.d. masks only"}
            else:
                rp = ref_cuda.pack_mask(m0)
                r_pack = alone_ms(lambda i: ref_cuda.pack_mask(sets[i % args.sets][3]), 20)
                r_attn = alone_ms(lambda i: ref_cuda.attention(q0, k0, v0, m0, rp, mask_checked=True), 20)
                comparators["reference_cuda_sm100"] = {
                    "pack_us": r_pack * 1e3, "attention_us": r_attn * 1e3, "ours_pack_us": pack_alone_ms * 1e3,
                    "ours_attention_us": attn_alone_ms * 1e3,
                    "what": "pack_mask_kernel and sparse_attn_wmma_full_fp16 of the reference (csrc/sparse_attention.cu:549-568, "
                            "82-412) compiled for sm_100a, same inputs, 20 launches back to back"}
        except Exception as e:  # a comparator must never take the bench line down
            comparators["reference_cuda_sm100"] = {"error": repr(e)[:200]}
        try:
            import torch.nn.functional as F

            f_ms = alone_ms(lambda i: F.scaled_dot_product_attention(q0, k0, v0, attn_mask=m0), 10)
            comparators["torch_sdpa_bool_mask"] = {"attention_us": f_ms * 1e3,
                                                   "what": "torch.nn.functional.scaled_dot_product_attention with the bool mask, backend of torch's choice"}
        except Exception as e:
            comparators["torch_sdpa_bool_mask"] = {"error": repr(e)[:200]}
        try:
            import torch.nn.functional as F
            from torch.nn.attention import SDPBackend, sdpa_kernel

            def cudnn(i):
                with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                    return F.scaled_dot_product_attention(q0, k0, v0, attn_mask=m0)

            f_ms = alone_ms(cudnn, 10)
            comparators["torch_sdpa_cudnn"] = {"attention_us": f_ms * 1e3,
                                               "what": "the reference's cuDNN adapter (run.py:508-525): SDPA pinned to SDPBackend.CUDNN_ATTENTION"}
        except Exception as e:
            comparators["torch_sdpa_cudnn"] = {"error": repr(e)[:200]}

        try:
            from flash_attn import flash_attn_func

            # the reference's adapter (run.py:587-606): dense attention WITHOUT the mask, as a no-mask baseline; it
            # times the layout change to [B, N, H, D] with the kernel, so this does too
            def fa(i):
                qf, kf, vf = (t.permute(0, 2, 1, 3).contiguous() for t in (q0, k0, v0))
                return flash_attn_func(qf, kf, vf, dropout_p=0.0, softmax_scale=None, causal=False).permute(0, 2, 1, 3)

            f_ms = alone_ms(fa, 10)
            qf, kf, vf = (t.permute(0, 2, 1, 3).contiguous() for t in (q0, k0, v0))
            k_ms = alone_ms(lambda i: flash_attn_func(qf, kf, vf, dropout_p=0.0, softmax_scale=None, causal=False), 10)
            comparators["flash_attn_dense_no_mask"] = {
                "attention_us": f_ms * 1e3, "kernel_only_us": k_ms * 1e3,
                "what": "the reference's flash-attn adapter (run.py:587-606): flash_attn_func on all keys, mask ignored, "
                        "layout change included; kernel_only_us without the layout change"}
        except Exception as e:
            comparators["flash_attn_dense_no_mask"] = {"error": repr(e)[:200]}

    # ---- max over ranks, and the per-rank figures ------------------------------------------------------
    mine = torch.tensor([median_region_ms, e2e_ms, statistics.mean(attn_ms), statistics.mean(pack_ms), attn_alone_ms,
                         pack_alone_ms, host_issue_s / (K * R) * 1e6, min(region_ms), max(region_ms)],
                        device=dev, dtype=torch.float64)
    allr = [mine]
    if dist:
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
    table = torch.stack(allr).cpu()
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    worst = table.max(dim=0).values.tolist()
    median_region_ms, e2e_ms, attn_mean_ms, pack_mean_ms, attn_alone_ms, pack_alone_ms = worst[:6]

    ms_per_step = median_region_ms / K
    value = world * dense / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * dense / (e2e_ms * 1e-3) / 1e12
    attn_tflops = skip_flops / (attn_mean_ms * 1e-3) / 1e12
    pack_gbs = workloads.pack_bytes(B, H, N) / (pack_mean_ms * 1e-3) / 1e9
    attn_traffic = NCU_TRAFFIC.get(("attn", args.config), (None, None))
    pack_traffic = NCU_TRAFFIC.get(("pack", args.config), (None, None))
    line = {
        "metric": "effective_tflops_dense_equiv", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": K, "warmup": args.warmup, "repeats": R, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "f16" if cfg.dtype == torch.float16 else "bf16", "data": "synthetic",
        "config": config_dict(cfg, args.sets),
        "timing": {"what": "R regions of K steps back to back, median region, max over ranks",
                   "region_ms_median_per_rank": table[:, 0].tolist(), "region_ms_min_per_rank": table[:, 7].tolist(),
                   "region_ms_max_per_rank": table[:, 8].tolist(),
                   "step_us_per_rank": (table[:, 0] / K * 1e3).tolist(),
                   "host_issue_us_per_step_per_rank": table[:, 6].tolist()},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step_per_rank": table[:, 1].tolist(),
                "h2d_gbs_aggregate": world * h2d / (e2e_ms * 1e-3) / 1e9, "numa_node_rank0": numa_node,
                "api": "sparse_attention_host(q, k, v, mask, out) on pinned host tensors"},
        "gpu_launches": 2 * K * R,
        "clocks": clocks,
        "roofline": {"kernel": "attn_fwd_kernel", "bound": "tensor", "achieved": attn_tflops,
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": attn_tflops / peaks["bf16_tflops"],
                     "traffic": attn_traffic[0], "traffic_source": attn_traffic[1], "peak_kind": peaks_kind + " burst",
                     "flops_per_launch": skip_flops, "ms_per_launch": attn_mean_ms,
                     "timed": "separate pass over K steps with CUDA events around every launch",
                     "hbm_frac": workloads.attention_bytes(B, H, N) / (attn_mean_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "back_to_back": {"ms_per_launch": attn_alone_ms,
                                      "achieved": skip_flops / (attn_alone_ms * 1e-3) / 1e12,
                                      "frac": skip_flops / (attn_alone_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}},
        "roofline_pack": {"kernel": "pack_flat_kernel", "bound": "hbm", "achieved": pack_gbs, "peak": peaks["hbm_gbs"],
                          "unit": "GB/s", "frac": pack_gbs / peaks["hbm_gbs"],
                          "traffic": pack_traffic[0], "traffic_source": pack_traffic[1], "peak_kind": peaks_kind,
                          "bytes_per_launch": workloads.pack_bytes(B, H, N), "ms_per_launch": pack_mean_ms,
                          "note": "launch time includes the gap between the two launches of a step",
                          "back_to_back": {"ms_per_launch": pack_alone_ms,
                                           "achieved": workloads.pack_bytes(B, H, N) / (pack_alone_ms * 1e-3) / 1e9,
                                           "frac": workloads.pack_bytes(B, H, N) / (pack_alone_ms * 1e-3) / 1e9
                                           / peaks["hbm_gbs"]}},
        "instrumented_ms_per_step": instrumented_ms / K,
        "attention_only_ms": attn_mean_ms, "pack_only_ms": pack_mean_ms,
        "latency_ms": ms_per_step,
    }
    if other_configs is not None:
        line["other_configs"] = other_configs
    if comparators is not None:
        line["comparators"] = comparators
    if not args.no_cpu_baseline and world == 1:
        # every thread of the process (torch's worker pool was started while the process was bound to the GPU's cores)
        for tid in os.listdir("/proc/self/task"):
            try:
                os.sched_setaffinity(int(tid), host_affinity)
            except OSError:
                pass
        sample_B = B if N <= 512 else max(1, B // 4)
        tf, dt, cores, passes = cpu_reference_tflops(workloads, cfg, 3, 1, sample_B, min_seconds=10.0)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                "sample": "B=%d of %d, %d timed passes (>= 10 s) of the PyTorch CPU masked attention in fp32"
                                          % (sample_B, B, passes), "ms_per_pass": dt * 1e3}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
