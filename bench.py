#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

One step = forward + backward of one batch through the public ops.  The default workload is the
headline configuration: causal attention, bf16, GQA, B=4, S=8192, Hq=32, Hkv=8, D=128, every
sequence packed with segments of length ~U[512, 4096] given as int64 segment ids, level 0.
Inputs are seeded synthetic N(0,1) tensors.  Rank 0 prints ONE JSON line.

* ``value``     throughput with inputs resident in HBM (CUDA events, max over ranks), in TFLOP/s of
                algorithmic work: 14 * D * (visible query-key pairs over query heads).
* ``e2e``       the same through the public ops with HOST buffers: every step copies q, k, v, dy
                from pinned memory and copies y, dq, dk, dv back, inside the timed region.  Batch
                rows are independent, so the step is pipelined over them (copies of the next and
                of the previous row run beside the kernels of the current one; within a row dy comes
                in last and y leaves first; device input buffers are double-buffered, so the next
                step's inputs come in while this step's results leave; the clock stops after the
                last step's results are on the host).
* ``roofline``  the dominant kernel's algorithmic FLOP/s from per-launch CUDA events, against the
                measured dense bf16 peak of MEASURED_PEAKS.json.
* ``cpu_baseline`` the CPU oracle timed on the host cores (rank 0, N=1 only), on the reference's own
                CPU-sized configuration.

With N > 1 (torchrun, one rank per GPU) every rank runs its own batch: batch x heads shard with no
communication, so scaling is weak.  ``--impl reference`` times the CPU oracle on a bounded slice of
the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "attn fwd+bwd TFLOPS (bf16 causal S=8K D=128), whole job"
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch on ONE batch row of the
# workload (S=8192, Hq=32, Hkv=8, D=128), from ncu captures of one launch each: the dense causal
# row and a row packed with segments ~U[512,4096] (the headline packing).  Traffic grows in
# proportion to the batch rows (they share no data), so a launch over B rows moves B times this.
NCU_DRAM_BYTES_PER_BATCH_ROW = {
    "dense": {"fwd": 137.9e6, "bwd_dq": 215.1e6, "bwd_dkv": 353.3e6},
    "packed": {"fwd": 137.5e6, "bwd_dq": 211.6e6, "bwd_dkv": 300.6e6},
}

NCU_DRAM_BYTES_DECODE = 1080.4e6


def tensor_roofline(achieved, peaks, peak_src, timed_seconds):
    """Fractions of the measured dense bf16 peaks.  The burst figure is the denominator for a timed
    region shorter than a second (the clocks have not settled under the power cap yet), the
    sustained one for longer regions; both are printed."""
    burst = float(peaks.get("bf16_tflops", peaks.get("bf16_tflops_sustained")))
    sustained = float(peaks.get("bf16_tflops_sustained", burst))
    use_burst = timed_seconds < 1.0
    peak = burst if use_burst else sustained
    return {"achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sustained,
            "peak_source": f"{peak_src} {'bf16_tflops (burst' if use_burst else 'bf16_tflops_sustained (sustained'}"
                           f": the timed region lasted {timed_seconds:.3f} s)"}

WORKLOADS = {
    # name: (B, S, Hq, Hkv, D, packed segments?, description)
    "causal_c2": dict(B=4, S=8192, Hq=32, Hkv=8, D=128, segments=True,
                      text="configs[1]: causal fwd+bwd bf16 GQA B=4 S=8192 Hq=32 Hkv=8 D=128, packed segments ~U[512,4096], level 0"),
    "causal_small": dict(B=1, S=8192, Hq=32, Hkv=8, D=128, segments=False,
                         text="profiling case: dense causal B=1 S=8192 Hq=32 Hkv=8 D=128 (0.24 GB of tensors, above L2)"),
    "causal_c2_row": dict(B=1, S=8192, Hq=32, Hkv=8, D=128, segments=True,
                          text="profiling case: one batch row of configs[1] (causal, packed segments ~U[512,4096]; 0.17 GB of tensors, above L2)"),
    "copy_probe": dict(B=4, S=8192, Hq=32, Hkv=8, D=128, segments=True, copy_probe=True,
                       text="host <-> device copies of the headline step's end-to-end leg, no kernels"),
    "causal_c2_dense": dict(B=4, S=8192, Hq=32, Hkv=8, D=128, segments=False,
                            text="configs[1] shape with one segment per sequence (dense causal)"),
    # sequence-sharded across the ranks (strong scaling): each rank holds S / N tokens and receives a
    # window-sized K/V halo from its predecessor
    "swa_c3": dict(B=1, S=32768, Hq=32, Hkv=8, D=128, segments=False, window=4096,
                   text="configs[2]: sliding-window fwd+bwd bf16 B=1 S=32768 Hq=32 Hkv=8 D=128 window=4096, sequence-sharded with KV halo exchange"),
    # causal attention over one long sequence, sequence-sharded in the zig-zag layout (strong scaling):
    # ring of K/V blocks, every rank computes half a block per step
    "ring_causal": dict(B=1, S=32768, Hq=32, Hkv=8, D=128, segments=False, ring=True,
                        text="causal fwd+bwd bf16 B=1 S=32768 Hq=32 Hkv=8 D=128, one sequence sharded over the ranks (zig-zag ring of K/V blocks)"),
    # configs[3] and configs[4]: device-resident timing only (no host-buffer leg)
    "sca_c4": dict(B=2, S=16384, Hq=16, Hkv=1, D=128, segments=False, other="sca", span=2048, dtype="fp16", std=0.5,
                   text="configs[3]: sliding-chunk fwd+bwd fp16 MQA B=2 S=16384 Hq=16 Hkv=1 D=128 chunk=2048, BOS every ~U[1024,8192] tokens"),
    "softdelta_c5": dict(B=2, S=8192, Hq=16, Hkv=16, D=128, segments=False, other="softdelta", dtype="bf16", std=1.0,
                         text="configs[4]: SoftDelta fwd+bwd bf16 B=2 S=8192 Hq=Hkv=16 D=128, gates ~U(0,1)"),
    "sw_softdelta_c5": dict(B=2, S=8192, Hq=16, Hkv=16, D=128, segments=False, other="softdelta", span=2048, dtype="bf16", std=1.0,
                            text="configs[4]: sliding-window SoftDelta fwd+bwd bf16 B=2 S=8192 Hq=Hkv=16 D=128 window=2048, gates ~U(0,1)"),
    # one new token per sequence against a long key cache: forward only, HBM-bound (K and V are
    # streamed once); reported in GB/s of K + V + q + y bytes, not in the headline metric
    "decode": dict(B=8, S=32768, Hq=32, Hkv=8, D=128, segments=False, decode=True,
                   text="decode: causal forward bf16 GQA B=8 Lq=1 Lk=32768 Hq=32 Hkv=8 D=128 (1.07 GB of K and V per step, above L2)"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f), "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


def make_host_inputs(w, seed):
    """q, k, v, dy as bf16 host tensors drawn N(0,1) in fp32 from a seeded generator; int64 segment ids."""
    g = torch.Generator().manual_seed(seed)
    B, S, Hq, Hkv, D = w["B"], w["S"], w["Hq"], w["Hkv"], w["D"]
    draw = lambda *shape: torch.randn(shape, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, dy = draw(B, S, Hq, D), draw(B, S, Hkv, D), draw(B, S, Hkv, D), draw(B, S, Hq, D)
    ids = None
    if w["segments"]:
        ids = torch.zeros(B, S, dtype=torch.int64)
        for b in range(B):
            pos, seg = 0, 0
            while pos < S:
                length = int(torch.randint(w.get("seg_lo", 512), w.get("seg_hi", 4096) + 1, (1,), generator=g))
                ids[b, pos:pos + length] = seg
                pos += length
                seg += 1
    return q, k, v, dy, ids


_ORIGINAL_AFFINITY = None


def bind_to_gpu_numa_node(local_rank):
    """Run this process (and so first-touch its pinned host buffers) on the CPUs of the NUMA node the GPU
    hangs off: with one rank per GPU and every rank copying 1.3 GB per step, buffers that all sit on one
    socket make the other socket's GPUs cross the inter-socket link both ways.  Best effort: returns what
    was found and done; containers that hide the topology simply stay unbound."""
    global _ORIGINAL_AFFINITY
    _ORIGINAL_AFFINITY = os.sched_getaffinity(0)
    info = {"numa_node": None, "cpus_before": len(_ORIGINAL_AFFINITY), "bound": False}
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(local_rank)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:          # NVML pads the PCI domain to eight digits, sysfs uses four
            bus = bus[4:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus |= set(range(int(lo), int(hi or lo) + 1))
        usable = cpus & os.sched_getaffinity(0)
        if usable:
            os.sched_setaffinity(0, usable)
            info.update(bound=True, cpus_after=len(usable))
    except Exception as exc:                       # no NVML, no sysfs, no permission: stay as we are
        info["error"] = type(exc).__name__
    return info


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_event = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop_event.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def stop(self):
        self._stop_event.set()
        if self.is_alive():
            self.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def cpu_reference():
    """(module, kind): the reference's own CPU oracle compiled into oracle/_ref (kind "reference") when it
    has been built (oracle/build_ref.py), else the restatement in oracle/ (kind "port")."""
    from oracle import build_ref
    ref = build_ref.load("_reference")
    if ref is not None:
        return ref, "reference"
    from oracle import attention_oracle
    return attention_oracle, "port"


def cpu_mask(impl, kind, length, ids):
    """[1, L, L] causal mask with segment isolation, built once outside the timed steps."""
    if kind == "reference":
        return impl._allowed_masks(length, length, 1, torch.device("cpu"), "full", None, ids, ids, False)[0]
    return impl.allowed_masks(length, length, 1, "full", None, ids, ids, False)[0]


def cpu_step(impl, kind, q, k, v, dy, mask):
    """One masked-softmax read forward + autograd backward in fp32 on the host; returns seconds."""
    read = impl._attention_from_mask if kind == "reference" else impl.attention_from_mask
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    t0 = time.perf_counter()
    y = read(*leaves, mask, q.shape[-1] ** -0.5)
    torch.autograd.grad(y, leaves, dy)
    return time.perf_counter() - t0


def cpu_baseline_config0(threads):
    """The reference's CPU-sized configuration (configs[0]): B=2, S=1024, Hq=Hkv=8, D=64, fp32."""
    impl, kind = cpu_reference()
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    B, S, H, D = 2, 1024, 8, 64
    q, k, v, dy = (torch.randn(B, S, H, D, generator=g) for _ in range(4))
    mask = cpu_mask(impl, kind, S, None).expand(B, -1, -1)
    times = [cpu_step(impl, kind, q, k, v, dy, mask) for _ in range(3)]
    pairs = B * H * S * (S + 1) // 2
    flops = 14 * D * pairs
    t = statistics.median(times)
    return {"value": flops / t * 1e-12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": "configs[0] in full (B=2 S=1024 Hq=Hkv=8 D=64 fp32 fwd+bwd), median of 3, "
                      f"{t:.3f} s per step"}


def run_reference(args, w):
    """CPU arm: the reference's own oracle (tests/_reference.py compiled into oracle/_ref; the restatement
    in oracle/ where that has not been built) on the host cores, with all the threads torch can use."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    impl, kind = cpu_reference()
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, k, v, dy, ids = make_host_inputs(w, seed=1)
    # bounded sample: batch row 0, query head 0 (with its KV head), full sequence
    qs, ks, vs, dys = (t[:1, :, :1].float() for t in (q, k, v, dy))
    ids_s = None if ids is None else ids[:1]
    mask = cpu_mask(impl, kind, w["S"], ids_s)
    flops = 14 * w["D"] * int(mask.sum())
    for _ in range(min(args.warmup, 1)):
        cpu_step(impl, kind, qs, ks, vs, dys, mask)
    dt = sum(cpu_step(impl, kind, qs, ks, vs, dys, mask) for _ in range(args.steps)) / args.steps
    value = flops / dt * 1e-12
    sample = ("one step = batch row 0, query head 0 of the workload (1/128 of a full step): the masked softmax read "
              "and its autograd backward in fp32 torch on the host, mask built once beforehand")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["text"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args, w):
    import torch.distributed as dist
    import xattn_b200 as xattn
    from xattn_b200 import _native

    # Every timed step builds its mask plan, as a training step with fresh masks would: the library's
    # plan cache (which would find the same segment-id tensor again every step) is off for the bench.
    os.environ["XATTN_B200_PLAN_CACHE"] = "0"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL kernels on high-priority streams: an exchange posted while an attention kernel fills the GPU
        # then starts when the first CTA retires instead of after the last one was scheduled
        dist.init_process_group("nccl", device_id=dev,
                                pg_options=dist.ProcessGroupNCCL.Options(is_high_priority_stream=True))

    host_binding = None if args.no_numa_bind else bind_to_gpu_numa_node(local)
    if w.get("copy_probe"):
        return run_copy_probe(args, w, world, rank, dev, host_binding)
    if "window" in w or w.get("ring"):
        return run_swa_sharded(args, w, world, rank, dev)
    if w.get("decode"):
        return run_decode(args, w, world, rank, dev)
    if w.get("other"):
        return run_other(args, w, world, rank, dev)
    host = make_host_inputs(w, seed=1 + rank)
    pinned = [None if t is None else t.pin_memory() for t in host]
    q, k, v, dy, ids = (None if t is None else t.to(dev) for t in pinned)
    meta = {} if ids is None else {"segment_idx": ids}
    D = w["D"]

    # algorithmic work of one step on this rank: 14 * D * visible pairs over query heads
    plan = _native.build_plan(w["B"], w["S"], w["S"], dev, q_segment_idx=ids, k_segment_idx=ids)
    n = w["B"] * w["S"]
    r4 = (n + 3) // 4 * 4
    pairs = int((plan[r4:r4 + n].long() - plan[:n].long()).clamp_min(0).sum().item()) * w["Hq"]
    flops_step = 14 * D * pairs

    level = args.level

    leaves = [t.requires_grad_() for t in (q, k, v)]

    def step():
        # the training form of the op: forward, then autograd's backward on the forward's saved state
        # (one mask plan per step; at level 1 the backward reuses the forward's statistics and anchors)
        y = xattn.causal_flash_attn(*leaves, **meta, high_precision_level=level)
        return (y, *torch.autograd.grad(y, leaves, dy))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    _native.check_status()

    # ---- device-resident timing -------------------------------------------------------------
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    _native.profile_enable(True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    _native.profile_enable(False)
    records = _native.profile_read()
    ms_total = e0.elapsed_time(e1)
    _native.check_status()

    # ---- end to end: host buffers in, host buffers out ------------------------------------------
    out_host = None
    h2d = sum(t.numel() * t.element_size() for t in pinned[:4])

    # Batch rows are independent, so the step is pipelined over them: row b + 1 comes in over PCIe
    # and row b - 1 goes out while row b is computed (one copy stream per direction).
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    Bn = w["B"]
    # two sets of device input buffers: the inputs of step i + 1 come in while step i's results go out
    dev_sets = [[torch.empty_like(t, device=dev) for t in pinned[:4]] for _ in range(2)]
    set_free = [None, None]
    step_no = 0
    ids_rows = None if ids is None else [ids[b:b + 1] for b in range(Bn)]

    def e2e_step():
        nonlocal out_host, step_no
        main = torch.cuda.current_stream(dev)
        which = step_no & 1
        step_no += 1
        dev_in = dev_sets[which]
        if set_free[which] is not None:
            s_in.wait_event(set_free[which])      # the kernels of two steps ago have read this set
        arrived = []
        with torch.cuda.stream(s_in):
            for b in range(Bn):
                # q, k, v first: the forward can start (and y can leave) while dy is still coming in
                for dst, src in zip(dev_in[:3], pinned[:3]):
                    dst[b:b + 1].copy_(src[b:b + 1], non_blocking=True)
                ev_qkv = torch.cuda.Event()
                ev_qkv.record(s_in)
                dev_in[3][b:b + 1].copy_(pinned[3][b:b + 1], non_blocking=True)
                ev_dy = torch.cuda.Event()
                ev_dy.record(s_in)
                arrived.append((ev_qkv, ev_dy))

        def send_back(b, outs, first):
            nonlocal out_host
            done = torch.cuda.Event()
            done.record(main)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                for j, src in enumerate(outs):
                    src.record_stream(s_out)
                    out_host[first + j][b:b + 1].copy_(src, non_blocking=True)

        for b in range(Bn):
            q_, k_, v_, dy_ = (t[b:b + 1] for t in dev_in)
            meta_b = {} if ids_rows is None else {"segment_idx": ids_rows[b]}
            main.wait_event(arrived[b][0])
            y_, lse_ = xattn.causal_flash_attn_fwd(q_, k_, v_, **meta_b, high_precision_level=level)
            if out_host is None:
                out_host = [torch.empty((Bn,) + tuple(t.shape[1:]), dtype=t.dtype).pin_memory()
                            for t in (y_, q_, k_, v_)]
            send_back(b, (y_,), 0)
            main.wait_event(arrived[b][1])
            grads = xattn.causal_flash_attn_bwd(dy_, q_, k_, v_, y_, lse_, **meta_b, high_precision_level=level)
            send_back(b, grads[:3], 1)
        set_free[which] = torch.cuda.Event()
        set_free[which].record(main)

    def e2e_drain():
        main = torch.cuda.current_stream(dev)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))
    for _ in range(0 if args.no_e2e else 2):
        e2e_step()
    e2e_drain()
    barrier()
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()                 # the last step's results are on the host before the clock stops
    f1.record()
    barrier()
    e2e_ms_total = f0.elapsed_time(f1)
    clocks = sampler.stop()
    d2h = sum(t.numel() * t.element_size() for t in out_host) if out_host else 0

    times = torch.tensor([ms_total / args.steps, e2e_ms_total / max(e2e_steps, 1)], dtype=torch.float64, device=dev)
    work = torch.tensor([float(flops_step)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    ms_step, e2e_ms_step = float(times[0]), float(times[1])
    total_flops = float(work[0])

    # With more than one GPU the sequence-sharded workloads run in the same process group, after the
    # headline measurement: configs[2] with its K/V halo exchange, and the causal ring.
    sharded = None
    if world > 1 and not args.no_sharded:
        del q, k, v, dy, dev_sets, out_host
        torch.cuda.empty_cache()
        sharded = {}
        for name in ("swa_c3", "ring_causal"):
            # the ring comes second: the window workload's chain exchanges have connected the neighbour links by then
            res = measure_sharded(args, WORKLOADS[name], world, rank, dev, with_e2e=False, steps=max(3, min(args.steps, 10)),
                                  ring_links=(name == "ring_causal"))
            if rank == 0:
                sharded[name] = {key: res[key] for key in (
                    "metric", "value", "unit", "ms_per_step", "scaling", "per_gpu_tflops", "single_gpu_ms",
                    "efficiency_vs_1gpu", "launch", "transport", "eager_ms_per_step", "eager_host_enqueue_ms_per_step",
                    "kernel_ms_per_step", "kernel_ms_per_step_slowest_rank",
                    "non_kernel_ms_per_step", "work_share_of_slowest_rank", "slice_rows", "kernels")}
                sharded[name]["workload"] = res["config"]["workload"]

    if rank == 0:
        peaks, peak_src = measured_peaks()
        per_kind = {}
        for kind, ms in records:
            per_kind.setdefault(kind, []).append(ms)
        launches = len(records)  # one record per scope; a plan scope holds four small kernels
        launches += 3 * len(per_kind.get("plan", []))
        # algorithmic FLOPs per launch: forward 4*D*P; in the backward the dQ kernel's S / dP
        # products repeat the dK/dV kernel's, so only its dQ product is new work
        algo = {"fwd": 4 * D * pairs, "bwd_dq": 2 * D * pairs, "bwd_dkv": 8 * D * pairs}
        executed = {"fwd": 4 * D * pairs, "bwd_dq": 6 * D * pairs, "bwd_dkv": 8 * D * pairs}
        kernels = {}
        for kind, vals in per_kind.items():
            avg = sum(vals) / len(vals)
            entry = {"launches": len(vals), "avg_ms": avg, "share": sum(vals) / max(ms_total, 1e-9)}
            if kind in algo:
                entry["algorithmic_tflops"] = algo[kind] / avg * 1e-9
                entry["executed_tflops"] = executed[kind] / avg * 1e-9
            kernels[kind] = entry
        dominant = max((kd for kd in kernels if kd in algo), key=lambda kd: kernels[kd]["avg_ms"] * kernels[kd]["launches"])
        peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
        achieved = kernels[dominant]["algorithmic_tflops"]
        packing = "packed" if w["segments"] else "dense"
        row_traffic = NCU_DRAM_BYTES_PER_BATCH_ROW[packing].get(dominant)
        line = {
            "metric": METRIC, "value": total_flops / ms_step * 1e-9, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["text"] if level == 0 else w["text"].replace("level 0", "level 1"),
                       "high_precision_level": level, "l2": "inputs (0.67 GB per step) exceed the 126 MB L2",
                       "mask_plan": "built in every step (plan cache off)",
                       "visible_pairs_per_step": pairs, "flops_per_step": flops_step,
                       "parallelism": f"batch x heads sharded over {world} GPU(s): embarrassingly parallel, no "
                                      "communication (every rank runs its own batch); the sequence-sharded "
                                      "workloads with their exchanges are under 'sharded' when more than one GPU runs"},
            "per_gpu_tflops": total_flops / ms_step * 1e-9 / world,
            "frac_of_measured_bf16_peak": {
                "burst": total_flops / ms_step * 1e-9 / world / float(peaks.get("bf16_tflops", peak)),
                "sustained": total_flops / ms_step * 1e-9 / world / peak, "source": peak_src},
            "e2e": None if not e2e_steps else {
                "value": total_flops / e2e_ms_step * 1e-9, "unit": "TFLOP/s", "ms_per_step": e2e_ms_step,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "host": host_binding,
            "roofline": {"bound": "tensor", "kernel": dominant,
                         **tensor_roofline(achieved, peaks, peak_src, ms_total * 1e-3),
                         "traffic": row_traffic * w["B"] if row_traffic else None,
                         "traffic_source": (f"ncu dram__bytes_read.sum + dram__bytes_write.sum of one {dominant} launch on "
                                            f"one {packing} batch row of this workload, times the {w['B']} batch rows"
                                            if row_traffic else None),
                         "executed_tflops": kernels[dominant]["executed_tflops"]},
            "kernels": kernels,
        }
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1 and not args.no_cpu_baseline:
            if _ORIGINAL_AFFINITY:
                os.sched_setaffinity(0, _ORIGINAL_AFFINITY)      # the CPU baseline gets every core back
            line["cpu_baseline"] = cpu_baseline_config0(os.cpu_count() or 1)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_copy_probe(args, w, world, rank, dev, host_binding):
    """The host-buffer leg of the headline step with the kernels taken out: every rank copies its
    q, k, v, dy (0.67 GB) from pinned memory to the GPU and as many bytes back, both directions at
    once, batch row by batch row as the end-to-end step does.  Shows what the host side of N
    simultaneous ranks delivers per GPU."""
    import torch.distributed as dist
    host = make_host_inputs(WORKLOADS["causal_c2"], seed=1 + rank)
    pinned = [t.pin_memory() for t in host[:4]]
    back = [torch.empty_like(t).pin_memory() for t in pinned]
    dev_in = [torch.empty_like(t, device=dev) for t in pinned]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    nbytes = sum(t.numel() * t.element_size() for t in pinned)

    def step(h2d=True, d2h=True):
        for b in range(pinned[0].shape[0]):
            if h2d:
                with torch.cuda.stream(s_in):
                    for dst, src in zip(dev_in, pinned):
                        dst[b:b + 1].copy_(src[b:b + 1], non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    for dst, src in zip(back, dev_in):
                        dst[b:b + 1].copy_(src[b:b + 1], non_blocking=True)

    def timed(**kw):
        for _ in range(3):
            step(**kw)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step(**kw)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / args.steps

    res = {}
    for name, kw in (("h2d_alone", dict(d2h=False)), ("d2h_alone", dict(h2d=False)), ("both", {})):
        dt = timed(**kw)
        rates = torch.tensor([nbytes / dt * 1e-9], dtype=torch.float64, device=dev)
        if world > 1:
            gathered = [torch.zeros_like(rates) for _ in range(world)]
            dist.all_gather(gathered, rates)
            rates = torch.cat(gathered)
        res[name] = {"gb_per_s_per_direction_min": float(rates.min()), "max": float(rates.max()),
                     "sum_over_ranks": float(rates.sum()), "ms": dt * 1e3}
    nodes = [host_binding]
    if world > 1:
        nodes = [None] * world
        dist.all_gather_object(nodes, host_binding)
    if rank == 0:
        print(json.dumps({"metric": "host <-> device copy rate of the end-to-end leg, per GPU", "unit": "GB/s",
                          "n_gpus": world, "steps": args.steps, "bytes_per_direction_per_step": nbytes,
                          "value": res["both"]["gb_per_s_per_direction_min"], "higher_is_better": True,
                          "rates": res, "host": nodes, "cpu_count": os.cpu_count()}))
    if world > 1:
        dist.destroy_process_group()


def run_decode(args, w, world, rank, dev):
    """Forward of Lq = 1 against Lk = S keys per sequence; every rank runs its own batch."""
    import torch.distributed as dist
    import xattn_b200 as xattn
    from xattn_b200 import _native

    B, S, Hq, Hkv, D = w["B"], w["S"], w["Hq"], w["Hkv"], w["D"]
    gen = torch.Generator().manual_seed(7 + rank)
    q = torch.randn(B, 1, Hq, D, generator=gen).to(dev, torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, generator=gen).to(dev, torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, generator=gen).to(dev, torch.bfloat16)
    # algorithmic bytes of one step: K and V read once, q read, y and lse written
    nbytes = (k.numel() + v.numel() + 2 * q.numel()) * 2 + B * Hq * 4

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        xattn.causal_flash_attn_fwd(q, k, v)
    _native.check_status()
    sampler = ClockSampler(dev.index)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    _native.profile_enable(True)
    e0.record()
    for _ in range(args.steps):
        xattn.causal_flash_attn_fwd(q, k, v)
    e1.record()
    barrier()
    _native.profile_enable(False)
    records = _native.profile_read()
    clocks = sampler.stop()
    _native.check_status()
    # The repeated-mask inference path of the reference's sliding-chunk op keeps its forward plan between
    # calls.  The same question here: one decode step with a BOS mask over the key cache, plan cache off
    # and on (the mask tensor is the same every step, as in a serving loop between cache updates).
    bos = torch.zeros(B, S, dtype=torch.bool, device=dev)
    bos[:, ::4096] = True
    cache_ms = {}
    for state in ("0", "1"):
        os.environ["XATTN_B200_PLAN_CACHE"] = state
        with torch.inference_mode():
            for _ in range(5):
                xattn.flash_sca_fwd(q, k, v, 2048, bos_mask=bos)
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            c0.record()
            for _ in range(50):
                xattn.flash_sca_fwd(q, k, v, 2048, bos_mask=bos)
            c1.record()
            torch.cuda.synchronize()
        cache_ms["off" if state == "0" else "on"] = c0.elapsed_time(c1) / 50
    os.environ["XATTN_B200_PLAN_CACHE"] = "0"
    _native.check_status()
    times = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step = float(times[0])
    if rank == 0:
        peaks, peak_src = measured_peaks()
        fwd = [ms for kind, ms in records if kind == "fwd"]      # split kernel + merge kernel
        kernel_ms = sum(fwd) / max(len(fwd), 1)
        peak = float(peaks["hbm_gbs"])
        achieved = nbytes / kernel_ms * 1e-6
        print(json.dumps({
            "metric": "decode attention forward, GB/s of K and V streamed, whole job", "value": world * nbytes / ms_step * 1e-6,
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["text"], "l2": "K and V (1.07 GB per step) exceed the 126 MB L2",
                       "bytes_per_step": nbytes, "parallelism": f"batch sharded over {world} GPU(s), no communication"},
            # a forward scope holds the split kernel and the merge kernel, a one-tile plan is one kernel
            "gpu_launches": 2 * len(fwd) + len([1 for kind, _ in records if kind == "plan"]),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "fwd (decode shape) + merge", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_DRAM_BYTES_DECODE,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of each "
                                           "kernel on this workload",
                         "peak_source": f"{peak_src} hbm_gbs (copy bandwidth)"},
            "kernel_ms": kernel_ms,
            "plan_cache": {"workload": "sliding-chunk decode step (chunk 2048) with a BOS mask over the 32768 cached keys, "
                                       "same mask tensor every step, launched from Python under inference mode",
                           "ms_per_step_cache_off": cache_ms["off"], "ms_per_step_cache_on": cache_ms["on"]},
        }))
    if world > 1:
        dist.destroy_process_group()


def run_other(args, w, world, rank, dev):
    """configs[3] (sliding chunk, fp16, MQA, BOS packing) and configs[4] (SoftDelta and its sliding-window form):
    forward + backward through the public ops with inputs resident in HBM; every rank runs its own batch."""
    import torch.distributed as dist
    import xattn_b200 as xattn
    from xattn_b200 import _native

    B, S, Hq, Hkv, D = w["B"], w["S"], w["Hq"], w["Hkv"], w["D"]
    dt = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    gen = torch.Generator().manual_seed(3 + rank)
    draw = lambda *shape: (torch.randn(shape, generator=gen) * w["std"]).to(dev, dt)
    q, k, v, dy = draw(B, S, Hq, D), draw(B, S, Hkv, D), draw(B, S, Hkv, D), draw(B, S, Hq, D)
    level = args.level

    def count_pairs(**plan_kw):
        plan = _native.build_plan(B, S, S, dev, **plan_kw)
        n = B * S
        r4 = (n + 3) // 4 * 4
        return int((plan[r4:r4 + n].long() - plan[:n].long()).clamp_min(0).sum().item())

    if w["other"] == "sca":
        bos = torch.zeros(B, S, dtype=torch.bool)
        bos[:, 0] = True
        for b in range(B):
            pos = 0
            while True:
                pos += int(torch.randint(1024, 8193, (1,), generator=gen))
                if pos >= S:
                    break
                bos[b, pos] = True
        bos = bos.to(dev)
        ids = bos.cumsum(1)
        pairs = Hq * count_pairs(visibility="chunk", span=w["span"], q_segment_idx=ids, k_segment_idx=ids)

        def step():
            y, lse = xattn.flash_sca_fwd(q, k, v, w["span"], bos_mask=bos, high_precision_level=level)
            return xattn.flash_sca_bwd(dy, q, k, v, y, lse, w["span"], bos_mask=bos, high_precision_level=level)
    else:
        gate = torch.rand(B, S, Hq, generator=gen).to(dev, dt)
        span = w.get("span")
        vis = dict(visibility="window", span=span) if span else {}
        # the query read over query heads plus the strict-past read over KV heads
        pairs = Hq * count_pairs(**vis) + Hkv * count_pairs(strict_past=True, **vis)

        def step():
            leaves = [t.detach().requires_grad_() for t in (q, k, v, gate)]
            if span:
                y = xattn.sliding_window_softdelta_attention(q=leaves[0], k=leaves[1], k_read=None, v=leaves[2], g=leaves[3],
                                                             window_size=span, high_precision_level=level)
            else:
                y = xattn.softdelta_attention(q=leaves[0], k=leaves[1], k_read=None, v=leaves[2], g=leaves[3],
                                              high_precision_level=level)
            return torch.autograd.grad(y, leaves, dy)

    flops_step = 14 * D * pairs

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    _native.check_status()
    sampler = ClockSampler(dev.index)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    _native.profile_enable(True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    _native.profile_enable(False)
    records = _native.profile_read()
    clocks = sampler.stop()
    _native.check_status()
    times = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step = float(times[0])
    if rank == 0:
        peaks, peak_src = measured_peaks()
        peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
        per_kind = {}
        for kind, ms in records:
            per_kind.setdefault(kind, []).append(ms)
        kernels = {kd: {"launches": len(vs), "ms_per_step": sum(vs) / args.steps, "share": sum(vs) / (ms_step * args.steps)}
                   for kd, vs in per_kind.items()}
        dkv_ms = kernels.get("bwd_dkv", {"ms_per_step": float("inf")})["ms_per_step"]
        achieved = 8 * D * pairs / dkv_ms * 1e-9
        print(json.dumps({
            "metric": "attn fwd+bwd TFLOPS, whole job", "value": world * flops_step / ms_step * 1e-9, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": w["text"], "high_precision_level": level, "l2": "tensors of one step exceed the 126 MB L2",
                       "visible_pairs_per_step": pairs, "flops_per_step": flops_step,
                       "parallelism": f"batch sharded over {world} GPU(s), no communication"},
            # a plan scope holds four kernels, a level-1 repair scope three, every other scope one
            "gpu_launches": len(records) + 3 * len(per_kind.get("plan", [])) + 2 * len(per_kind.get("repair", [])),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "bwd_dkv (all its launches of a step)",
                         **tensor_roofline(achieved, peaks, peak_src, ms_step * args.steps * 1e-3), "traffic": None},
            "kernels": kernels,
        }))
    if world > 1:
        dist.destroy_process_group()


def window_slice_bounds(S, world, window, equal=False, shortest=None):
    """Row boundaries of the ranks' contiguous slices of a causal sliding-window workload: about equal
    numbers of visible pairs per slice (the first ``window`` rows of the sequence see fewer keys, so with
    equal slices rank 0 has less to do than everybody else), boundaries on multiples of 128 rows, every
    slice at least ``shortest`` rows long (default: one window, so that the halo comes from the previous
    rank alone; half a window makes the halo reach two ranks back).  Where that cannot be had (eight ranks
    over 32768 rows with a window of 4096: an equal slice IS one window), or with ``equal``, equal slices."""
    import bisect
    even = [r * (S // world) for r in range(world + 1)]
    if equal or world == 1:
        return even
    cum, acc = [], 0
    for i in range(S):
        acc += min(i, window) + 1
        cum.append(acc)
    cand = [0] + [min(S, (bisect.bisect_left(cum, acc * r / world) + 1 + 64) // 128 * 128) for r in range(1, world)] + [S]
    least = max(window if shortest is None else shortest, 128)
    return cand if all(b - a >= least for a, b in zip(cand, cand[1:])) else even


def measure_sharded(args, w, world, rank, dev, with_e2e, steps, ring_links=False):
    """One sequence of S tokens split over the ranks of the current process group, total work fixed:
    configs[2] (sliding window, contiguous slices, K/V halo exchange) or the causal ring (zig-zag
    slices).  Returns the result dictionary on rank 0 (None elsewhere).  Rank 0 also times the same
    sequence unsharded on its own GPU while the others wait, for the strong-scaling efficiency."""
    import torch.distributed as dist
    import xattn_b200 as xattn
    from xattn_b200 import _native, parallel as P

    ring = bool(w.get("ring"))
    # a two-rank communicator per pair of neighbours (a transfer inside the N-rank communicator gets a
    # share of the channels that shrinks with N); XATTN_BENCH_NO_LINKS=1 keeps everything on the job's own
    links = world > 2 and not os.environ.get("XATTN_BENCH_NO_LINKS")
    if links and not P.neighbor_links_open():
        P.open_neighbor_links()
    S, D, window = w["S"], w["D"], w.get("window", 0)
    if S % (2 * world) or S // world < window:
        raise SystemExit("sequence length must split into even slices of at least one window")
    bounds = ([r * (S // world) for r in range(world + 1)] if ring else
              window_slice_bounds(S, world, window, equal=bool(os.environ.get("XATTN_BENCH_EQUAL_SLICES")),
                                  shortest=window // 2 if os.environ.get("XATTN_BENCH_SHORT_SLICES") else window))
    lengths = [b - a for a, b in zip(bounds, bounds[1:])]
    g = torch.Generator().manual_seed(2)
    draw = lambda *shape: torch.randn(shape, generator=g, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, dy = draw(1, S, w["Hq"], D), draw(1, S, w["Hkv"], D), draw(1, S, w["Hkv"], D), draw(1, S, w["Hq"], D)
    sl = P.zigzag_indices(S, rank, world) if ring else slice(bounds[rank], bounds[rank + 1])
    pinned = [t[:, sl].contiguous().pin_memory() for t in (q, k, v, dy)]
    ql, kl, vl, dyl = (t.to(dev) for t in pinned)
    pairs = w["Hq"] * (S * (S + 1) // 2 if ring else sum(min(i, window) + 1 for i in range(S)))   # whole job
    flops_step = 14 * D * pairs

    def step(a, b, c, d):
        a, b, c = (t.detach().requires_grad_() for t in (a, b, c))
        y = (P.ring_causal_flash_attn(a, b, c, layout="zigzag", use_links=links and ring_links) if ring else
             P.sequence_parallel_flash_swa(a, b, c, window, slice_lengths=lengths))
        return (y, *torch.autograd.grad(y, (a, b, c), d))

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(ql, kl, vl, dyl)
    _native.check_status()
    # 1. A few eager steps with the library's per-launch events on: the kernel breakdown, and what a step
    #    costs when every launch and every NCCL call is issued from Python.
    eager_steps = max(3, min(steps, 5))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    _native.profile_enable(True)
    h0 = time.perf_counter()
    e0.record()
    for _ in range(eager_steps):
        step(ql, kl, vl, dyl)
    e1.record()
    host_ms = (time.perf_counter() - h0) / eager_steps * 1e3
    barrier()
    _native.profile_enable(False)
    records = _native.profile_read()
    eager_ms = e0.elapsed_time(e1) / eager_steps
    # 2. The timed region: the same step captured once in a CUDA graph (exchanges included: NCCL send / recv
    #    are stream operations) and replayed.  A sharded step is short (about a millisecond of kernels per
    #    rank at eight GPUs) against some forty Python-issued launches and two NCCL group calls of about half a
    #    millisecond of host time each, so issued eagerly it is bound by the host, not by the GPUs or NVLink.
    #    XATTN_BENCH_NO_GRAPH=1 times the eager step instead.
    launch = "eager (one Python call per launch)"
    graph = None
    if not os.environ.get("XATTN_BENCH_NO_GRAPH"):
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step(ql, kl, vl, dyl)
        torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = step(ql, kl, vl, dyl)
        barrier()
        for _ in range(3):
            graph.replay()
        launch = "CUDA graph replay of the captured step, exchanges included"
    run = graph.replay if graph is not None else (lambda: step(ql, kl, vl, dyl))
    sampler = ClockSampler(dev.index)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    g0.record()
    for _ in range(steps):
        run()
    g1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = g0.elapsed_time(g1) / steps
    _native.check_status()
    if graph is not None:
        # the graph holds NCCL work: it has to be gone before the process group is torn down (a live
        # graph made the teardown wait for ever), so it goes before anything else happens
        del graph, captured, run
        import gc
        gc.collect()
        torch.cuda.synchronize()
    barrier()
    out_host = None
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(steps, 10)) if with_e2e else 0

    def e2e_step():
        nonlocal out_host
        outs = step(*(t.to(dev, non_blocking=True) for t in pinned))
        if out_host is None:
            out_host = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        for dst, src in zip(out_host, outs):
            dst.copy_(src, non_blocking=True)

    for _ in range(2 if with_e2e else 0):
        e2e_step()
    barrier()
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / max(e2e_steps, 1)
    # the same sequence unsharded on one GPU (rank 0 alone), device-timed
    single_ms = None
    if world > 1 and rank == 0:
        qf, kf, vf, dyf = (t.to(dev) for t in (q, k, v, dy))

        def single():
            a, b, c = (t.detach().requires_grad_() for t in (qf, kf, vf))
            y = xattn.causal_flash_attn(a, b, c) if ring else xattn.flash_swa(a, b, c, window)
            return torch.autograd.grad(y, (a, b, c), dyf)

        for _ in range(3):
            single()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(max(3, min(steps, 5))):
            single()
        s1.record()
        torch.cuda.synchronize()
        single_ms = s0.elapsed_time(s1) / max(3, min(steps, 5))
        _native.check_status()
        del qf, kf, vf, dyf
    barrier()
    own_kernel_ms = sum(t for _, t in records) / eager_steps
    times = torch.tensor([ms, e2e_ms, own_kernel_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, slowest_kernel_ms = float(times[0]), float(times[1]), float(times[2])
    if rank != 0:
        return None
    peaks, peak_src = measured_peaks()
    per_kind = {}
    for kind, t in records:
        per_kind.setdefault(kind, []).append(t)
    kernels = {kd: {"launches": len(vs), "avg_ms": sum(vs) / len(vs), "ms_per_step": sum(vs) / eager_steps,
                    "share": sum(vs) / (ms * eager_steps)} for kd, vs in per_kind.items()}
    kernel_ms = sum(kv["ms_per_step"] for kv in kernels.values())
    rank_pairs = pairs / world
    dkv = kernels.get("bwd_dkv", {"avg_ms": float("inf"), "launches": 1})
    # the ring launches the kernel once per block step; the work of a rank is spread over them
    achieved = 8 * D * rank_pairs / (dkv["avg_ms"] * dkv["launches"] / eager_steps) * 1e-9
    h2d = sum(t.numel() * t.element_size() for t in pinned) * world
    d2h = sum(t.numel() * t.element_size() for t in out_host) * world if out_host else 0
    return {
        "metric": ("causal ring attn fwd+bwd TFLOPS (bf16 S=32K D=128), whole job" if ring else
                   "sliding-window attn fwd+bwd TFLOPS (bf16 S=32K w=4096 D=128), whole job"),
        "value": flops_step / ms * 1e-9, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["text"], "l2": "0.27 GB of tensors per step in total",
                   "visible_pairs_per_step": pairs, "flops_per_step": flops_step,
                   "parallelism": (f"sequence split over {world} GPU(s) in the zig-zag layout; ring of K/V blocks "
                                   "(NCCL send/recv), partial outputs merged by lse, dK/dV travel home with their block"
                                   if ring else
                                   f"sequence split over {world} GPU(s) in contiguous slices of about equal work; K/V "
                                   f"halo of {window} tokens from the previous rank (NCCL send/recv), halo gradients sent back")},
        "per_gpu_tflops": flops_step / ms * 1e-9 / world,
        # strong scaling: time of the unsharded sequence on one GPU over N times the sharded time
        "single_gpu_ms": single_ms,
        "efficiency_vs_1gpu": None if single_ms is None else single_ms / (world * ms),
        # kernel time of rank 0 and of the slowest rank against the step: what is left of the step beyond the
        # slowest rank's kernels is exchange, copies and launch gaps.  With contiguous slices rank 0 has
        # less work than the others (its first rows see fewer keys), so it waits for them.
        "launch": launch,
        "transport": ("NCCL send/recv on high-priority streams, " +
                      ("one two-rank communicator per pair of neighbours" if links and (ring_links or not ring)
                       else "the job's communicator")),
        "eager_ms_per_step": eager_ms, "eager_host_enqueue_ms_per_step": host_ms,
        "kernel_ms_per_step": kernel_ms, "kernel_ms_per_step_slowest_rank": slowest_kernel_ms,
        "non_kernel_ms_per_step": ms - slowest_kernel_ms,
        "work_share_of_slowest_rank": (1.0 / world if ring else
                                       max(sum(min(i, window) + 1 for i in range(bounds[r], bounds[r + 1]))
                                           for r in range(world)) * w["Hq"] / pairs),
        "slice_rows": None if ring else [b - a for a, b in zip(bounds, bounds[1:])],
        "e2e": None if not e2e_steps else {"value": flops_step / e2e_ms * 1e-9, "unit": "TFLOP/s",
                                           "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                                           "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        # kernels of this library per timed step (counted on the eager steps) times the timed steps
        "gpu_launches": (len(records) + 3 * len(per_kind.get("plan", []))) // eager_steps * steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "bwd_dkv",
                     **tensor_roofline(achieved, peaks, peak_src, ms * steps * 1e-3), "traffic": None},
        "kernels": kernels,
    }


def run_swa_sharded(args, w, world, rank, dev):
    import torch.distributed as dist
    if world == 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=os.environ.get("MASTER_PORT", "29533"))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    line = measure_sharded(args, w, world, rank, dev, with_e2e=not args.no_e2e, steps=args.steps)
    if rank == 0:
        print(json.dumps(line))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default="causal_c2", choices=sorted(WORKLOADS))
    ap.add_argument("--level", type=int, default=0, choices=(0, 1),
                    help="high_precision_level (default 0; the causal, sca_c4 and softdelta workloads take 1 too)")
    ap.add_argument("--segment-lengths", default=None, metavar="LO,HI",
                    help="packed causal workloads: draw segment lengths ~U[LO,HI] instead of the headline's 512,4096 "
                         "(LO = HI gives equal segments)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="do not move the process to the CPUs of the GPU's NUMA node before pinning host buffers")
    ap.add_argument("--no-sharded", action="store_true",
                    help="with more than one GPU: skip the sequence-sharded workloads after the headline measurement")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.segment_lengths:
        lo, hi = (int(x) for x in args.segment_lengths.split(","))
        if not w.get("segments") or lo < 1 or hi < lo:
            raise SystemExit("--segment-lengths needs a packed causal workload and 1 <= LO <= HI")
        w = dict(w, seg_lo=lo, seg_hi=hi, text=w["text"].replace("~U[512,4096]", f"~U[{lo},{hi}]"))
    if args.impl == "reference" and (w.get("decode") or w.get("other") or w.get("copy_probe") or w["S"] > 8192):
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm runs the causal S=8192 workloads: one "
                          "(batch row, head) slice of a 32768-token sequence needs 4.3 GB per score matrix in fp32"}))
    elif args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
