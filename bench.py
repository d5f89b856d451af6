#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one causal GQA forward + backward pass over one batch of the sweep
configuration (batch 8, 32 query heads over 8 KV heads, head_dim 128, T 4096, f32,
i.i.d. N(0,1) inputs), i.e. 3.5 * 2*B*H*D*T*(T+1) floating-point operations by the
reference's own count (src/scale.zig:157-163; the backward is 5 GEMMs against the
forward's 2).  The line printed also carries the decode configuration (batch 64,
context 8192, Llama-3-8B heads) in GB/s, the roofline of the dominant kernel, the CPU
baseline (the oracle port timed on a bounded sample) and the end-to-end figure through
the reference-facing C ABI with host buffers.

With N > 1 (launched by torchrun, one rank per GPU) the same job -- batch 8 -- is SHARDED: every
rank runs 8 / N of the sequences (sequences are independent, so there is no data-path collective)
and the NCCL all-gather that returns out, dq, dk, dv to every rank is inside the timed region, on
a second stream so that it overlaps the next step's kernels.  `value` is the whole job's rate over
the slowest rank's time ("scaling": "strong"); the line also carries the phases by themselves
(`phases`: compute only, gather only), the replica run of the same per-GPU workload on every rank
(`weak`), the 32k prefill with its KV heads sharded (`long_context`) and the ragged decode with its
sequences balanced over the ranks (`ragged_decode`), both with their all-gathers timed.

`--impl reference` times the reference's CPU implementation of the same step (the C
restatement under oracle/, the reference itself being Zig and not buildable here) on the
host cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import threading
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The sweep point the headline is quoted on, and the decode configuration.
PREFILL = dict(batch=8, T=4096, n_heads=32, n_kv_heads=8, head_dim=128)
DECODE = dict(batch=64, n_ctx=8192, n_heads=32, n_kv_heads=8, head_dim=128)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


WORKLOAD = "causal GQA attention fwd+bwd, batch 8, 32/8 heads, head_dim 128, T 4096, f32"


def headline_config():
    """The `config` object, the same in both arms."""
    return {"workload": WORKLOAD, **PREFILL,
            "l2": "inputs (1.25 GiB per step) exceed the 126 MB L2; nothing is flushed between steps"}


def fwd_flops(batch, T, n_heads, head_dim):
    return 2.0 * batch * n_heads * head_dim * T * (T + 1)


def load_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the captured kernels, from the file
    written beside the ncu summaries: {kernel: {"bytes": ..., "units": sequences in the captured launch, ...}}.
    Traffic is per sequence, so a launch of B sequences moves bytes * B / units.  None when the file is absent."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read through NVML (the library nvidia-smi itself
    reads) every 2 ms from a thread while the timed region runs; `nvidia-smi -lms 50` when the NVML
    binding is absent.  A timed region of a few tens of milliseconds holds too few nvidia-smi samples
    to say anything about the clock under load."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.thread = None
        self.rows = []   # (sm MHz, max MHz, watts, reason bits)
        self.path = f"/tmp/zt_clocks_{os.getpid()}.csv"

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.gpu_index < len(ids) and ids[self.gpu_index].isdigit():
                return int(ids[self.gpu_index])
        return self.gpu_index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            mx = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            self._stop = False

            def loop():
                while not self._stop:
                    try:
                        self.rows.append((pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM), mx,
                                          pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0,
                                          pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=5)
            # NVML reason bits: 0x4 sw_power_cap, 0x8 hw_slowdown, 0x20 sw_thermal, 0x40 hw_thermal
            bits = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}
            reasons = set()
            for row in self.rows:
                for bit, name in bits.items():
                    if row[3] & bit:
                        reasons.add(name)
            sm = [r[0] for r in self.rows]
            return {"sm_mhz": statistics.median(sm) if sm else None,
                    "sm_min_mhz": min(sm) if sm else None,
                    "sm_max_mhz": self.rows[0][1] if self.rows else None,
                    "power_w": statistics.median([r[2] for r in self.rows]) if self.rows else None,
                    "samples": len(sm), "source": "nvml, 2 ms", "reasons": sorted(reasons)}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "source": "nvidia-smi -lms 50", "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def bind_near_gpu(local: int, world: int) -> str:
    """With several ranks on one host, run this rank on the CPUs NVML names as the GPU's own (its NUMA node), so
    that the pinned host buffers it allocates afterwards are first touched there and its copies do not cross the
    socket interconnect.  Returns a note for the JSON line.  Single-rank runs keep every CPU (the CPU baseline
    wants them)."""
    if world <= 1:
        return "unbound"
    try:
        import pynvml
        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = local
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if local < len(ids) and ids[local].isdigit():
                idx = int(ids[local])
        handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
        n_words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, n_words)
        cpus = {w * 64 + b for w, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return "unbound (no overlap with the allowed CPUs)"
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} CPUs of the GPU's NUMA node"
    except Exception as e:  # NVML binding absent, or the call is not supported here
        return f"unbound ({type(e).__name__})"


# ------------------------------------------------------------------------------------------------
# reference arm: the CPU port on a bounded sample
# ------------------------------------------------------------------------------------------------

def cpu_sample(threads: int, row_stride: int, repeats: int, warmup: int):
    """Times every row_stride-th query row of the prefill step on the host.  Returns
    (flops per sample, [seconds per timed sample])."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import zt_oracle as oracle
    c = PREFILL
    B, T, H, Hkv, D = c["batch"], c["T"], c["n_heads"], c["n_kv_heads"], c["head_dim"]
    q = oracle.fill_normal((B, T, H * D), 0, 0)
    k = oracle.fill_normal((B, T, Hkv * D), 0, 1)
    v = oracle.fill_normal((B, T, Hkv * D), 0, 2)
    do = oracle.fill_normal((B, T, H * D), 0, 3)
    times, flops = [], 0.0
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        flops, *_ = oracle.sampled_step(q, k, v, do, H, Hkv, D, row_stride, row_stride - 1, threads=threads)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return flops, times


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = host_threads()
    # about 1/256 of the rows: ~15 GFLOP per sample, a second or so on a few dozen cores
    stride = 256
    flops, times = cpu_sample(threads, stride, args.steps, min(args.warmup, 1))
    sec = sum(times) / len(times)
    value = flops / sec / 1e12
    line = {
        "impl": "reference", "metric": "attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64-accumulate/f32-store",
        "data": "synthetic",
        "config": headline_config(),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"every {stride}th query row of every head of the batch "
                                   f"({flops / 1e9:.2f} GFLOP per step, exact count), OpenMP over (item, KV head)"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "C restatement of src/attention.zig + autograd.attentionBackward (oracle/zt_oracle.c); the Zig "
                "reference needs Zig 0.16 and cannot be built on this box",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def run_ours(args):
    import ctypes
    import numpy as np
    import torch
    import torch.distributed as dist

    rank, world, local = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cpu_binding = bind_near_gpu(local, world)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    zt = importlib.import_module("z-transformer_b200")
    L = zt.lib.load()
    peaks, peak_kind = load_peaks()
    traffic = load_traffic()
    tf32_sust, tf32_burst = peaks["bf16_tflops_sustained"] / 2.0, peaks["bf16_tflops"] / 2.0

    c = dict(PREFILL)
    if args.small:  # profiling case: same kernels and tile walk, a quarter of the batch
        c["batch"] = 2
    B, T, H, Hkv, D = c["batch"], c["T"], c["n_heads"], c["n_kv_heads"], c["head_dim"]
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    main_stream = torch.cuda.current_stream(dev)
    comm_stream = torch.cuda.Stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def prefill_run(Bl, Hl, Hkvl, Tl, steps, warmup, gather, sample_clocks=False, push="auto"):
        """`steps` forward+backward passes over this rank's Bl sequences of Hl/Hkvl heads (device-resident inputs).
        gather: None, or "batch" / "heads": every rank ends each step with every rank's out, dq, dk, dv, in one of
        two ways (push):
          "kernel"  out (2/5 of the bytes) is not gathered by a collective: the forward's epilogue stores every row into
                    all ranks' gathered tensors as it stores it locally (peer stores over NVLink,
                    zt_attn_forward_batched_keep_peers); dq + dk + dv go by one NCCL all-gather on a second stream,
                    which also tells a rank that its peers' kernels have finished writing to it.  (The backward that
                    stores dq into peers as well, zt_attn_backward_batched_kept_peers, is the two-kernel form at
                    head_dim 128: a quarter slower than the fused one, which adds dq's shares in memory.)  Costs nothing
                    while the bytes a rank must send fit easily into the time its kernels run;
          "nccl"    plain kernels, then NCCL all-gathers on the second stream beside the next step's kernels: out as
                    soon as the forward has it, dq + dk + dv (one buffer, one collective) after the backward.  Better
                    when the step is NVLink-bound (the transfer takes about as long as the kernels): the peer stores
                    would hold the SMs at the end of every CTA.
          "auto"    times a few steps of the kernels alone and picks "kernel" when the bytes a rank must send, at the
                    measured 770 GB/s per direction, take less than half that time.
        Outputs are double-buffered: a step's kernels never write what an earlier step's gather still reads."""
        q, do = (torch.randn((Bl, Tl, Hl * D), generator=gen, device=dev) for _ in range(2))
        k, v = (torch.randn((Bl, Tl, Hkvl * D), generator=gen, device=dev) for _ in range(2))
        lse, delta = (torch.empty((Bl, Tl, Hl), device=dev) for _ in range(2))
        ws_bytes = L.zt_attn_backward_workspace_bytes(Bl, Tl, Hl, Hkvl, D)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        stream = main_stream.cuda_stream
        token = ctypes.c_ulonglong(0)
        nq, nk = q.numel(), k.numel()

        def plain_set():
            pack = torch.empty(2 * nq + 2 * nk, device=dev)  # out | dq | dk | dv: the gradients are one buffer
            return {"pack": pack, "out": pack[:nq].view_as(q), "dq": pack[nq:2 * nq].view_as(q),
                    "dk": pack[2 * nq:2 * nq + nk].view_as(k), "dv": pack[2 * nq + nk:].view_as(v)}

        def plain_step(o):
            rc = L.zt_attn_forward_batched_keep(q.data_ptr(), k.data_ptr(), v.data_ptr(), o["out"].data_ptr(),
                                                lse.data_ptr(), ws.data_ptr(), ws_bytes, Bl, Tl, Hl, Hkvl, D, stream,
                                                ctypes.byref(token))
            return rc

        def plain_backward(o):
            return L.zt_attn_backward_batched_kept(q.data_ptr(), k.data_ptr(), v.data_ptr(), o["out"].data_ptr(),
                                                   lse.data_ptr(), do.data_ptr(), o["dq"].data_ptr(), o["dk"].data_ptr(),
                                                   o["dv"].data_ptr(), delta.data_ptr(), ws.data_ptr(), ws_bytes, Bl, Tl,
                                                   Hl, Hkvl, D, stream, token.value)

        def timed_steps(fn, n):
            barrier()
            e0.record()
            for i in range(n):
                fn(i)
            e1.record()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1) / n)

        base = plain_set()

        def compute_only(i):
            if plain_step(base) or plain_backward(base):
                raise RuntimeError("libztattn refused the step: " + zt.lib.last_error())

        sent = int((2 * nq + 2 * nk) * 4 * (world - 1)) if gather else 0
        res = {}
        if gather:
            for i in range(max(warmup, 3)):
                compute_only(i)
            res["compute_ms"] = timed_steps(compute_only, max(3, min(steps, 5)))
            res["nvlink_floor_ms"] = sent / 770e9 * 1e3
            if push == "auto":
                push = "kernel" if res["nvlink_floor_ms"] < 0.5 * res["compute_ms"] else "nccl"
            res["push"] = push
        n_sets = 2 if gather else 1
        outs = []
        for s_ in range(n_sets):
            if not gather:
                outs.append(base)
            elif push == "nccl":
                o = plain_set()
                o["out_all"] = torch.empty((world,) + tuple(q.shape), device=dev)
                o["grads_all"] = torch.empty((world, nq + 2 * nk), device=dev)
                outs.append(o)
            else:
                o = {"grads": torch.empty(nq + 2 * nk, device=dev)}
                o["dq"], o["dk"] = o["grads"][:nq].view_as(q), o["grads"][nq:nq + nk].view_as(k)
                o["dv"] = o["grads"][nq + nk:].view_as(v)
                o["g_out"] = zt.sharding.GatheredOutput(q.shape, world, rank, dev)
                o["out"] = o["g_out"].local
                o["out_peers"] = o["g_out"].peer_pointers()
                o["grads_all"] = torch.empty((world, nq + 2 * nk), device=dev)
                outs.append(o)
        comm_done = [torch.cuda.Event() for _ in range(n_sets)]
        ev_grad, ev_out = torch.cuda.Event(), torch.cuda.Event()

        def side_by_side(o):
            """[G, 1, T, Hs D] -> [1, T, H D]: the ranks' column slices laid side by side (KV-head sharding)."""
            gts = (o["out_all"] if push == "nccl" else o["g_out"].gathered,
                   o["grads_all"][:, :nq].reshape((world,) + tuple(q.shape)),
                   o["grads_all"][:, nq:nq + nk].reshape((world,) + tuple(k.shape)),
                   o["grads_all"][:, nq + nk:].reshape((world,) + tuple(v.shape)))
            for gt in gts:
                gt.movedim(0, -2).reshape(*gt.shape[1:-1], world * gt.shape[-1]).contiguous()

        def step(i):
            o = outs[i % n_sets]
            if gather and i >= n_sets:
                main_stream.wait_event(comm_done[i % n_sets])
            # the training pair: the forward leaves its f16 planes of q, k, v in the backward's workspace
            if gather and push == "kernel":
                rc = L.zt_attn_forward_batched_keep_peers(q.data_ptr(), k.data_ptr(), v.data_ptr(), o["out"].data_ptr(),
                                                          lse.data_ptr(), ws.data_ptr(), ws_bytes, Bl, Tl, Hl, Hkvl, D,
                                                          stream, ctypes.byref(token), *o["out_peers"])
                rc |= plain_backward(o)
            else:
                rc = plain_step(o)
                if gather:  # "nccl": out leaves while the backward runs
                    ev_out.record(main_stream)
                    with torch.cuda.stream(comm_stream):
                        comm_stream.wait_event(ev_out)
                        dist.all_gather_into_tensor(o["out_all"], o["out"])
                rc |= plain_backward(o)
            if rc != 0:
                raise RuntimeError("libztattn refused the step: " + zt.lib.last_error())
            if gather:
                ev_grad.record(main_stream)
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ev_grad)
                    dist.all_gather_into_tensor(o["grads_all"], o["grads"] if push == "kernel" else o["pack"][nq:])
                    if gather == "heads":
                        side_by_side(o)
                    comm_done[i % n_sets].record(comm_stream)

        def drain():
            if gather:
                for ev in comm_done:
                    main_stream.wait_event(ev)

        for i in range(warmup):
            step(i)
        drain()
        barrier()
        sampler = ClockSampler(local) if (sample_clocks and rank == 0) else None
        if sampler:
            sampler.start()
        zt.lib.profile(True)
        zt.lib.profile_read()
        launches0 = zt.lib.launch_count()
        barrier()
        e0.record()
        for i in range(steps):
            step(i)
        drain()
        e1.record()
        barrier()
        launches = zt.lib.launch_count() - launches0
        kernels = zt.lib.profile_read()
        zt.lib.profile(False)
        clocks = sampler.stop() if sampler else None
        res.update({"ms_per_step": max_over_ranks(e0.elapsed_time(e1) / steps), "kernels": kernels,
                    "launches": int(launches), "clocks": clocks, "bytes_sent_per_rank": sent})
        return res

    # ---- the headline step ------------------------------------------------------------------------------------
    F = fwd_flops(B, T, H, D)   # of the whole job: batch 8 (the replica run does it on every rank)
    strong = world > 1 and B % world == 0 and not args.small
    weak_res = None
    if strong:
        # the job's 8 sequences split over the ranks, outputs gathered; then the replica run for comparison
        main = prefill_run(B // world, H, Hkv, T, args.steps, args.warmup, "batch", sample_clocks=True, push=args.gather)
        weak_res = prefill_run(B, H, Hkv, T, max(3, args.steps // 2), args.warmup, None)
        Bl = B // world
        value = 3.5 * F / (main["ms_per_step"] * 1e-3) / 1e12
    else:
        main = prefill_run(B, H, Hkv, T, args.steps, args.warmup, None, sample_clocks=True)
        Bl = B
        value = world * 3.5 * F / (main["ms_per_step"] * 1e-3) / 1e12
    ms_step, kernels, launches, clocks = main["ms_per_step"], main["kernels"], main["launches"], main["clocks"]
    Fl = fwd_flops(Bl, T, H, D)  # of one rank's launch

    # ---- roofline of the dominant kernel (by summed device time over the timed region) ----------
    # Algorithmic operations credited per launch: forward 2 GEMMs = F; the fused backward kernel S, dP, dV, dK, dQ
    # = 2.5 F.  In the two-kernel form the key-outer kernel (S, dP, dV, dK) = 2 F and the query-outer one dQ = 0.5 F
    # (its recomputed S and dP are overhead, not credited).
    credit = {"attn_fwd_simt": Fl, "attn_fwd_tc": Fl, "attn_fwd_tc16": Fl, "attn_fwd_tc16g": Fl, "attn_fwd_tc16x": Fl,
              "attn_bwd_dkdv_simt": 2.0 * Fl, "attn_bwd_dq_simt": 0.5 * Fl, "attn_bwd_dkdv_tc": 2.0 * Fl,
              "attn_bwd_dq_tc": 0.5 * Fl, "attn_bwd_fused_tc": 2.5 * Fl}
    total_kernel_ms = sum(ms for _, ms in kernels.values()) or 1.0
    klist = []
    for name, (n, ms) in sorted(kernels.items(), key=lambda kv: -kv[1][1]):
        entry = {"kernel": name, "launches": n, "ms_per_launch": ms / n, "share": ms / total_kernel_ms}
        if name in credit:
            entry["tflops"] = credit[name] / (ms / n * 1e-3) / 1e12
            entry["frac_of_tf32_peak"] = entry["tflops"] / tf32_sust
            entry["frac_of_tf32_peak_burst"] = entry["tflops"] / tf32_burst
        klist.append(entry)
    dom = klist[0] if klist else None
    roofline = None
    if dom and "tflops" in dom:
        tr = (traffic or {}).get(dom["kernel"])
        step_tflops = 3.5 * Fl / ((main.get("compute_ms") or ms_step) * 1e-3) / 1e12  # one GPU's kernels
        roofline = {"bound": "tensor", "kernel": dom["kernel"], "achieved": dom["tflops"], "peak": tf32_sust,
                    "unit": "TFLOP/s", "frac": dom["tflops"] / tf32_sust,
                    "traffic": tr["bytes"] * Bl / tr["units"] if tr else None,
                    "traffic_source": (f"profiles/ncu_dram_traffic.json ({tr['source']}), scaled by sequences per launch"
                                       if tr else None),
                    "peak_source": f"{peak_kind}: TF32 dense = bf16_tflops_sustained ({peaks['bf16_tflops_sustained']}) / 2 "
                                   "(no TF32 figure is measured; a TF32 MMA is half the rate of a bf16 one)",
                    "frac_of_burst_peak": dom["tflops"] / tf32_burst,
                    "burst_peak": tf32_burst,
                    "step_frac": step_tflops / tf32_sust, "step_frac_of_burst_peak": step_tflops / tf32_burst}

    # MMA work issued per step by the f16-split kernels: every credited product is three kind::f16 MMAs.  Forward 2
    # products of 0.5 F each; the fused backward 5 (the two-kernel form 4 + 3: its dQ kernel recomputes S and dP).
    issued = None
    n_products = None
    if {"attn_fwd_tc16", "attn_fwd_tc16g"} & set(kernels):
        if "attn_bwd_fused_tc" in kernels:
            n_products = 2 + 5
        elif {"attn_bwd_dkdv_tc", "attn_bwd_dq_tc"} <= set(kernels):
            n_products = 2 + 4 + 3
    if n_products:
        issued_flop = 3.0 * n_products * 0.5 * Fl
        t_s = (main.get("compute_ms") or ms_step) * 1e-3
        issued = {"flop_per_step": issued_flop, "f16_tflops": issued_flop / t_s / 1e12,
                  "of_bf16_sustained_peak": issued_flop / t_s / 1e12 / peaks["bf16_tflops_sustained"],
                  "credited_over_issued": 3.5 * Fl / issued_flop,
                  "note": "kind::f16 MMA flops issued (3 per credited product; masked halves of diagonal tiles not "
                          "counted) against the measured bf16 GEMM peak"}

    phases = None
    if strong:
        phases = {"compute_ms": main["compute_ms"], "step_ms": ms_step, "gather": main["push"],
                  "bytes_sent_per_rank": main["bytes_sent_per_rank"], "nvlink_floor_ms": main["nvlink_floor_ms"],
                  "limiter": "NVLink" if main["nvlink_floor_ms"] > 0.8 * main["compute_ms"] else "compute",
                  "note": "compute: the step's kernels alone. step: with every rank receiving every rank's out, dq, dk, dv "
                          "('kernel': out stored by the forward's epilogue into every rank's gathered tensor, dq + dk + dv by one "
                          "NCCL all-gather; 'nccl': NCCL all-gathers on a second stream beside the next kernels). "
                          "nvlink_floor: the bytes a rank must send per step over the measured 770 GB/s per direction"}
    weak = None
    if weak_res:
        weak = {"value": world * 3.5 * F / (weak_res["ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": weak_res["ms_per_step"], "scaling": "weak",
                "note": "every rank runs the whole batch of 8 on its own data, no gather (replicas)"}

    # ---- the same step with rope.forward on q and k fused in (src/model.zig:372-375), on request -------------
    rope = None
    if args.rope and not strong:
        q, do = (torch.randn((B, T, H * D), generator=gen, device=dev) for _ in range(2))
        k, v = (torch.randn((B, T, Hkv * D), generator=gen, device=dev) for _ in range(2))
        rws = zt.RopeWorkspace(B, T, H, Hkv, D, dev)

        def rope_step():
            o, lse_ = zt.attention_forward_rope(q, k, v, H, Hkv, D, pos=0, workspace=rws, want_lse=True)
            zt.attention_backward_rope(q, k, v, o, lse_, do, H, Hkv, D, pos=0, workspace=rws, kept=True)

        for _ in range(max(args.warmup, 3)):
            rope_step()
        barrier()
        zt.lib.profile(True)
        zt.lib.profile_read()
        e0.record()
        for _ in range(args.steps):
            rope_step()
        e1.record()
        barrier()
        rk = zt.lib.profile_read()
        zt.lib.profile(False)
        rope_ms = e0.elapsed_time(e1) / args.steps
        rope = {"ms_per_step": rope_ms, "plain_ms_per_step": ms_step, "extra_ms": rope_ms - ms_step,
                "tflops": world * 3.5 * F / (rope_ms * 1e-3) / 1e12,
                "kernels": {n: {"launches": c_, "ms_per_launch": ms / c_} for n, (c_, ms) in rk.items()},
                "note": "q, k handed over unrotated; rotation inside the pre-pass (forward and backward); R^T as one in-place "
                        "pass each over dq and dk (the fused backward adds dq's shares in memory, so dq is rotated once "
                        "it is complete); credited FLOPs unchanged"}
        del rws, q, k, v, do

    # ---- the attention part of a block: rope -> attention -> wo (src/model.zig:372-396) -------------------------
    # one call (the attention kernel's epilogue leaves ctx as the projection's operand planes) against the two calls
    # one after the other, timed alternately so that clock drift under the power cap falls on both alike
    block = None
    if world == 1 and not args.small and not args.no_extras:
        d_model = H * D
        q, do = (torch.randn((B, T, H * D), generator=gen, device=dev) for _ in range(2))
        k, v = (torch.randn((B, T, Hkv * D), generator=gen, device=dev) for _ in range(2))
        wo = torch.randn((H * D, d_model), generator=gen, device=dev) / float(H * D) ** 0.5
        blk = zt.AttentionBlock(B, T, H, Hkv, D, d_model, device=dev)
        times = {False: [], True: []}
        for f in (False, True):
            for _ in range(3):
                blk.forward(q, k, v, wo, fused=f)
        for rnd in range(6):
            for f in ((False, True) if rnd % 2 == 0 else (True, False)):
                torch.cuda.synchronize(dev)
                e0.record()
                for _ in range(3):
                    blk.forward(q, k, v, wo, fused=f)
                e1.record()
                torch.cuda.synchronize(dev)
                times[f].append(e0.elapsed_time(e1) / 3)
        dwo = torch.zeros_like(wo)
        blk.forward(q, k, v, wo)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(3):
            blk.forward(q, k, v, wo)
            blk.backward(do, dwo)
        e1.record()
        torch.cuda.synchronize(dev)
        step_ms = e0.elapsed_time(e1) / 3
        proj_flops = 2.0 * B * T * (H * D) * d_model
        fused_ms, two_ms = statistics.median(times[True]), statistics.median(times[False])
        block = {"config": f"rope + attention + wo, d_model {d_model}, at the headline shape",
                 "forward_ms_fused": fused_ms, "forward_ms_two_calls": two_ms,
                 "saved_ms": two_ms - fused_ms,
                 "hbm_bytes_not_moved": 3 * B * T * H * D * 4,
                 "forward_backward_ms": step_ms,
                 "forward_backward_tflops": (3.5 * F + 3.0 * proj_flops) / (step_ms * 1e-3) / 1e12,
                 "note": "fused: zt_attn_block_forward; the projection's passes over ctx (4 B read for the maximum, 4 B "
                         "read + 4 B written for the planes, per element) do not run; credited flops: attention 3.5 F "
                         "plus three projection products (forward, inputGrad, weightGrad)"}
        del q, k, v, do, wo, dwo, blk

    # ---- end to end with host buffers (rank-local) ----------------------------------------------------
    # Every sequence's q, k, v, dout go up from pinned host memory and its out, dq, dk, dv come back,
    # inside the timed region.  Two ways:
    #  * `e2e`: zt.AttnPipeline, the library's call for host-resident sequences: copies up, kernels and
    #    copies down of consecutive sequences overlap on three streams (PCIe is full duplex);
    #  * `e2e_sync`: device.Attn's call pattern as the reference's trainer drives it
    #    (src/model.zig:481-514): upload, zt_attn_forward, zt_attn_backward, download, one sequence
    #    after the other on one stream.  The reference ABI's backward is given neither out nor the
    #    log-sum-exp, so it recomputes the forward; the credited work is 3.5 F either way.
    # With N ranks the job's 8 sequences are split: every rank moves and computes its own 8 / N.
    e2e_steps = max(1, min(args.steps, 3))
    e2e_B = 1 if args.small else Bl
    hq, hdo = (torch.randn((e2e_B, T, H * D)).pin_memory() for _ in range(2))
    hk, hv = (torch.randn((e2e_B, T, Hkv * D)).pin_memory() for _ in range(2))
    hout, hdq = (torch.empty((e2e_B, T, H * D)).pin_memory() for _ in range(2))
    hdk, hdv = (torch.empty((e2e_B, T, Hkv * D)).pin_memory() for _ in range(2))
    holder = zt.Attn(T, H, Hkv, D, device=dev)
    pipe = zt.AttnPipeline(T, H, Hkv, D, slots=3, device=dev)

    def e2e_sync_step():
        for b in range(e2e_B):
            holder.q.copy_(hq[b].view(-1), non_blocking=True)
            holder.k.copy_(hk[b].view(-1), non_blocking=True)
            holder.v.copy_(hv[b].view(-1), non_blocking=True)
            holder.dout.copy_(hdo[b].view(-1), non_blocking=True)
            holder.forward(1, 64)
            holder.backward(64)
            hout[b].view(-1).copy_(holder.out, non_blocking=True)
            hdq[b].view(-1).copy_(holder.dq, non_blocking=True)
            hdk[b].view(-1).copy_(holder.dk, non_blocking=True)
            hdv[b].view(-1).copy_(holder.dv, non_blocking=True)

    def e2e_step():
        pipe.step(hq, hk, hv, hdo, hout, hdq, hdk, hdv)

    def timed(fn, reps=e2e_steps):
        fn()
        barrier()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / reps)

    e2e_sync_ms = timed(e2e_sync_step)
    e2e_ms = timed(e2e_step)
    job_share = world * e2e_B / B  # batch-8 jobs' worth of flops that one e2e step does, all ranks together
    e2e_value = job_share * 3.5 * F / (e2e_ms * 1e-3) / 1e12
    e2e_sync_value = job_share * 3.5 * F / (e2e_sync_ms * 1e-3) / 1e12
    h2d = (2 * hq[0].numel() + 2 * hk[0].numel()) * 4 * e2e_B
    d2h = h2d
    # What the host's copy engines give this rank, measured beside the figure they bound: one direction at a
    # time and both at once (PCIe is full duplex), 256 MiB pinned buffers, all ranks copying together.
    n_copy = hq[0].numel() if hq[0].numel() * 4 <= (256 << 20) else (256 << 20) // 4
    src_h, dst_h = hq.view(-1)[:n_copy], hout.view(-1)[:n_copy]
    dbuf_up, dbuf_dn = torch.empty(n_copy, device=dev), torch.randn(n_copy, device=dev)
    up = lambda: dbuf_up.copy_(src_h, non_blocking=True)

    def down():
        with torch.cuda.stream(comm_stream):
            dst_h.copy_(dbuf_dn, non_blocking=True)

    def both():
        up()
        down()

    def timed_copy(fn):
        ms = timed(lambda: (fn(), comm_stream.synchronize()), 5)
        return n_copy * 4 / (ms * 1e-3) / 1e9
    h2d_gbs, d2h_gbs, duplex_gbs = timed_copy(up), timed_copy(down), timed_copy(both)
    copy_bound_ms = max(h2d, d2h) / (duplex_gbs * 1e9) * 1e3
    pcie = {"h2d_gbs": h2d_gbs, "d2h_gbs": d2h_gbs, "each_way_when_both_run_gbs": duplex_gbs,
            "copy_bound_ms_per_step": copy_bound_ms, "e2e_over_copy_bound": copy_bound_ms / e2e_ms,
            "note": "pinned host <-> device cudaMemcpyAsync of 256 MiB per direction, every rank at once, max over "
                    "ranks; the copy bound of a step is its bytes one way over the duplex rate"}
    del pipe
    del hq, hdo, hk, hv, hout, hdq, hdk, hdv, holder, dbuf_up, dbuf_dn

    # ---- decode configuration -------------------------------------------------------------------
    d = dict(DECODE)
    if args.small:
        d["batch"] = 8
    Bd, n_ctx = d["batch"], d["n_ctx"]
    Bd_l = Bd // world if (strong and Bd % world == 0) else Bd  # the job's 64 sequences split over the ranks
    kc = torch.randn((Bd_l, n_ctx, Hkv * D), generator=gen, device=dev)
    vc = torch.randn((Bd_l, n_ctx, Hkv * D), generator=gen, device=dev)
    qd = torch.randn((Bd_l, H * D), generator=gen, device=dev)
    n_keys = torch.full((Bd_l,), n_ctx, dtype=torch.int32, device=dev)
    wsd = zt.DecodeWorkspace(Bd_l, n_ctx, H, Hkv, D, dev)
    outd = torch.empty_like(qd)
    outd_all = torch.empty((world,) + tuple(outd.shape), device=dev) if strong else None
    dsteps = max(args.steps, 10)

    def dstep():
        zt.decode_attention(qd, kc, vc, n_keys, H, Hkv, D, workspace=wsd, out=outd)
        if strong:
            dist.all_gather_into_tensor(outd_all, outd)

    for _ in range(max(args.warmup, 3)):
        dstep()
    barrier()
    zt.lib.profile(True)
    zt.lib.profile_read()
    e0.record()
    for _ in range(dsteps):
        dstep()
    e1.record()
    barrier()
    dk_prof = zt.lib.profile_read()
    zt.lib.profile(False)
    d_ms = max_over_ranks(e0.elapsed_time(e1) / dsteps)
    d_bytes_l = float(Bd_l) * n_ctx * 2 * Hkv * D * 4 + 2.0 * Bd_l * H * D * 4
    d_gbs = world * d_bytes_l / (d_ms * 1e-3) / 1e9
    dn, dms = dk_prof.get("decode_splitk_kernel", (1, d_ms))
    d_kernel_gbs = d_bytes_l / (dms / dn * 1e-3) / 1e9
    dtr = (traffic or {}).get("decode_splitk_kernel")
    decode = {"metric": "decode_attn_hbm_gbs", "value": d_gbs, "unit": "GB/s", "ms_per_step": d_ms,
              "scaling": "strong (the 64 sequences split over the ranks, outputs all-gathered inside the step)" if strong
                         else "weak",
              "config": {"workload": "KV-cache decode attention, batch 64, context 8192 (new token's row included), "
                                     "32/8 heads, head_dim 128, f32", **d, "batch_per_gpu": Bd_l},
              "bytes_per_step": world * d_bytes_l,
              "roofline": {"bound": "hbm", "kernel": "decode_splitk_kernel", "achieved": d_kernel_gbs,
                           "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": d_kernel_gbs / peaks["hbm_gbs"],
                           "traffic": dtr["bytes"] * Bd_l / dtr["units"] if dtr else None,
                           "traffic_source": (f"profiles/ncu_dram_traffic.json ({dtr['source']}), scaled by sequences "
                                              "per launch") if dtr else None,
                           "peak_source": f"{peak_kind}: hbm_gbs"},
              "kernels": {n: {"launches": c_, "ms_per_launch": ms / c_} for n, (c_, ms) in dk_prof.items()}}
    # decode end to end with host buffers: q up, out down; the cache stays resident in HBM
    hqd, houtd = torch.randn((Bd_l, H * D)).pin_memory(), torch.empty((Bd_l, H * D)).pin_memory()
    barrier()
    e0.record()
    for _ in range(dsteps):
        qd.copy_(hqd, non_blocking=True)
        dstep()
        houtd.copy_(outd, non_blocking=True)
    e1.record()
    barrier()
    decode["e2e"] = {"value": world * d_bytes_l / (max_over_ranks(e0.elapsed_time(e1) / dsteps) * 1e-3) / 1e9,
                     "unit": "GB/s", "h2d_bytes_per_step": hqd.numel() * 4, "d2h_bytes_per_step": houtd.numel() * 4}
    del kc, vc

    # ---- the two sharded configurations of the benchmark definition, with their gathers --------------------------
    long_context = ragged = None
    if not args.small and not args.no_extras and Hkv % world == 0 and 256 % world == 0:
        # 32k prefill: the 8 KV heads (and their query heads) split over the ranks; outputs are column slices,
        # all-gathered and laid side by side
        sh = zt.sharding.shard_kv_heads(H, Hkv, world, rank)
        T4 = 32768
        r4 = prefill_run(1, sh.n_heads, sh.n_kv_heads, T4, 3, 3, "heads" if world > 1 else None, push=args.gather)
        F4 = fwd_flops(1, T4, H, D)
        long_context = {"config": "T 32768, batch 1, 32/8 heads, head_dim 128, fwd+bwd; KV heads sharded over the ranks",
                        "ms_per_step": r4["ms_per_step"], "tflops": 3.5 * F4 / (r4["ms_per_step"] * 1e-3) / 1e12,
                        "frac_of_tf32_peak_per_gpu": 3.5 * F4 / (r4["ms_per_step"] * 1e-3) / 1e12 / world / tf32_sust,
                        "scaling": "strong", "kv_heads_per_gpu": sh.n_kv_heads}
        if world > 1:
            long_context.update({"compute_ms": r4["compute_ms"], "gather": r4["push"],
                                 "bytes_sent_per_rank": r4["bytes_sent_per_rank"],
                                 "nvlink_floor_ms": r4["nvlink_floor_ms"]})
        # ragged decode: 256 sequences, lengths uniform in [1, 16384], balanced longest-first over the ranks
        rng = np.random.default_rng(0)
        lengths = rng.integers(1, 16385, size=256)
        assignment, inverse = zt.sharding.balance_sequences(lengths, world)
        mine = lengths[np.array(assignment[rank])].astype(np.int32)
        B5, ctx5 = 256 // world, 16384
        kc5 = torch.empty((B5, ctx5, Hkv * D), device=dev)
        vc5 = torch.empty_like(kc5)
        for i in range(0, B5, 16):
            kc5[i:i + 16].normal_(generator=gen)
            vc5[i:i + 16].normal_(generator=gen)
        q5 = torch.randn((B5, H * D), generator=gen, device=dev)
        nk5 = torch.from_numpy(mine).to(dev)
        ws5 = zt.DecodeWorkspace(B5, ctx5, H, Hkv, D, dev)
        out5 = torch.empty_like(q5)
        all5 = torch.empty((world,) + tuple(out5.shape), device=dev)
        inv5 = torch.as_tensor(inverse, dtype=torch.long, device=dev)

        def step5(with_gather=True):
            zt.decode_attention(q5, kc5, vc5, nk5, H, Hkv, D, workspace=ws5, out=out5)
            if world > 1 and with_gather:
                dist.all_gather_into_tensor(all5, out5)
                all5.view(256, H * D).index_select(0, inv5)  # back into the caller's order

        ms5 = timed(step5, 10)
        ms5_compute = timed(lambda: step5(False), 10)
        bytes5 = float(lengths.sum()) * 2 * Hkv * D * 4 + 2.0 * 256 * H * D * 4
        loads = [int(lengths[np.array(a)].sum()) for a in assignment]
        ragged = {"config": "ragged decode, 256 sequences, context U[1, 16384] (seed 0), 32/8 heads, head_dim 128; "
                            "sequences balanced longest-first over the ranks",
                  "ms_per_step": ms5, "compute_ms": ms5_compute, "gbs": bytes5 / (ms5 * 1e-3) / 1e9,
                  "gbs_per_gpu": bytes5 / (ms5 * 1e-3) / 1e9 / world,
                  "frac_of_hbm_peak_per_gpu": bytes5 / (ms5 * 1e-3) / 1e9 / world / peaks["hbm_gbs"],
                  "bytes_per_step": bytes5, "keys_per_rank_max_over_mean": max(loads) / (sum(loads) / world),
                  "scaling": "strong"}
        del kc5, vc5

    # ---- CPU baseline on rank 0 at N = 1 --------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and not args.small:
        threads = host_threads()
        stride = 128
        flops, times = cpu_sample(threads, stride, 1, 0)
        cpu = {"value": flops / times[0] / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"every {stride}th query row of every head of the batch, fwd+bwd "
                         f"({flops / 1e9:.1f} GFLOP, exact count), one pass, {times[0]:.1f} s"}
        # the reference's own execution model is one thread (src/README.md:59-63): a sixteenth of the sample
        flops1, times1 = cpu_sample(1, stride * 16, 1, 0)
        cpu["single_thread"] = {"value": flops1 / times1[0] / 1e12, "unit": "TFLOP/s",
                                "sample": f"every {stride * 16}th query row ({flops1 / 1e9:.2f} GFLOP), "
                                          f"{times1[0]:.1f} s"}

    if rank == 0:
        cfg = headline_config()
        if args.small:
            cfg["batch"] = B
        line = {
            "metric": "attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": cfg,
            "sharding": (f"the batch of 8 split over {world} ranks ({Bl} per GPU); every rank ends the step with every "
                         f"rank's out, dq, dk, dv (gather: {main['push']})") if strong else
                        ("one GPU" if world == 1 else "replicas"),
            "roofline": roofline, "issued_mma": issued, "phases": phases, "weak": weak, "rope": rope, "block": block,
            "kernels": klist,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "host_cpus": cpu_binding, "pcie": pcie,
                    "api": "zt.AttnPipeline.step: per sequence, pinned host -> device, zt_attn_forward_batched_keep + "
                           "zt_attn_backward_batched_kept, device -> pinned host; three streams, three buffer slots"
                           + (f"; each rank moves and computes its {Bl} of the job's 8 sequences" if strong else "")},
            "e2e_sync": {"value": e2e_sync_value, "unit": "TFLOP/s", "ms_per_step": e2e_sync_ms,
                         "api": "device.Attn pattern: upload, zt_attn_forward, zt_attn_backward, download, one "
                                "sequence after the other on one stream"},
            "gpu_launches": int(launches), "clocks": clocks, "decode": decode, "long_context": long_context,
            "ragged_decode": ragged, "small": bool(args.small),
            "paths": {"prefill": [k_["kernel"] for k_ in klist]},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# every configuration of the benchmark definition, one JSON line each (not the headline contract)
# ------------------------------------------------------------------------------------------------

def run_all_configs(args):
    """Throughput of every configuration on this rank's GPU: the GPT-mini forward, the 16-point
    fwd+bwd sweep, the Llama-3 decode, the 32k prefill (KV heads sharded over the ranks) and the ragged
    decode (sequences sharded over the ranks).  Device-resident inputs, CUDA events, max over ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    zt = importlib.import_module("z-transformer_b200")
    zt.lib.load()
    peaks, peak_kind = load_peaks()
    tf32_peak, hbm_peak = peaks["bf16_tflops_sustained"] / 2.0, peaks["hbm_gbs"]
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 + rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def emit(**kw):
        if rank == 0:
            print(json.dumps({"n_gpus": world, "dtype": "f32", "data": "synthetic", **kw}), flush=True)

    def prefill(tag, B, T, H, Hkv, D, backward, reps):
        q, do = (torch.randn((B, T, H * D), generator=gen, device=dev) for _ in range(2))
        k, v = (torch.randn((B, T, Hkv * D), generator=gen, device=dev) for _ in range(2))
        state = {}

        def fwd():
            state["o"], state["lse"] = zt.attention_forward(q, k, v, H, Hkv, D, want_lse=True)

        ms_f = timed(fwd, reps)
        path_f = zt.lib.last_path()
        F = fwd_flops(B, T, H, D)
        out = {"config": tag, "batch_per_gpu": B, "T": T, "n_heads": H, "n_kv_heads": Hkv, "head_dim": D,
               "fwd_ms": ms_f, "fwd_tflops": F / ms_f / 1e9, "fwd_frac_tf32_peak": F / ms_f / 1e9 / tf32_peak,
               "fwd_path": path_f}
        if backward:
            bws = zt.BackwardWorkspace(B, T, H, Hkv, D, dev)

            def bwd():
                zt.attention_backward(q, k, v, state["o"], state["lse"], do, H, Hkv, D, workspace=bws)
            ms_b = timed(bwd, reps)
            out.update({"bwd_ms": ms_b, "bwd_tflops": 2.5 * F / ms_b / 1e9, "bwd_path": zt.lib.last_path(),
                        "fwd_bwd_tflops": 3.5 * F / (ms_f + ms_b) / 1e9,
                        "fwd_bwd_frac_tf32_peak": 3.5 * F / (ms_f + ms_b) / 1e9 / tf32_peak})
            # The step as a trainer issues it: the forward keeps its operand planes for the backward, and the
            # eight launches are captured once into a CUDA graph (all scratch is the caller's workspace).
            L = zt.lib.load()
            o_, dq_ = torch.empty_like(q), torch.empty_like(q)
            dk_, dv_ = torch.empty_like(k), torch.empty_like(v)
            lse_, delta_ = (torch.empty((B, T, H), device=dev) for _ in range(2))

            def pair(stream):
                import ctypes
                token = ctypes.c_ulonglong(0)
                rc = L.zt_attn_forward_batched_keep(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_.data_ptr(),
                                                    lse_.data_ptr(), bws.buf.data_ptr() if bws.nbytes else None,
                                                    bws.nbytes, B, T, H, Hkv, D, stream, ctypes.byref(token))
                rc |= L.zt_attn_backward_batched_kept(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_.data_ptr(),
                                                      lse_.data_ptr(), do.data_ptr(), dq_.data_ptr(), dk_.data_ptr(),
                                                      dv_.data_ptr(), delta_.data_ptr(),
                                                      bws.buf.data_ptr() if bws.nbytes else None, bws.nbytes, B, T, H,
                                                      Hkv, D, stream, token.value)
                if rc != 0:
                    raise RuntimeError(zt.lib.last_error())

            if out["bwd_path"] == "tcgen05":
                pair(torch.cuda.current_stream(dev).cuda_stream)
                torch.cuda.synchronize(dev)
                graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream(dev)
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side):
                        pair(torch.cuda.current_stream(dev).cuda_stream)
                ms_g = timed(graph.replay, max(reps, 20))
                out.update({"step_graph_ms": ms_g, "step_graph_tflops": 3.5 * F / ms_g / 1e9,
                            "step_graph_frac_tf32_peak": 3.5 * F / ms_g / 1e9 / tf32_peak})
        return out

    # 1. GPT-mini forward (replicated on every rank: it does not shard)
    emit(**prefill("1 gpt-mini fwd", 1, 256, 4, 2, 32, False, 50), scaling="replicas only")
    # 2. the sweep; the batch of 8 is split over the ranks
    Bs = max(1, 8 // world)
    for D in (32, 64, 128, 256):
        for T in (512, 1024, 2048, 4096):
            r = prefill(f"2 sweep D{D} T{T}", Bs, T, 32, 8, D, True, 5 if D < 256 else 2)
            for key in ("fwd_tflops", "bwd_tflops", "fwd_bwd_tflops", "step_graph_tflops"):
                if key in r:
                    r[key + "_job"] = r[key] * world
            emit(**r, scaling="strong (batch 8 split over ranks)")
    # 3. Llama-3 decode, sequences split over the ranks
    def decode(tag, B, n_ctx, nk_host):
        H, Hkv, D = 32, 8, 128
        kc = torch.empty((B, n_ctx, Hkv * D), device=dev)
        vc = torch.empty_like(kc)
        for i in range(0, B, 16):
            kc[i:i + 16].normal_(generator=gen)
            vc[i:i + 16].normal_(generator=gen)
        qd = torch.randn((B, H * D), generator=gen, device=dev)
        nk = torch.from_numpy(nk_host.astype(np.int32)).to(dev)
        ws = zt.DecodeWorkspace(B, n_ctx, H, Hkv, D, dev)
        outd = torch.empty_like(qd)
        ms = timed(lambda: zt.decode_attention(qd, kc, vc, nk, H, Hkv, D, workspace=ws, out=outd), 20)
        local_bytes = float(nk_host.sum()) * 2 * Hkv * D * 4 + 2.0 * B * H * D * 4
        total = torch.tensor([local_bytes], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(total)
        gbs = float(total.item()) / ms / 1e6
        emit(config=tag, batch_per_gpu=B, n_ctx=n_ctx, ms=ms, bytes_per_step_job=float(total.item()), gbs_job=gbs,
             gbs_per_gpu=gbs / world, frac_hbm_peak_per_gpu=gbs / world / hbm_peak, path=zt.lib.last_path(),
             scaling="strong (sequences split over ranks)")
        del kc, vc

    decode("3 llama3 decode B64 ctx8192", 64 // world, 8192, np.full(64 // world, 8192))
    # 4. 32k prefill, KV heads split over the ranks
    sh = zt.sharding.shard_kv_heads(32, 8, world, rank)
    r = prefill("4 prefill T32768 (KV heads sharded)", 1, 32768, sh.n_heads, sh.n_kv_heads, 128, True, 2)
    for key in ("fwd_tflops", "bwd_tflops", "fwd_bwd_tflops", "step_graph_tflops"):
        if key in r:
            r[key + "_job"] = r[key] * world
    emit(**r, scaling="strong (8 KV heads split over ranks)")
    # 5. ragged decode: lengths uniform in [1, 16384], longest-first balanced over the ranks
    rng = np.random.default_rng(0)
    lengths = rng.integers(1, 16385, size=256)
    assignment, _ = zt.sharding.balance_sequences(lengths, world)
    decode("5 ragged decode B256 len U[1,16384]", 256 // world, 16384, lengths[np.array(assignment[rank])])
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--gather", choices=["auto", "kernel", "nccl"], default="auto",
                    help="N > 1: how the sharded outputs reach every rank (see prefill_run); auto picks by the "
                         "ratio of transfer to kernel time")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the 32k prefill and the ragged decode (extra keys `long_context`, `ragged_decode`)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--rope", action="store_true",
                    help="also time the step with the rotary embedding of q and k fused in (extra key `rope`)")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: batch 2 prefill and batch 8 decode (same kernels, a quarter of the work); "
                         "its line is not a benchmark result")
    ap.add_argument("--all-configs", action="store_true",
                    help="run every configuration of the benchmark definition (one JSON line each) instead of "
                         "the headline step")
    args = ap.parse_args()
    if args.all_configs:
        return run_all_configs(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
