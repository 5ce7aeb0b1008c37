#!/usr/bin/env python
"""Benchmark of the KV-cache attention stage (fused RoPE + K/V append, fused ragged-batch decode attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A *step* advances every context of the batch by one token through all attention layers of the workload: per layer
one append launch and one decode launch.  The default workload is the Llama2-70B GQA configuration (80 layers,
256 contexts per GPU, lognormal lengths) on paged context slots.  With N > 1 (launched by torch.distributed.run,
one rank per GPU) every rank owns its own contexts — a context's KV lives on exactly one GPU and the attention
path has no collective — so the job is N x 256 contexts (weak scaling).

Printed (rank 0, one JSON line):
  value     whole-job tokens/s with q / new K,V rows already resident in HBM (CUDA events, max over ranks)
  e2e       the same through the host-buffer entry point of the C ABI: pinned host q and K/V rows are copied in and
            xb is copied out every layer, inside the timed region
  roofline  achieved HBM GB/s of the decode kernel = algorithmic bytes per launch / mean launch time, against the
            measured copy bandwidth of this GPU pool
  cpu_baseline  the reference's own amd64/OpenMP operations (or the C restatement when that library is absent)
            timed on this host's cores on a bounded sample of the same workload

`--impl reference` times only that CPU path, as a separate run with the same metric and configuration.
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

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode-attn tokens/s (fused append + decode attention, all layers)"
ELEM = {"f16": 2, "bf16": 2, "f32": 4}
DT_CODE = {"f16": 0, "f32": 1, "bf16": 2}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama2_70b_gqa")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the workload's)")
    ap.add_argument("--batch", type=int, default=0, help="override contexts per GPU (0 = the workload's)")
    ap.add_argument("--seed", type=int, default=20240)
    ap.add_argument("--e2e-steps", type=int, default=-1, help="end-to-end steps (-1 = min(steps, 5), 0 = skip)")
    ap.add_argument("--cpu-contexts", type=int, default=48, help="contexts in the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--static", action="store_true", help="fully resident slots instead of paged ones")
    ap.add_argument("--decode-chunk", type=int, default=0)
    ap.add_argument("--pipeline-steps", action="store_true",
                    help="create the stage with pipeline_steps = 1: the append launch of layer l+1 may start while the "
                         "decode launch of layer l runs (the layers of a step use separate buffers and rows)")
    ap.add_argument("--overlap-prefill", action="store_true",
                    help="mixed workloads: issue the prompt chunks on a second stream so that they run beside the decode "
                         "launches of the same step instead of after them")
    ap.add_argument("--producer", action="store_true",
                    help="each layer-step also runs the stage's producer on the device (rmsnorm + q/kv projection with "
                         "the RoPE + append epilogue, gh_attn_project_append) instead of taking q and K/V rows as given")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------------------
# clocks

def bind_near_gpu(index: int) -> str:
    """With several ranks on one host, keep each rank's threads (and, by first touch, its pinned host buffers) on the
    CPUs NVML reports as closest to its GPU, so that the host<->device copies of the end-to-end path do not cross
    sockets.  Changes this process's CPU affinity only; nothing on the GPU."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        pick = near & allowed
        if not pick or pick == allowed:
            return "unchanged (%d cpus)" % len(allowed)
        os.sched_setaffinity(0, pick)
        return "%d of %d cpus, those nearest the GPU" % (len(pick), len(allowed))
    except Exception as e:  # noqa: BLE001
        return "unchanged (%s)" % type(e).__name__


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only) while a region runs."""

    def __init__(self, uuid: str | None):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid) \
                if uuid else pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # noqa: BLE001
            self.nv, self.err = None, str(e)

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "sw_power_cap": 0x4, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append(mhz)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# DRAM traffic of one decode launch relative to its algorithmic bytes, from the ncu capture summarised in
# profiles/decode_mma_kernel_llama2_70b.md (dram__bytes_read.sum + dram__bytes_write.sum = 1.378 GB against 1.361 GB
# algorithmic on this very batch; traffic grows in proportion to the cached tokens).  Other workloads: not captured.
NCU_TRAFFIC_RATIO = {"llama2_70b_gqa": 1.0123}


def measured_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's amd64/OpenMP operations on a bounded sample

def cpu_layer_step_timer(wl, lens_sample, seed):
    """Returns (run_once, kind, cores): run_once() executes one layer-step of the sample on the host cores."""
    from tests import cases

    ref = cases.Reference.try_load()
    dtype = DT_CODE[wl.dtype]
    if wl.dtype == "bf16":  # the amd64 backend has no bf16: time its fp16 path (same bytes per element)
        dtype = DT_CODE["f16"]
    case = cases.make_case("cpu_sample", wl.shape.name, dtype, np.asarray(lens_sample, dtype=np.uint32), seed)
    if ref is not None and wl.shape.name in ref.names:
        runner, kind, cores = ref, "reference", ref.threads()
    else:
        runner, kind, cores = cases.Oracle(), "port", usable_cpus()
    return (lambda: runner.layer_step(case)), kind, cores


def time_cpu_sample(wl, lens, n_ctx, n_layers, seed, reps):
    n_ctx = min(n_ctx, len(lens))
    # an evenly spaced sample of the sorted lengths keeps the sample's mean length close to the workload's
    idx = np.argsort(lens)[np.linspace(0, len(lens) - 1, n_ctx).astype(int)]
    sample = lens[idx]
    run_once, kind, cores = cpu_layer_step_timer(wl, sample, seed)
    run_once()  # warm-up (page faults, thread pool)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        run_once()
        times.append(time.perf_counter() - t0)
    t_layer = min(times)
    tokens_per_s = n_ctx / (t_layer * n_layers)
    row = wl.shape.row_bytes(ELEM[wl.dtype])
    kv_gbs = float((sample + 1).sum() * row + n_ctx * row) / t_layer / 1e9
    return {
        "value": tokens_per_s, "unit": "tokens/s", "cores": cores, "kind": kind,
        "sample": f"{n_ctx} of {len(lens)} contexts (evenly spaced over the sorted lengths), 1 of {n_layers} layers, "
                  f"best of {reps} layer-steps of {t_layer * 1e3:.1f} ms, scaled to {n_layers} layers",
        "kv_gbs": kv_gbs, "ms_per_layer_step": t_layer * 1e3,
    }, times


def usable_cpus() -> int:
    """CPUs this process may run on (a container's cpuset can be much smaller than the machine)."""
    try:
        return len(os.sched_getaffinity(0)) or 1
    except AttributeError:
        return os.cpu_count() or 1


def use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core, so
    the variable is put back before the OpenMP runtime of the reference library starts."""
    os.environ["OMP_NUM_THREADS"] = str(usable_cpus())


def run_reference_arm(args, wl, n_layers, batch):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_threads()
    headroom = args.warmup + args.steps + 8
    lens = wl.lengths(args.seed, headroom)[:batch]
    n_ctx = min(args.cpu_contexts, batch)
    idx = np.argsort(lens)[np.linspace(0, len(lens) - 1, n_ctx).astype(int)]
    sample = lens[idx]
    run_once, kind, cores = cpu_layer_step_timer(wl, sample, args.seed)
    for _ in range(max(args.warmup, 1)):
        run_once()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run_once()
    t_layer = (time.perf_counter() - t0) / args.steps
    value = n_ctx / (t_layer * n_layers)
    sample_txt = (f"each step = one layer-step of {n_ctx} of {batch} contexts (evenly spaced over the sorted lengths) "
                  f"on the host cores, {t_layer * 1e3:.1f} ms; value scaled to {n_layers} layers")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * n_layers * batch / n_ctx * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "description": wl.description, "layers": n_layers, "contexts_per_gpu": batch},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample_txt},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------------------------

def main():
    args = parse_args()
    from glinthawk_b200.workload import WORKLOADS, algorithmic_bytes

    wl = WORKLOADS[args.workload]
    n_layers = args.layers or wl.n_layers
    batch = args.batch or wl.batch
    if args.impl == "reference":
        run_reference_arm(args, wl, n_layers, batch)
        return

    import torch
    import torch.distributed as dist

    from glinthawk_b200 import dist_util
    from glinthawk_b200.rope import rope_tables
    from glinthawk_b200.stage import AttentionStage

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention stage has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    host_affinity = bind_near_gpu(local_rank) if world > 1 else "unchanged (single rank)"
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    sh, elem = wl.shape, ELEM[wl.dtype]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[wl.dtype]
    W, K = args.warmup, args.steps
    E = min(K, 5) if args.e2e_steps < 0 else args.e2e_steps
    if wl.prefill_contexts:
        E = 0  # the host-buffer entry point covers decode steps only
    headroom = W + K + E + 2
    lens0 = dist_util.weak_scaling_lengths(wl, args.seed, rank, headroom, batch)  # every rank draws its own contexts

    # ---- set-up (untimed): slots, cached KV, inputs ----
    t_setup = time.perf_counter()
    n_pf, t_pf = wl.prefill_contexts, wl.prefill_tokens
    stage = AttentionStage(sh, tdt, n_layers_hosted=n_layers, max_batch=max(batch, n_pf), max_contexts=batch + n_pf,
                           paged=not args.static, device=local_rank, decode_chunk=args.decode_chunk,
                           pipeline_steps=args.pipeline_steps)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    stage.set_rope_tables(torch.from_numpy(cos).to(dev).to(tdt), torch.from_numpy(sin).to(dev).to(tdt))
    slots = stage.get_contexts(np.arange(1, batch + 1, dtype=np.uint32))
    row_elems = 2 * sh.kv_dim
    if n_pf:  # prompt chunks go into slots of their own, rewritten from position 0 every step
        pf_slots = stage.get_contexts(np.arange(batch + 1, batch + n_pf + 1, dtype=np.uint32))
        pf_pos0 = np.full(n_pf, wl.prefill_pos0, dtype=np.uint32)
        if wl.prefill_pos0:  # the part of the prompt that earlier chunks cached
            for i in range(n_pf):
                for l in range(n_layers):
                    stage.prepare(int(pf_slots[i]), l, wl.prefill_pos0 - 1)
                    stage.fill_normal(stage.layer_ptr(int(pf_slots[i]), l), wl.prefill_pos0 * row_elems, tdt, args.seed + 13,
                                      offset=(i * n_layers + l) * sh.seq_len * row_elems)
        pf_q = torch.empty((n_layers, n_pf, t_pf, sh.dim), dtype=tdt, device=dev)
        pf_kv = torch.empty((n_layers, n_pf, t_pf, row_elems), dtype=tdt, device=dev)
        pf_xb = torch.zeros_like(pf_q)
        stage.fill_normal(pf_q, pf_q.numel(), tdt, args.seed + 11)
        stage.fill_normal(pf_kv, pf_kv.numel(), tdt, args.seed + 12)
    for i in range(batch):
        for l in range(n_layers):
            stage.prepare(int(slots[i]), l, int(lens0[i]) + headroom - 1)
            stage.fill_normal(stage.layer_ptr(int(slots[i]), l), int(lens0[i]) * row_elems, tdt, args.seed + 1000 * rank,
                              offset=(i * n_layers + l) * sh.seq_len * row_elems)
    q_all = torch.empty((n_layers, batch, sh.dim), dtype=tdt, device=dev)
    kv_all = torch.empty((n_layers, batch, row_elems), dtype=tdt, device=dev)
    xb_all = torch.zeros((n_layers, batch, sh.dim), dtype=tdt, device=dev)
    stage.fill_normal(q_all, q_all.numel(), tdt, args.seed + 1)
    stage.fill_normal(kv_all, kv_all.numel(), tdt, args.seed + 2)
    torch.cuda.synchronize()
    t_setup = time.perf_counter() - t_setup

    if args.producer:  # residual stream, rmsnorm weights and per-layer projection matrices (random, scaled so q, k, v ~ N(0,1))
        x_all = torch.randn((batch, sh.dim), device=dev).to(tdt)
        rms_w = torch.ones(sh.dim, device=dev, dtype=tdt)
        wq_all = torch.empty((n_layers, sh.dim, sh.dim), dtype=tdt, device=dev)
        wkv_all = torch.empty((n_layers, row_elems, sh.dim), dtype=tdt, device=dev)
        for l in range(n_layers):
            wq_all[l] = (torch.randn((sh.dim, sh.dim), device=dev) / sh.dim ** 0.5).to(tdt)
            wkv_all[l] = (torch.randn((row_elems, sh.dim), device=dev) / sh.dim ** 0.5).to(tdt)
        E = 0  # the host-buffer entry point takes q and K/V rows, not the residual stream
    torch.cuda.synchronize()
    pos = lens0.astype(np.uint32).copy()  # position of the token appended next = tokens cached so far
    stream = torch.cuda.current_stream()

    import ctypes as C

    from glinthawk_b200._lib import lib as ghlib

    # raw pointers per layer, computed once: the per-layer host work inside the timed loop is one C call
    esz = q_all.element_size()
    q_ptr = [C.c_void_p(q_all.data_ptr() + l * batch * sh.dim * esz) for l in range(n_layers)]
    kv_ptr = [C.c_void_p(kv_all.data_ptr() + l * batch * row_elems * esz) for l in range(n_layers)]
    xb_ptr = [C.c_void_p(xb_all.data_ptr() + l * batch * sh.dim * esz) for l in range(n_layers)]
    st_ptr = C.c_void_p(stream.cuda_stream)
    handle = stage._h

    producer_events, prefill_events = [], []
    pf_stream = torch.cuda.Stream(device=dev) if (n_pf and args.overlap_prefill) else None

    def issue_chunk(l, record):
        ps = pf_stream if pf_stream is not None else stream
        if record is not None:
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(ps)
        stage.prefill_chunk(l, pf_slots, pf_pos0, t_pf, pf_q[l], pf_kv[l], pf_xb[l], stream=ps)
        if record is not None:
            f1.record(ps)
            prefill_events.append((f0, f1))

    def device_step(record=None):
        """One token for every context through all layers.  With `record`, every 8th layer's decode launch is
        bracketed by events (the append and decode launches of the other layers stay back to back, which is what
        lets the decode kernel's prologue overlap the append kernel)."""
        stage.batch_begin(slots, pos)
        if pf_stream is not None:  # the chunks of this step may start once the previous step has been issued ...
            fork = torch.cuda.Event()
            fork.record(stream)
            pf_stream.wait_event(fork)
        for l in range(n_layers):
            if pf_stream is not None:
                issue_chunk(l, record)
            if args.producer:
                timed = record is not None and l % 8 == min(3, n_layers - 1)
                if timed:
                    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    p0.record(stream)
                stage.project_append(l, x_all, rms_w, wq_all[l], wkv_all[l], q_all[l])
                if timed:
                    p1.record(stream)
                    producer_events.append((p0, p1))
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                stage.decode(l, q_all[l], xb_all[l])
                if timed:
                    e1.record(stream)
                    record.append((e0, e1))
            elif record is not None and l % 8 == min(3, n_layers - 1):
                stage.append(l, q_all[l], kv_all[l])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                stage.decode(l, q_all[l], xb_all[l])
                e1.record(stream)
                record.append((e0, e1))
            elif ghlib.gh_attn_step(handle, l, q_ptr[l], kv_ptr[l], xb_ptr[l], st_ptr) != 0:
                raise RuntimeError(ghlib.gh_attn_last_error(handle).decode())
            if n_pf and pf_stream is None:
                issue_chunk(l, record)
        if pf_stream is not None:  # ... and the step is over when both streams are
            join = torch.cuda.Event()
            join.record(pf_stream)
            stream.wait_event(join)
        pos[:] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(W, 3)):
        device_step()
    barrier()

    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:  # noqa: BLE001
        pass
    launches0 = stage.stats().kernel_launches
    producer_events.clear()
    prefill_events.clear()
    decode_events, kv_tokens = [], []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(uuid) as clocks:
        ev0.record(stream)
        for _ in range(K):
            kv_tokens.append(int((pos.astype(np.int64) + 1).sum()))
            device_step(decode_events)
        ev1.record(stream)
        barrier()
    ms = ev0.elapsed_time(ev1)
    launches = stage.stats().kernel_launches - launches0
    ms = dist_util.max_over_ranks(ms, dev)
    ms_per_step = ms / K
    value = (batch + n_pf * t_pf) * world / (ms_per_step / 1e3)  # tokens advanced per second, prompt tokens included

    decode_ms = [a.elapsed_time(b) for a, b in decode_events]
    decode_ms_mean = sum(decode_ms) / len(decode_ms)
    ab = algorithmic_bytes(np.full(1, 0), sh, elem)  # structure only
    mean_tokens = sum(kv_tokens) / len(kv_tokens)
    row = 2 * sh.kv_dim * elem
    decode_bytes = mean_tokens * row + 2 * batch * sh.dim * elem
    step_bytes = n_layers * (mean_tokens * row + batch * row)  # KV read + bytes appended, all layers
    peak, peak_src = measured_peak()
    achieved = decode_bytes / (decode_ms_mean / 1e3) / 1e9
    del ab

    # ---- end to end through the host-buffer entry point (H2D of q and K/V rows, D2H of xb, every layer) ----
    e2e = None
    if E > 0:
        q_h = torch.empty((n_layers, batch, sh.dim), dtype=tdt).pin_memory()
        kv_h = torch.empty((n_layers, batch, row_elems), dtype=tdt).pin_memory()
        xb_h = torch.empty((n_layers, batch, sh.dim), dtype=tdt).pin_memory()
        q_h.copy_(q_all)
        kv_h.copy_(kv_all)
        streams = [torch.cuda.Stream(device=dev) for _ in range(3)]

        def host_step():
            stage.batch_begin(slots, pos, stream=stream)
            ready = torch.cuda.Event()
            ready.record(stream)
            for s in streams:
                s.wait_event(ready)
            for l in range(n_layers):
                stage.forward_attention_host(l, tdt, q_h[l], kv_h[l], xb_h[l], stream=streams[l % len(streams)])
            for s in streams:
                done = torch.cuda.Event()
                done.record(s)
                stream.wait_event(done)
            pos[:] += 1

        host_step()  # warm-up (allocates the staging buffers)
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record(stream)
        for _ in range(E):
            host_step()
        h1.record(stream)
        barrier()
        e2e_ms = h0.elapsed_time(h1)
        e2e_ms = dist_util.max_over_ranks(e2e_ms, dev)
        checksum = float(xb_h[-1].float().abs().mean())
        e2e = {"value": batch * world / (e2e_ms / E / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": n_layers * batch * (sh.dim + row_elems) * elem + batch * 32,
               "d2h_bytes_per_step": n_layers * batch * sh.dim * elem, "steps": E,
               "ms_per_step": e2e_ms / E, "result_mean_abs": checksum}

    stats = stage.stats()
    if stats.device_error:
        raise SystemExit(f"device error flag {stats.device_error}")
    prefill = None
    if n_pf:
        fms = [a.elapsed_time(b) for a, b in prefill_events]
        fms_mean = sum(fms) / len(fms)
        # causal attention of the chunk: every token against the cached prefix and the chunk's tokens up to itself
        keys = n_pf * (t_pf * wl.prefill_pos0 + t_pf * (t_pf + 1) / 2)
        flops = 4.0 * keys * sh.n_heads * sh.head_size
        chunk_bytes = n_pf * t_pf * (2 * row_elems + 2 * sh.dim) * elem  # append: K/V rows and q, read and written
        prefill = {"kernels": "append_ordered_kernel + " + ("decode_mma_kernel in chunk mode"
                                                             if os.environ.get("GLINTHAWK_PREFILL") == "mma"
                                                             else "prefill_umma_kernel (tcgen05)"),
                   "ms_per_chunk_call": fms_mean, "prompt_tokens_per_call": n_pf * t_pf,
                   "causal_attention_tflops": flops / (fms_mean / 1e3) / 1e12, "append_bytes": chunk_bytes}
    producer = None
    if args.producer:
        pms = [a.elapsed_time(b) for a, b in producer_events]
        pms_mean = sum(pms) / len(pms)
        w_bytes = (sh.dim + row_elems) * sh.dim * elem
        flops = 2.0 * batch * (sh.dim + row_elems) * sh.dim
        producer = {"kernels": "rmsnorm_kernel + project_kernel (tcgen05) + project_finish_kernel",
                    "ms_per_layer": pms_mean, "weight_bytes_per_layer": w_bytes,
                    "weights_gbs": w_bytes / (pms_mean / 1e3) / 1e9, "tflops": flops / (pms_mean / 1e3) / 1e12,
                    "weights_frac_of_measured_hbm": w_bytes / (pms_mean / 1e3) / 1e9 / peak}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.producer:  # the CPU sample times the stage alone
        use_all_host_threads()
        cpu, _ = time_cpu_sample(wl, lens0, args.cpu_contexts, n_layers, args.seed, reps=3)

    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": max(W, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.name + ("+producer" if args.producer else ""),
                       "description": wl.description + (
                           "; every layer-step starts from the residual stream: rmsnorm, q and kv projections, RoPE and "
                           "append run fused on the device" if args.producer else ""),
                       "layers": n_layers, "contexts_per_gpu": batch, "slots": "static" if args.static else "paged (2 MiB pages)",
                       "mean_cached_tokens": mean_tokens / batch, "kv_resident_gb": stats.bytes_mapped / 1e9,
                       "l2": "inputs larger than L2: each layer-step streams %.2f GB of KV" % (mean_tokens * row / 1e9),
                       "parallelism": f"contexts sharded by request over {world} GPU(s), no collective",
                       "host_affinity": host_affinity, "pipeline_steps": bool(args.pipeline_steps),
                       "seed": args.seed, "split_chunk_tokens": stats.last_chunk, "work_items": stats.last_items},
            "value_per_gpu": value / world,
            "hbm_gbs_step": step_bytes / (ms_per_step / 1e3) / 1e9,
            "roofline": {"bound": "hbm", "kernel": "decode_mma_kernel" if stats.last_kernel else "decode_generic_kernel",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"of {peak_src}", "frac_of_nominal_8tbs": achieved / 8000.0,
                         "bytes_per_launch": decode_bytes, "ms_per_launch": decode_ms_mean,
                         "traffic": (decode_bytes * NCU_TRAFFIC_RATIO[wl.name]
                                     if wl.name in NCU_TRAFFIC_RATIO and batch == wl.batch and stats.last_kernel else None)},
            "clocks": clocks.summary(),
            "e2e": e2e,
            "gpu_launches": int(launches),
            "cpu_baseline": cpu, "producer": producer, "prefill": prefill,
            "setup_s": t_setup,
        }
        print(json.dumps(out))
    stage.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
