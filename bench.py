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
            xb is copied out every layer, inside the timed region; per-rank times and copy rates alongside
  roofline  achieved HBM GB/s of the decode kernel = algorithmic bytes per launch / mean launch time, against the
            measured copy bandwidth of this GPU pool
  via_ops   the same step issued the way the reference's model code issues it: per layer copy_kv_cache + apply_rope
            and the attention operations with host arrays of row pointers (the C++ adapter's call sequence)
  strong    one FIXED set of 256 requests divided among the N ranks by cached tokens (what the reference's router
            does with a batch): per-rank batches of 256 / N contexts, long contexts cut into several work items
  handoff   (N even) ranks paired as (dense stage, attention stage): q and K/V rows arrive from the peer GPU and xb
            goes back over NCCL point-to-point, every layer
  parity    the CUDA path against the CPU checker on the bench's own configuration, untimed
  cpu_baseline  the reference's own amd64/OpenMP operations (or the C restatement when that library is absent)
            timed on this host's cores on one layer-step of the same workload
  producer, prefill, other_configs   short extra regions (N = 1): the stage's fused producer on this workload, the
            prompt-chunk kernel on the Llama3-8B mixed configuration, and one layer-step each of the Llama2-7B,
            Llama2-13B and Llama3-8B decode configurations

`--impl reference` times only the CPU path, as a separate run with the same metric and configuration.
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
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
    ap.add_argument("--cpu-contexts", type=int, default=0, help="contexts in the CPU baseline sample (0 = all)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the via_ops / strong / handoff / parity / producer / prefill regions (profiling runs)")
    ap.add_argument("--static", action="store_true", help="fully resident slots instead of paged ones")
    ap.add_argument("--decode-chunk", type=int, default=0)
    ap.add_argument("--force-generic", action="store_true", help="CUDA-core decode kernel instead of TMA + tensor cores")
    ap.add_argument("--strong-share", default="",
                    help="R/N on one GPU: run rank R's share of the fixed request set divided N ways (what one GPU of "
                         "an N-GPU strong-scaling run sees)")
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
# host placement and clocks

def _cpulist(text: str) -> set[int]:
    out: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.update(range(int(lo), int(hi or lo) + 1))
    return out


def bind_near_gpu(index: int) -> dict:
    """With several ranks on one host, keep each rank's threads on the CPUs of the NUMA node its GPU hangs off and ask
    the kernel to place this process's memory there (pinned host buffers are allocated on the node of the calling
    thread's policy), so that the host<->device copies of the end-to-end path do not cross sockets.  Changes this
    process's CPU affinity and memory policy only; nothing on the GPU.  Returns what was found and done."""
    info: dict = {"gpu_numa_node": None, "cpus_allowed": None, "cpus_bound": None, "mem_policy": "default"}
    try:
        import torch
        p = torch.cuda.get_device_properties(index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        dev = Path("/sys/bus/pci/devices") / bdf
        node = int((dev / "numa_node").read_text())
        info["gpu_numa_node"] = node
        allowed = os.sched_getaffinity(0)
        info["cpus_allowed"] = len(allowed)
        status = Path("/proc/self/status").read_text()
        for line in status.splitlines():
            if line.startswith("Mems_allowed_list"):
                info["mems_allowed"] = line.split(":", 1)[1].strip()
        if node < 0:
            return info
        near = _cpulist((Path("/sys/devices/system/node") / f"node{node}" / "cpulist").read_text()) & allowed
        if near and near != allowed:
            os.sched_setaffinity(0, near)
        info["cpus_bound"] = len(near)
        # set_mempolicy(MPOL_PREFERRED, {node}): allocate on the GPU's node where it has room (x86-64 syscall 238)
        libc = C.CDLL(None, use_errno=True)
        mask = (C.c_ulong * 16)()
        mask[node // 64] = 1 << (node % 64)
        rc = libc.syscall(238, 1, mask, C.c_ulong(16 * 64))
        info["mem_policy"] = f"preferred node {node}" if rc == 0 else f"default (set_mempolicy: errno {C.get_errno()})"
    except Exception as e:  # noqa: BLE001
        info["error"] = type(e).__name__
    return info


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


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, bf16 TFLOP/s burst, where they come from)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return 6650.0, 1590.0, "fallback"


def ncu_traffic_ratio(workload: str, batch: int) -> float | None:
    """DRAM traffic of one decode launch relative to its algorithmic bytes, from the ncu capture recorded beside the
    kernel's profile summary.  The record names the kernel source it was captured from (a hash); when the kernel has
    changed since, there is no figure."""
    rec = ROOT / "profiles" / "decode_mma_kernel_llama2_70b.traffic.txt"
    try:
        kv = dict(line.split("=", 1) for line in rec.read_text().splitlines() if "=" in line and not line.startswith("#"))
        kv = {k.strip(): v.strip() for k, v in kv.items()}
        src = ROOT / "glinthawk_b200" / "csrc" / "decode_mma.cu"
        if kv["workload"] != workload or int(kv["batch"]) != batch:
            return None
        if hashlib.sha256(src.read_bytes()).hexdigest() != kv["kernel_source_sha256"]:
            return None
        return float(kv["dram_traffic_over_algorithmic_bytes"])
    except Exception:  # noqa: BLE001
        return None


EXTRA_STEPS = 3  # timed steps of each of the short regions behind the main one


def plan_steps(args, wl) -> tuple[int, int, int, int]:
    """(warm-up steps, timed steps, end-to-end steps, free positions every context keeps): both arms derive the
    contexts' lengths from the same figures."""
    W, K = max(args.warmup, 3), args.steps
    E = min(K, 5) if args.e2e_steps < 0 else args.e2e_steps
    if wl.prefill_contexts or args.producer:
        E = 0  # the host-buffer entry point covers decode steps from given q and K/V rows only
    return W, K, E, W + K + E + 4 + 4 * (EXTRA_STEPS + 2)


def run_config(wl, n_layers: int, batch: int, world: int, args) -> dict:
    """What the line's `config` names: the same dictionary in both arms."""
    return {"workload": wl.name + ("+producer" if args.producer else ""),
            "description": wl.description + (
                "; every layer-step starts from the residual stream: rmsnorm, q and kv projections, RoPE and "
                "append run fused on the device" if args.producer else ""),
            "layers": n_layers, "contexts_per_gpu": batch, "seed": args.seed,
            "slots": "static" if args.static else "paged (2 MiB pages)",
            "l2": "inputs larger than L2: every layer-step streams the whole batch's K and V of that layer from HBM",
            "parallelism": f"contexts sharded by request over {world} GPU(s), no collective"}


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's amd64/OpenMP operations

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


def cpu_sample_case(wl, lens, n_ctx: int, seed: int):
    """The CPU arm's inputs: n_ctx of the workload's contexts (evenly spaced over the sorted lengths, so that the
    sample's mean length stays the workload's; all of them when n_ctx covers the batch), one layer."""
    from tests import cases

    n_ctx = min(n_ctx or len(lens), len(lens))
    idx = np.arange(len(lens)) if n_ctx == len(lens) else np.argsort(lens)[np.linspace(0, len(lens) - 1, n_ctx).astype(int)]
    dtype = DT_CODE["f16"] if wl.dtype == "bf16" else DT_CODE[wl.dtype]  # amd64 has no bf16: its fp16 path, same bytes
    return cases.make_case("cpu_sample", wl.shape.name, dtype, np.asarray(lens[idx], dtype=np.uint32), seed), idx


def cpu_runner(wl, case):
    """(run_once, checker, kind, flavour, cores): run_once() executes one layer-step of `case` on the host cores and
    nothing else (buffers are set up here).  The reference library exists in up to three builds (the reference's own
    -march=native, x86-64-v4, x86-64-v3); each one this CPU can run is tried on a small slice of the case and the
    fastest is used, so that the baseline is the best the reference's code does on this host."""
    from oracle import build as oracle_build
    from tests import cases

    best = None
    any_build = cases.Reference.try_load()
    if any_build is not None and wl.shape.name in any_build.names:
        n_try = min(case.B, 16)
        small = cases.Case(case.name, case.shape, case.dtype, case.pos[:n_try], case.active[:n_try], case.cache[:n_try],
                           case.q[:n_try], case.kv_new[:n_try], case.fcr, case.fci, case.seed)
        tried = {}
        for flavour in oracle_build.runnable_flavours():
            ref = cases.Reference.try_load(flavour)
            run_small = ref.timed_layer_step(small)
            run_small()
            t0 = time.perf_counter()
            run_small()
            tried[flavour] = time.perf_counter() - t0
            if best is None or tried[flavour] < tried[best[1]]:
                best = (ref, flavour)
        if best is not None:
            ref, flavour = best
            label = flavour + " (fastest of " + ", ".join(f"{k}: {v * 1e3:.0f} ms" for k, v in tried.items()) + \
                f" on {n_try} contexts)"
            return ref.timed_layer_step(case), ref, "reference", label, ref.threads()
    oracle = cases.Oracle()
    return oracle.timed_layer_step(case), oracle, "port", "c restatement", usable_cpus()


def time_cpu_sample(wl, case, n_total: int, n_layers: int, reps: int):
    run_once, _, kind, flavour, cores = cpu_runner(wl, case)
    run_once()  # warm-up (page faults, thread pool)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        run_once()
        times.append(time.perf_counter() - t0)
    t_layer = min(times)
    n_ctx = case.B
    row = wl.shape.row_bytes(ELEM[wl.dtype])
    kv_gbs = float((case.pos.astype(np.int64) + 1).sum() * row + n_ctx * row) / t_layer / 1e9
    return {
        "value": n_ctx / (t_layer * n_layers), "unit": "tokens/s", "cores": cores, "kind": kind, "flavour": flavour,
        "sample": f"one layer-step of {n_ctx} of {n_total} contexts, 1 of {n_layers} layers (layers are independent and "
                  f"cost the same), best of {reps} runs of {t_layer * 1e3:.1f} ms; value = contexts / (that x {n_layers})",
        "kv_gbs": kv_gbs, "ms_per_layer_step": t_layer * 1e3,
    }


def run_reference_arm(args, wl, n_layers, batch):
    """Each step is one layer-step of the workload's whole batch on the host cores, timed as it is; only the number of
    layers is scaled (a token passes through n_layers identical, independent layer-steps)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    use_all_host_threads()
    lens = wl.lengths(args.seed, plan_steps(args, wl)[3])[:batch]
    case, _ = cpu_sample_case(wl, lens, args.cpu_contexts, args.seed)
    run_once, _, kind, flavour, cores = cpu_runner(wl, case)
    for _ in range(max(args.warmup, 1)):
        run_once()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run_once()
    t_layer = (time.perf_counter() - t0) / args.steps
    n_ctx = case.B
    value = n_ctx / (t_layer * n_layers)
    sample_txt = (f"each step = one layer-step of {n_ctx} of {batch} contexts on the host cores ({flavour} build of the "
                  f"reference's amd64/OpenMP operations), {t_layer * 1e3:.1f} ms as timed; value = contexts / (step x "
                  f"{n_layers} layers); one host, whatever --gpus says")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": t_layer * 1e3,
        "ms_per_step_all_layers_scaled": t_layer * n_layers * batch / n_ctx * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": run_config(wl, n_layers, batch, world, args),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "flavour": flavour,
                         "sample": sample_txt},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------------------------------------
# parity of the CUDA path with the CPU checker, on the bench's own configuration (untimed)

def parity_check(stage, wl, case, checker, kind: str, first_id: int) -> dict:
    """Uploads the CPU arm's own inputs into spare slots, runs one layer-step through the fused entry point and
    compares what it leaves behind with the checker's result for the same inputs."""
    import torch

    from tests import cases, gpu_util

    if DT_CODE[wl.dtype] != case.dtype:  # (a bf16 workload must come with the bf16 checker, not the reference's fp16)
        return {"skipped": "case and workload differ in storage type"}
    want = checker.layer_step(case)
    slots = stage.get_contexts(np.arange(first_id, first_id + case.B, dtype=np.uint32))
    for i in range(case.B):
        p = int(case.pos[i])
        stage.prepare(int(slots[i]), 0, p, True)
        if p > 0:
            stage.layer_view(int(slots[i]), 0, p).copy_(gpu_util.to_dev(case.cache[i][:p], case.dtype))
    q, kv = gpu_util.to_dev(case.q, case.dtype), gpu_util.to_dev(case.kv_new, case.dtype)
    xb = torch.zeros_like(q)
    stage.batch_begin(slots, case.pos)
    stage.step(0, q, kv, xb)
    torch.cuda.synchronize()
    kvd = wl.shape.kv_dim
    v_exact, k_ulps, k_rel, q_ulps = True, 0, 0.0, 0
    for i in range(case.B):
        p = int(case.pos[i])
        got = gpu_util.to_host(stage.layer_view(int(slots[i]), 0, p + 1)[p], case.dtype)
        v_exact &= bool(np.array_equal(got[kvd:].view(np.uint8), want.rows[i][kvd:].view(np.uint8)))
        k_ulps = max(k_ulps, int(np.abs(gpu_util._ordered(got[:kvd], case.dtype) - gpu_util._ordered(want.rows[i][:kvd], case.dtype)).max()))
        g32, w32 = cases.as_f32(got[:kvd], case.dtype), cases.as_f32(want.rows[i][:kvd], case.dtype)
        big = np.abs(w32) > 1e-2
        k_rel = max(k_rel, float((np.abs(g32 - w32)[big] / np.abs(w32[big])).max()))
    q_got = gpu_util.to_host(q, case.dtype)
    q_ulps = int(np.abs(gpu_util._ordered(q_got, case.dtype) - gpu_util._ordered(want.q, case.dtype)).max())
    xb_abs = float(np.abs(cases.as_f32(gpu_util.to_host(xb, case.dtype), case.dtype) - cases.as_f32(want.xb, case.dtype)).max())
    tol = cases.TOL_XB[case.dtype]
    for cid in range(first_id, first_id + case.B):
        stage.release_context(cid)
    return {"contexts": case.B, "layer_steps": 1, "against": kind, "v_bit_exact": v_exact, "k_max_ulps": k_ulps,
            "k_max_rel": k_rel, "q_max_ulps": q_ulps, "xb_max_abs": xb_abs, "xb_tolerance": tol,
            "ok": bool(v_exact and k_rel <= 1e-3 and xb_abs <= tol)}


# ------------------------------------------------------------------------------------------------------------

def main():
    args = parse_args()
    from glinthawk_b200.workload import WORKLOADS

    wl = WORKLOADS[args.workload]
    n_layers = args.layers or wl.n_layers
    batch = args.batch or wl.batch
    if args.impl == "reference":
        run_reference_arm(args, wl, n_layers, batch)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention stage has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    placement = bind_near_gpu(local_rank) if world > 1 else {"note": "single rank: left as it is"}
    if world > 1:
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=300))

    env = dict(rank=rank, world=world, local_rank=local_rank, dev=dev, placement=placement)
    extras = not args.no_extras
    out = run_workload(args, wl, n_layers, batch, env, main_line=True, extras=extras)

    # ---- short extra region (one GPU): the prompt-chunk kernel on the Llama3-8B mixed configuration ----
    if extras and world == 1 and not wl.prefill_contexts and not args.producer and args.workload == "llama2_70b_gqa":
        pf_args = argparse.Namespace(**{**vars(args), "steps": 5, "warmup": 3, "e2e_steps": 0, "producer": False,
                                        "strong_share": "", "static": False, "decode_chunk": 0, "force_generic": False,
                                        "pipeline_steps": False, "overlap_prefill": False})
        pf_wl = WORKLOADS["llama3_8b_mixed"]
        try:
            pf = run_workload(pf_args, pf_wl, pf_wl.n_layers, pf_wl.batch, env, main_line=False, extras=False, parity_too=True)
            out["prefill"] = {"workload": pf_wl.name, "ms_per_step": pf["ms_per_step"], "tokens_s": pf["value"],
                              "decode_parity": pf["parity"],
                              "dtype": pf_wl.dtype + " (checked against the C restatement with bf16 storage: the "
                                                     "reference's amd64 backend has no bf16)", **pf["prefill"]}
        except Exception as e:  # noqa: BLE001  (an extra region must not take the main figures down with it)
            out["prefill"] = {"error": f"{type(e).__name__}: {e}"[:400]}
        # ---- and one layer each of the other benchmark configurations (the decode kernel on their shapes) ----
        others = {}
        for name in ("llama2_7b_layer", "llama2_13b", "llama3_8b_decode"):
            o_wl = WORKLOADS[name]
            try:
                o = run_workload(pf_args, o_wl, 1, o_wl.batch, env, main_line=False, extras=False)
            except Exception as e:  # noqa: BLE001
                others[name] = {"error": f"{type(e).__name__}: {e}"[:400]}
                continue
            others[name] = {"contexts": o_wl.batch, "layers_run": 1, "layers_of_the_configuration": o_wl.n_layers,
                            "dtype": o_wl.dtype, "ms_per_layer_step": o["ms_per_step"],
                            "kv_streamed_gb": o["run"]["kv_streamed_per_layer_step_gb"],
                            "decode_kernel": o["roofline"]["kernel"], "decode_gbs": o["roofline"]["achieved"],
                            "decode_frac_of_measured_hbm": o["roofline"]["frac"]}
        out["other_configs"] = others
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_workload(args, wl, n_layers, batch, env, *, main_line: bool, extras: bool, parity_too: bool = False) -> dict:
    import torch
    import torch.distributed as dist

    from glinthawk_b200 import dist_util
    from glinthawk_b200._lib import lib as ghlib
    from glinthawk_b200.rope import rope_tables
    from glinthawk_b200.stage import AttentionStage
    rank, world, local_rank, dev = env["rank"], env["world"], env["local_rank"], env["dev"]
    sh, elem = wl.shape, ELEM[wl.dtype]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[wl.dtype]
    W, K, E, headroom = plan_steps(args, wl)
    n_pf, t_pf = wl.prefill_contexts, wl.prefill_tokens
    plain = not n_pf and not args.producer
    do_via_ops = extras and plain
    do_strong = plain and (bool(args.strong_share) or (extras and world > 1))
    do_handoff = extras and plain and world > 1 and world % 2 == 0
    do_parity = ((extras and plain) or parity_too) and rank == 0
    do_producer_extra = extras and plain and world == 1 and wl.dtype != "f32"
    extra_steps = EXTRA_STEPS
    lens_global = wl.lengths(args.seed, headroom)[:batch]
    lens0 = dist_util.weak_scaling_lengths(wl, args.seed, rank, headroom, batch)  # every rank draws its own contexts

    # ---- set-up (untimed): slots, cached KV, inputs ----
    t_setup = time.perf_counter()
    n_cpu = min(args.cpu_contexts or batch, batch) if (world == 1 and main_line) else min(48, batch)
    stage = AttentionStage(sh, tdt, n_layers_hosted=n_layers, max_batch=max(batch, n_pf), device=local_rank,
                           max_contexts=batch + n_pf + (n_cpu if do_parity else 0), paged=not args.static,
                           decode_chunk=args.decode_chunk, pipeline_steps=args.pipeline_steps,
                           force_generic=args.force_generic)
    cos, sin = rope_tables(sh.head_size, sh.seq_len, sh.rope_theta)
    cos_d, sin_d = torch.from_numpy(cos).to(dev).to(tdt), torch.from_numpy(sin).to(dev).to(tdt)
    stage.set_rope_tables(cos_d, sin_d)
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

    n_w = n_layers  # distinct weight sets resident for the producer
    if args.producer or do_producer_extra:
        # residual stream, rmsnorm weights and per-layer projection matrices (random, scaled so q, k, v ~ N(0,1)); the
        # short extra region keeps 8 layers' matrices (1.3 GB for Llama2-70B, ten times L2) and cycles through them
        n_w = n_layers if args.producer else min(n_layers, 8)
        x_all = torch.randn((batch, sh.dim), device=dev).to(tdt)
        rms_w = torch.ones(sh.dim, device=dev, dtype=tdt)
        wq_all = torch.empty((n_w, sh.dim, sh.dim), dtype=tdt, device=dev)
        wkv_all = torch.empty((n_w, row_elems, sh.dim), dtype=tdt, device=dev)
        for l in range(n_w):
            wq_all[l] = (torch.randn((sh.dim, sh.dim), device=dev) / sh.dim ** 0.5).to(tdt)
            wkv_all[l] = (torch.randn((row_elems, sh.dim), device=dev) / sh.dim ** 0.5).to(tdt)
    torch.cuda.synchronize()
    pos = lens0.astype(np.uint32).copy()  # position of the token appended next = tokens cached so far
    stream = torch.cuda.current_stream()

    # raw pointers per layer, computed once: the per-layer host work inside the timed loop is one C call
    esz = q_all.element_size()
    q_ptr = [C.c_void_p(q_all.data_ptr() + l * batch * sh.dim * esz) for l in range(n_layers)]
    kv_ptr = [C.c_void_p(kv_all.data_ptr() + l * batch * row_elems * esz) for l in range(n_layers)]
    xb_ptr = [C.c_void_p(xb_all.data_ptr() + l * batch * sh.dim * esz) for l in range(n_layers)]
    st_ptr = C.c_void_p(stream.cuda_stream)
    handle = stage._h

    def ck(rc):
        if rc != 0:
            raise RuntimeError(ghlib.gh_attn_last_error(handle).decode())

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

    def device_step(record=None, producer=False, sel=None):
        """One token for every context through all layers.  With `record`, every 8th layer's decode launch is
        bracketed by events (the append and decode launches of the other layers stay back to back, which is what
        lets the decode kernel's prologue overlap the append kernel).  `sel`: indices of the contexts that take
        part (default all)."""
        if sel is None:
            stage.batch_begin(slots, pos)
        else:
            stage.batch_begin(slots[sel], pos[sel])
        if pf_stream is not None:  # the chunks of this step may start once the previous step has been issued ...
            fork = torch.cuda.Event()
            fork.record(stream)
            pf_stream.wait_event(fork)
        for l in range(n_layers):
            if pf_stream is not None:
                issue_chunk(l, record)
            if producer:
                timed = record is not None and l % 8 == min(3, n_layers - 1)
                if timed:
                    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    p0.record(stream)
                stage.project_append(l, x_all, rms_w, wq_all[l % n_w], wkv_all[l % n_w], q_all[l])
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
            else:
                ck(ghlib.gh_attn_step(handle, l, q_ptr[l], kv_ptr[l], xb_ptr[l], st_ptr))
            if n_pf and pf_stream is None:
                issue_chunk(l, record)
        if pf_stream is not None:  # ... and the step is over when both streams are
            join = torch.cuda.Event()
            join.record(pf_stream)
            stream.wait_event(join)
        if sel is None:
            pos[:] += 1
        else:
            pos[sel] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warm=1):
        """ms per call of fn() over `steps` calls after `warm` untimed ones: CUDA events, barrier on both sides,
        max over ranks."""
        for _ in range(warm):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        barrier()
        mine = a.elapsed_time(b) / steps
        return dist_util.max_over_ranks(mine, dev), mine

    def guarded(fn):
        """A region behind the main one must not take the headline figures down with it.  With one rank a failure
        becomes an {"error": ...} entry; with several ranks an exception cannot be contained (the other ranks would
        wait in the next barrier), so it propagates."""
        if world > 1:
            return fn()
        try:
            return fn()
        except Exception as e:  # noqa: BLE001
            try:
                torch.cuda.synchronize()
            except Exception:  # noqa: BLE001
                pass
            return {"error": f"{type(e).__name__}: {e}"[:400]}

    def gather(value: float) -> list[float]:
        if world == 1:
            return [float(value)]
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        allv = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allv, t)
        return [float(v.item()) for v in allv]

    for _ in range(W):
        device_step(producer=args.producer)
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
            device_step(decode_events, producer=args.producer)
        ev1.record(stream)
        barrier()
    ms = ev0.elapsed_time(ev1)
    launches = stage.stats().kernel_launches - launches0
    main_stats = stage.stats()
    ms = dist_util.max_over_ranks(ms, dev)
    ms_per_step = ms / K
    value = (batch + n_pf * t_pf) * world / (ms_per_step / 1e3)  # tokens advanced per second, prompt tokens included

    decode_ms = [a.elapsed_time(b) for a, b in decode_events]
    decode_ms_mean = sum(decode_ms) / len(decode_ms)
    mean_tokens = sum(kv_tokens) / len(kv_tokens)
    row = 2 * sh.kv_dim * elem
    decode_bytes = mean_tokens * row + 2 * batch * sh.dim * elem
    step_bytes = n_layers * (mean_tokens * row + batch * row)  # KV read + bytes appended, all layers
    peak, bf16_peak, peak_src = measured_peaks()
    achieved = decode_bytes / (decode_ms_mean / 1e3) / 1e9

    prefill = None
    if n_pf:
        fms = [a.elapsed_time(b) for a, b in prefill_events]
        fms_mean = sum(fms) / len(fms)
        # causal attention of the chunk: every token against the cached prefix and the chunk's tokens up to itself
        keys = n_pf * (t_pf * wl.prefill_pos0 + t_pf * (t_pf + 1) / 2)
        flops = 4.0 * keys * sh.n_heads * sh.head_size
        chunk_bytes = n_pf * t_pf * (2 * row_elems + 2 * sh.dim) * elem  # append: K/V rows and q, read and written
        # The chunk calls of a step sit between the decode calls of the same batch: what the interleaved step leaves
        # in xb must be what the same layer-step gives with nothing in between (q is rotated in place, so both runs
        # start from a copy of the same q).
        l_last = n_layers - 1
        q_keep = q_all[l_last].clone()
        device_step()
        torch.cuda.synchronize()
        xb_mixed = xb_all[l_last].clone()
        pos[:] -= 1
        q_all[l_last].copy_(q_keep)
        stage.batch_begin(slots, pos)
        stage.step(l_last, q_all[l_last], kv_all[l_last], xb_all[l_last])
        torch.cuda.synchronize()
        pos[:] += 1
        tflops = flops / (fms_mean / 1e3) / 1e12
        prefill = {"kernels": "append_ordered_kernel + prefill_umma_kernel (tcgen05)",
                   "ms_per_chunk_call": fms_mean, "prompt_tokens_per_call": n_pf * t_pf, "cached_prefix_tokens": wl.prefill_pos0,
                   "causal_attention_tflops": tflops, "frac_of_bf16_peak": tflops / bf16_peak,
                   "bf16_peak_tflops": bf16_peak, "peak_source": f"of {peak_src}", "append_bytes": chunk_bytes,
                   "decode_between_chunks_equals_decode_alone": bool(torch.equal(xb_mixed, xb_all[l_last]))}
    producer = None
    if args.producer:
        producer = producer_summary(producer_events, sh, row_elems, elem, batch, peak)

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

        e2e_ms, e2e_mine = timed(host_step, E)
        h2d = n_layers * batch * (sh.dim + row_elems) * elem
        d2h = n_layers * batch * sh.dim * elem

        # what the host can feed: the same buffers copied with no kernels in between, every rank at the same time
        def copies_in():
            q_all.copy_(q_h, non_blocking=True)
            kv_all.copy_(kv_h, non_blocking=True)

        def copies_out():
            xb_h.copy_(xb_all, non_blocking=True)

        _, in_ms = timed(copies_in, 3)
        _, out_ms = timed(copies_out, 3)
        e2e = {"value": batch * world / (e2e_ms / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d + batch * 32, "d2h_bytes_per_step": d2h, "steps": E, "ms_per_step": e2e_ms,
               "ms_per_step_by_rank": gather(e2e_mine),
               "copy_only_h2d_gbs_by_rank": gather(h2d / (in_ms / 1e3) / 1e9),
               "copy_only_d2h_gbs_by_rank": gather(d2h / (out_ms / 1e3) / 1e9),
               "note": "copy_only_*: the step's host buffers copied with no kernels between them, all ranks at once"}
        stage.fill_normal(q_all, q_all.numel(), tdt, args.seed + 1)  # (copies_in overwrote the device inputs)
        stage.fill_normal(kv_all, kv_all.numel(), tdt, args.seed + 2)
        del q_h, kv_h, xb_h

    # ---- the reference's call sequence: host arrays of row pointers, operation by operation ----
    def region_via_ops():
        row_bytes = row_elems * elem
        base_ptrs = [np.array([stage.layer_ptr(int(s), l) for s in slots], dtype=np.uint64) for l in range(n_layers)]
        cos_p, sin_p = C.c_void_p(cos_d.data_ptr()), C.c_void_p(sin_d.data_ptr())

        def ops_step():
            pos_p = C.c_void_p(pos.ctypes.data)
            off = pos.astype(np.uint64) * np.uint64(row_bytes)
            for l in range(n_layers):
                rows = base_ptrs[l] + off  # what TokenContext::key() returns for every prompt of the batch
                ck(ghlib.gh_op_copy_kv_cache_apply_rope(handle, batch, pos_p, cos_p, sin_p, q_ptr[l],
                                                        C.c_void_p(rows.ctypes.data), kv_ptr[l], st_ptr))
                ck(ghlib.gh_op_attention_fused(handle, q_ptr[l], C.c_void_p(base_ptrs[l].ctypes.data), xb_ptr[l], batch,
                                               pos_p, st_ptr))
            pos[:] += 1

        ops_ms, _ = timed(ops_step, extra_steps)
        return {"ms_per_step": ops_ms, "tokens_s": batch * world / (ops_ms / 1e3), "over_value": ops_ms / ms_per_step,
                   "sequence": "per layer: gh_op_copy_kv_cache_apply_rope (the adapter holds copy_kv_cache back until "
                               "apply_rope names the same rows) + gh_op_attention_fused, host pointer arrays"}

    via_ops = guarded(region_via_ops) if do_via_ops else None

    # ---- strong scaling: ONE set of requests divided among the ranks by cached tokens ----
    def region_strong():
        n_div, r_div = world, rank
        if args.strong_share:
            r_div, n_div = (int(v) for v in args.strong_share.split("/"))
        # this rank holds the same multiset of lengths in its own order: the k-th shortest stands for the k-th shortest
        sel = dist_util.strong_share_on_local_contexts(lens_global, lens0, r_div, n_div)
        strong_events = []
        device_step(sel=sel)
        tokens_mine = int((pos[sel].astype(np.int64) + 1).sum())
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(extra_steps):
            device_step(strong_events, sel=sel)
        b.record(stream)
        barrier()
        s_mine = a.elapsed_time(b) / extra_steps
        s_ms = dist_util.max_over_ranks(s_mine, dev)
        s_stats = stage.stats()
        d_ms = sum(x.elapsed_time(y) for x, y in strong_events) / len(strong_events)
        d_bytes = tokens_mine * row + 2 * len(sel) * sh.dim * elem
        strong = {"contexts_total": batch, "divided_over": n_div, "contexts_this_rank": len(sel),
                  "ms_per_step": s_ms, "ms_per_step_by_rank": gather(s_mine), "tokens_s": batch / (s_ms / 1e3),
                  "efficiency_vs_n1": (ms_per_step / n_div) / s_ms,
                  "cached_tokens_by_rank": gather(float(tokens_mine)),
                  "work_items": s_stats.last_items, "split_chunk_tokens": s_stats.last_chunk,
                  "contexts_cut": s_stats.last_split_contexts,
                  "decode_ms_per_launch": d_ms, "decode_gbs": d_bytes / (d_ms / 1e3) / 1e9,
                  "decode_frac_of_measured_hbm": d_bytes / (d_ms / 1e3) / 1e9 / peak,
                  "note": "rank 0's figures for work items, cuts and the decode launch (the blocks of a cut context "
                          "combine their records inside it); efficiency = (N=1 step time / N) / this step time"}
        if args.strong_share:
            strong["note"] += "; emulated on one GPU: this rank's share only"
        return strong

    strong = guarded(region_strong) if do_strong else None

    # ---- stage hand-off between GPUs: q and K/V rows in, xb out, over NCCL point-to-point ----
    handoff = None
    if do_handoff:
        handoff = handoff_region(stage, env, n_layers, batch, slots, pos, q_all, kv_all, xb_all, extra_steps,
                                 ms_per_step, lambda l: ck(ghlib.gh_attn_step(handle, l, q_ptr[l], kv_ptr[l], xb_ptr[l], st_ptr)))

    # ---- short extra region: the stage's producer in front of every layer-step ----
    def region_producer():
        producer_events.clear()
        rec = []
        device_step(producer=True)
        p_ms, _ = timed(lambda: device_step(rec, producer=True), extra_steps, warm=1)
        res = producer_summary(producer_events, sh, row_elems, elem, batch, peak)
        res["ms_per_step_with_producer"] = p_ms
        res["weights_resident"] = f"{n_w} layers' matrices, cycled ({n_w * (sh.dim + row_elems) * sh.dim * elem / 1e9:.2f} GB)"
        return res

    if do_producer_extra:
        producer = guarded(region_producer)  # (an {"error": ...} entry for shapes the fused projection does not take)

    stats = stage.stats()
    if stats.device_error:
        raise SystemExit(f"device error flag {stats.device_error}")
    stage.synchronize()

    # ---- CPU checker and CPU baseline on this workload's own inputs ----
    parity, cpu = None, None
    if do_parity or (rank == 0 and world == 1 and not args.no_cpu_baseline and plain and main_line):
        use_all_host_threads()
        if wl.dtype == "bf16":  # the reference's amd64 backend has no bf16: the C restatement with bf16 storage checks
            from tests import cases
            sample = np.argsort(lens_global)[np.linspace(0, batch - 1, n_cpu).astype(int)]
            case = cases.make_case("cpu_sample", sh.name, DT_CODE["bf16"], lens_global[sample].astype(np.uint32), args.seed)
            checker, kind = cases.Oracle(), "port"
        else:
            case, _ = cpu_sample_case(wl, lens_global, n_cpu, args.seed)
            if do_parity:
                _, checker, kind, _, _ = cpu_runner(wl, case)
        if do_parity:
            parity = guarded(lambda: parity_check(stage, wl, case, checker, kind, first_id=batch + n_pf + 1))
        if world == 1 and not args.no_cpu_baseline and plain and main_line:
            # (for a bf16 workload the CPU arm times the reference's fp16 path: same bytes per element)
            cpu_case = case if wl.dtype != "bf16" else cpu_sample_case(wl, lens_global, n_cpu, args.seed)[0]
            cpu = guarded(lambda: time_cpu_sample(wl, cpu_case, batch, n_layers, reps=3))

    out = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic",
        "config": run_config(wl, n_layers, batch, world, args),
        "run": {"mean_cached_tokens": mean_tokens / batch, "kv_resident_gb": stats.bytes_mapped / 1e9,
                "kv_streamed_per_layer_step_gb": mean_tokens * row / 1e9, "host_placement": env["placement"],
                "pipeline_steps": bool(args.pipeline_steps), "split_chunk_tokens": main_stats.last_chunk,
                "work_items": main_stats.last_items, "contexts_cut": main_stats.last_split_contexts, "setup_s": t_setup},
        "value_per_gpu": value / world,
        "hbm_gbs_step": step_bytes / (ms_per_step / 1e3) / 1e9,
        "roofline": {"bound": "hbm", "kernel": "decode_mma_kernel" if main_stats.last_kernel else "decode_generic_kernel",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": f"of {peak_src}", "frac_of_nominal_8tbs": achieved / 8000.0,
                     "bytes_per_launch": decode_bytes, "ms_per_launch": decode_ms_mean,
                     "traffic": (lambda r: decode_bytes * r if r is not None and main_stats.last_kernel else None)(
                         ncu_traffic_ratio(wl.name, batch))},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": int(launches),
        "cpu_baseline": cpu, "parity": parity, "via_ops": via_ops, "strong": strong, "handoff": handoff,
        "producer": producer, "prefill": prefill,
    }
    stage.close()
    del q_all, kv_all, xb_all
    torch.cuda.empty_cache()
    return out


def producer_summary(events, sh, row_elems, elem, batch, peak) -> dict:
    pms = [a.elapsed_time(b) for a, b in events]
    pms_mean = sum(pms) / len(pms)
    w_bytes = (sh.dim + row_elems) * sh.dim * elem
    flops = 2.0 * batch * (sh.dim + row_elems) * sh.dim
    return {"kernels": "rmsnorm_kernel + project_kernel (tcgen05) + project_finish_kernel",
            "ms_per_layer": pms_mean, "weight_bytes_per_layer": w_bytes,
            "weights_gbs": w_bytes / (pms_mean / 1e3) / 1e9, "tflops": flops / (pms_mean / 1e3) / 1e12,
            "weights_frac_of_measured_hbm": w_bytes / (pms_mean / 1e3) / 1e9 / peak}


def handoff_region(stage, env, n_layers, batch, slots, pos, q_all, kv_all, xb_all, steps, local_ms_per_step, step_layer):
    """Ranks 2i (dense stage) and 2i+1 (attention stage, owner of the contexts) form a pair.  Per layer the dense rank
    sends q and the new K/V rows and receives xb.  The two directions use communicators of their own, so the inputs
    of later layers arrive while earlier layers compute; NCCL matches the operations of a pair in issue order, and
    both sides issue them layer by layer."""
    import torch
    import torch.distributed as dist

    from glinthawk_b200 import dist_util, handoff

    rank, world, dev = env["rank"], env["world"], env["dev"]
    pairs = [(2 * i, 2 * i + 1) for i in range(world // 2)]
    groups = {}
    for pr in pairs:  # every rank takes part in the creation of every group
        groups[pr] = (dist.new_group(list(pr)), dist.new_group(list(pr)))
    pair = pairs[rank // 2]
    g_in, g_out = groups[pair]
    attention_side = rank % 2 == 1
    peer = pair[0] if attention_side else pair[1]
    link = handoff.LayerLink(peer, g_in, g_out)
    stream = torch.cuda.current_stream()
    xb_rx = torch.zeros_like(xb_all) if not attention_side else None

    def step():
        if attention_side:
            stage.batch_begin(slots, pos)
            handoff.attention_side_step(link, n_layers, q_all, kv_all, xb_all, step_layer)
            pos[:] += 1
        else:
            handoff.dense_side_step(link, n_layers, q_all, kv_all, xb_rx)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    step()  # creates the communicators
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(steps):
        step()
    b.record(stream)
    barrier()
    ms = dist_util.max_over_ranks(a.elapsed_time(b) / steps, dev)
    # what arrived on the dense side against the attention side's own buffer, sent once more after the timed region
    same = torch.ones(1, device=dev)
    if attention_side:
        handoff.wait_all(dist.batch_isend_irecv([dist.P2POp(dist.isend, xb_all, peer, group=g_out)]))
    else:
        again = torch.empty_like(xb_rx)
        handoff.wait_all(dist.batch_isend_irecv([dist.P2POp(dist.irecv, again, peer, group=g_out)]))
        torch.cuda.synchronize()
        same = torch.tensor([1.0 if torch.equal(again, xb_rx) else 0.0], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    per_layer = (batch * q_all.shape[2] * 2 + batch * kv_all.shape[2]) * q_all.element_size()
    return {"pairs": len(pairs), "ms_per_step": ms, "ms_per_layer": ms / n_layers,
            "local_ms_per_layer": local_ms_per_step / n_layers, "over_local": ms / local_ms_per_step,
            "bytes_per_layer": per_layer, "tokens_s": batch * len(pairs) / (ms / 1e3),
            "outputs_identical": bool(same.item() == 1.0),
            "transport": "NCCL send/recv over NVLink, one communicator per direction"}


if __name__ == "__main__":
    main()
