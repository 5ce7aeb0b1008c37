"""Host-side pieces of bench.py that need no GPU: both arms describe the same configuration, the step plan is
shared, and the ncu traffic record is only used for the kernel source it was captured from."""
import argparse
import hashlib
from pathlib import Path

import bench
from glinthawk_b200.workload import WORKLOADS


def _args(**kw):
    base = dict(steps=20, warmup=5, e2e_steps=-1, producer=False, static=False, seed=20240, cpu_contexts=0)
    base.update(kw)
    return argparse.Namespace(**base)


def test_both_arms_print_the_same_config_and_lengths():
    wl = WORKLOADS["llama2_70b_gqa"]
    ours = bench.run_config(wl, 80, 256, 8, _args())
    ref = bench.run_config(wl, 80, 256, 8, _args(impl="reference"))
    assert ours == ref and ours["workload"] == "llama2_70b_gqa" and "8 GPU" in ours["parallelism"]
    W, K, E, headroom = bench.plan_steps(_args(), wl)
    assert (W, K, E) == (5, 20, 5) and headroom >= W + K + E + 4 * (bench.EXTRA_STEPS + 2)
    assert bench.plan_steps(_args(warmup=1), wl)[0] == 3, "at least three warm-up steps"
    assert bench.plan_steps(_args(), WORKLOADS["llama3_8b_mixed"])[2] == 0, "no host-buffer region for prompt chunks"
    lens = wl.lengths(20240, headroom)
    assert lens.max() + headroom <= wl.shape.seq_len


def test_traffic_record_belongs_to_the_current_kernel_source():
    rec = Path(bench.ROOT) / "profiles" / "decode_mma_kernel_llama2_70b.traffic.txt"
    kv = dict(line.split("=", 1) for line in rec.read_text().splitlines() if "=" in line and not line.startswith("#"))
    kv = {k.strip(): v.strip() for k, v in kv.items()}
    src = Path(bench.ROOT) / kv["kernel_source"]
    ratio = bench.ncu_traffic_ratio("llama2_70b_gqa", 256)
    if hashlib.sha256(src.read_bytes()).hexdigest() == kv["kernel_source_sha256"]:
        assert ratio is not None and 1.0 <= ratio < 1.1
    else:
        assert ratio is None, "a record of another kernel version must not be used"
    assert bench.ncu_traffic_ratio("llama2_70b_gqa", 32) is None and bench.ncu_traffic_ratio("llama2_7b_layer", 64) is None
