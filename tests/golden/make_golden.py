"""Generates ``tests/golden/*.npz`` by running the REFERENCE's own amd64 attention operations (compiled from the
reference tree into ``oracle/_ref`` by ``oracle/build.py``) on the seeded cases of ``tests/cases.py``.

    python tests/golden/make_golden.py

Each fixture stores the outputs of one layer-step (appended row after RoPE, rotated q, attention output) — the
``proj_*`` fixtures those of the stage's producer (rmsnorm output, projected q and K/V rows, before and after the
rotation) — plus a checksum of the seeded inputs, so that a drift in the input generator is caught instead of silently
invalidating the fixture.  Inputs are regenerated from the seed at test time; they are not stored.
"""
from __future__ import annotations

import sys
import zlib
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import build as oracle_build  # noqa: E402
from tests import cases  # noqa: E402


def input_checksum(case: cases.Case) -> int:
    crc = 0
    for a in [*case.cache, case.q, case.kv_new, case.fcr, case.fci, case.pos]:
        crc = zlib.crc32(np.ascontiguousarray(a).tobytes(), crc)
    return crc


def main() -> None:
    oracle_build.build_ref()
    ref = cases.Reference.try_load()
    if ref is None:
        raise SystemExit("the reference library could not be built or loaded here")
    out_dir = Path(__file__).resolve().parent
    for spec in cases.GOLDEN_SPECS:
        case = cases.golden_case(spec)
        res = ref.layer_step(case)
        rows = np.stack([r if r is not None else np.zeros_like(case.kv_new[0]) for r in res.rows])
        np.savez_compressed(out_dir / f"{case.name}.npz", rows=rows, q=res.q, xb=res.xb,
                            input_crc=np.uint32(input_checksum(case)), threads=np.int32(ref.threads()))
        print(f"{case.name}: xb absmax {np.abs(res.xb.astype(np.float32)).max():.4f}")
    oracle = cases.Oracle()
    for spec in cases.GOLDEN_PROJ_SPECS:
        case = cases.golden_proj_case(spec)
        res = ref.pre_attention(case, oracle)
        crc = 0
        for a in [case.x, case.rms_w, case.wq, case.wkv, case.fcr, case.fci, case.pos]:
            crc = zlib.crc32(np.ascontiguousarray(a).tobytes(), crc)
        np.savez_compressed(out_dir / f"{case.name}.npz", xb=res.xb, q=res.q, kv=res.kv, q_rot=res.q_rot, rows=res.rows,
                            input_crc=np.uint32(crc), threads=np.int32(ref.threads()))
        print(f"{case.name}: q absmax {np.abs(res.q.astype(np.float32)).max():.4f}")


if __name__ == "__main__":
    main()
