"""The C++ adapter (glinthawk_b200/cpp/glinthawk_b200_ops.hh) driven through the reference's own context view types:
reference-side C++ -> adapter -> C ABI -> CUDA kernels.  The binary is compiled against the reference tree by
oracle/build.py (where that tree exists) and travels in oracle/_ref."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

from tests import cases

pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "adapter_check"


@pytest.mark.skipif(not BIN.exists(), reason="adapter_check was not built (needs the reference tree at build time)")
def test_reference_types_through_adapter(tmp_path, oracle):
    case = cases.make_case("adapter", "mini_g8", cases.F16, [0, 63, 64, 300, 511], seed=77)
    want = oracle.layer_step(case)
    blob = tmp_path / "case.bin"
    with open(blob, "wb") as f:
        f.write(np.uint32(case.B).tobytes())
        f.write(case.pos.astype(np.uint32).tobytes())
        for a in (case.q, case.kv_new, case.fcr, case.fci, *case.cache):
            f.write(np.ascontiguousarray(a).tobytes())
    out = tmp_path / "xb.bin"
    r = subprocess.run([str(BIN), str(blob), str(out)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    xb = np.fromfile(out, dtype=np.float16).reshape(case.B, case.shape.dim)
    np.testing.assert_allclose(xb.astype(np.float32), want.xb.astype(np.float32), rtol=0, atol=cases.TOL_XB[cases.F16])
