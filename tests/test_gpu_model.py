"""Drop-in at model level: the reference's own `Llama2` model class on a tiny Llama-2
shape (stories15M: dim 288, 6 layers, 6 heads of 48, vocabulary 32000, 256-token slots, fp32, N(0, 0.02) weights),
batch of 4 prompts of 1-32 random tokens fed one token per pass, then 64 greedy steps — once with the reference's
amd64 backend, once with the attention stage replaced by this library through the C++ adapter and the C ABI.
Logits are compared on every pass, the KV cache at the end.  The binary is built by oracle/build.py where the
reference tree exists and travels in oracle/_ref."""
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

from glinthawk_b200.rope import rope_tables

pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "model_harness"
DIM, HIDDEN, LAYERS, HEADS, VOCAB, SEQ, HS = 288, 768, 6, 6, 32000, 256, 48


def write_model(model_dir: Path, seed: int) -> None:
    """The reference's on-disk format: CONFIG (7 x int32, src/models/llama2/base.hh:244-257), BASEWEIGHTS_FP32
    (embedding, final rmsnorm, RoPE cos, RoPE sin; base.hh:355-373) and LAYER<i>_FP32 (base.hh:477-499)."""
    rng = np.random.default_rng(seed)
    w = lambda *shape: rng.normal(0.0, 0.02, size=shape).astype(np.float32)  # noqa: E731
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "CONFIG").write_bytes(struct.pack("=7i", DIM, HIDDEN, LAYERS, HEADS, HEADS, VOCAB, SEQ))
    cos, sin = rope_tables(HS, SEQ)
    with open(model_dir / "BASEWEIGHTS_FP32", "wb") as f:
        for a in (w(VOCAB, DIM), 1.0 + w(DIM), cos, sin):
            f.write(np.ascontiguousarray(a, dtype=np.float32).tobytes())
    for l in range(LAYERS):
        with open(model_dir / f"LAYER{l}_FP32", "wb") as f:
            for a in (1.0 + w(DIM), w(DIM, DIM), w(DIM, 2 * DIM), w(DIM, DIM), 1.0 + w(DIM), w(DIM, HIDDEN),
                      w(DIM, HIDDEN), w(DIM, HIDDEN)):
                f.write(a.tobytes())


def write_prompts(path: Path, seed: int, batch: int = 4):
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, VOCAB, size=int(rng.integers(1, 33))).astype(np.uint32) for _ in range(batch)]
    with open(path, "wb") as f:
        f.write(struct.pack("=I", batch))
        for p in prompts:
            f.write(struct.pack("=I", len(p)))
            f.write(p.tobytes())
    return prompts


def read_run(path: Path, batch: int):
    raw = path.read_bytes()
    steps = struct.unpack_from("=I", raw, 0)[0]
    off = 4
    logits, tokens = [], []
    for _ in range(steps):
        logits.append(np.frombuffer(raw, np.float32, batch * VOCAB, off).reshape(batch, VOCAB))
        off += batch * VOCAB * 4
        tokens.append(np.frombuffer(raw, np.uint32, 2 * batch, off).reshape(batch, 2))
        off += 8 * batch
    caches = []
    for _ in range(batch):
        rows = struct.unpack_from("=I", raw, off)[0]
        off += 4
        n = LAYERS * rows * 2 * DIM
        caches.append(np.frombuffer(raw, np.float32, n, off).reshape(LAYERS, rows, 2 * DIM))
        off += 4 * n
    assert off == len(raw)
    return np.stack(logits), np.stack(tokens), caches


@pytest.mark.skipif(not BIN.exists(), reason="model_harness was not built (needs the reference tree at build time)")
def test_reference_model_with_b200_attention_matches_reference_model(tmp_path):
    write_model(tmp_path / "model", seed=15)
    prompts = write_prompts(tmp_path / "prompts.bin", seed=16)
    runs = {}
    for impl in ("ref", "b200"):
        out = tmp_path / f"{impl}.bin"
        r = subprocess.run([str(BIN), impl, str(tmp_path / "model"), str(tmp_path / "prompts.bin"), "64", str(out)],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        runs[impl] = read_run(out, len(prompts))
    (l_ref, t_ref, c_ref), (l_b, t_b, c_b) = runs["ref"], runs["b200"]
    assert l_ref.shape[0] == max(len(p) for p in prompts) + 63
    assert np.isfinite(l_ref).all() and np.isfinite(l_b).all()
    # logits on every pass; fp32 attention outputs agree to ~1e-6, which the dense layers carry through
    np.testing.assert_allclose(l_b, l_ref, rtol=0, atol=1e-4)
    assert np.array_equal(t_b, t_ref), "greedy tokens and positions must coincide on every pass"
    for a, b in zip(c_ref, c_b):
        assert a.shape == b.shape and a.shape[1] >= 64
        np.testing.assert_allclose(b[:, :, :DIM], a[:, :, :DIM], rtol=1e-3, atol=1e-4)  # rotated K
        np.testing.assert_allclose(b[:, :, DIM:], a[:, :, DIM:], rtol=0, atol=1e-5)     # V through 6 layers
