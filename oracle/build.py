"""Build recipe for the parity checkers (TEST INFRASTRUCTURE ONLY).

Two artefacts, neither of which the product path may load:

* ``oracle/libattn_oracle.so`` — the plain-C restatement in ``oracle/attn_oracle.c``.
* ``oracle/_ref/libghref_<flavour>.so`` — the reference project's own amd64/OpenMP attention operations,
  compiled from the reference tree WHERE IT LIES (no source is copied into this repository) through
  ``oracle/ref_harness.cc``.  Only built when the reference tree is present; the built libraries travel
  with the repository snapshot to machines that do not have the tree.

Two things stand between GCC 13 and the reference headers, and both are handled without touching arithmetic:

1. ``glog`` is not installed: ``oracle/shim/glog/logging.h`` supplies the macros the headers use.
2. GCC 13 rejects the out-of-class member definitions in ``src/arch/amd64/llama2/ops.hh`` because their
   template heads omit the class's ``requires ModelConfig<Config>`` clause (GCC 12, which the reference's CI
   pins, accepted them).  A temporary copy of that ONE header with the clause inserted after each such
   template head is written to a scratch directory outside the repository and put first on the include path.

Flavours: ``native`` uses the reference's own flags (``etc/cflags.cmake``: -O3 -march=native -ffast-math
-fsingle-precision-constant, plus OpenMP); ``v4`` and ``v3`` swap -march=native for -march=x86-64-v4 (AVX-512) and
-march=x86-64-v3 (AVX2) so that a library still loads on a host whose CPU lacks the build host's extensions.
``load_ref()`` picks ``native`` only when the running CPU advertises every instruction-set extension the build host
had (flags that do not stand for compiler-generated instructions are not compared), else the widest of the other
two that the CPU can run.

The reference tree is looked for where the environment variable GLINTHAWK_REFERENCE points, else in a directory
named ``reference`` beside the repository; when neither exists nothing is built and prebuilt libraries are used.
"""
from __future__ import annotations

import ctypes
import json
import os
import re
import shutil
import subprocess
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_ROOT = Path(os.environ.get("GLINTHAWK_REFERENCE") or HERE.parent.parent / "reference")
REF_OUT = HERE / "_ref"
ORACLE_SO = HERE / "libattn_oracle.so"

_REF_FLAGS = ["-std=c++20", "-O3", "-DNDEBUG", "-ffast-math", "-fsingle-precision-constant", "-fopenmp",
              "-DTARGET_PLATFORM_AMD64", "-shared", "-fPIC", "-w"]
_TEMPLATE_HEAD = "template<typename Config, typename DType, typename ContextType>"
_MARCH = {"native": "-march=native", "v4": "-march=x86-64-v4", "v3": "-march=x86-64-v3"}
_V4_FLAGS = {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"}
# /proc/cpuinfo flags that stand for instructions a compiler emits on its own under -march=native (vector, bit
# manipulation and conversion extensions).  The rest of the list (rtm, pku, hypervisor and mitigation flags, ...) says
# nothing about whether code built on one host runs on another.
_CODEGEN_FLAGS = {"pni", "ssse3", "sse4_1", "sse4_2", "popcnt", "abm", "movbe", "bmi1", "bmi2", "adx", "avx", "avx2", "fma",
                  "f16c", "avx_vnni", "avx512f", "avx512dq", "avx512cd", "avx512bw", "avx512vl", "avx512ifma",
                  "avx512vbmi", "avx512_vbmi2", "avx512_vnni", "avx512_bitalg", "avx512_vpopcntdq", "avx512_bf16",
                  "avx512_fp16", "gfni", "vaes", "vpclmulqdq", "pclmulqdq", "aes", "sha_ni", "lahf_lm", "cx16",
                  "amx_tile", "amx_int8", "amx_bf16"}


def _cpu_flags() -> list[str]:
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                return sorted(set(line.split(":", 1)[1].split()))
    except OSError:
        pass
    return []


def _newer(target: Path, *sources: Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources)


def build_oracle(force: bool = False) -> Path:
    srcs = [HERE / "attn_oracle.c", HERE / "attn_oracle_impl.inc"]
    if not force and _newer(ORACLE_SO, *srcs):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-Wall", "-Wextra",
           str(srcs[0]), "-o", str(ORACLE_SO), "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


_MODEL_HEAD = "template<typename Config, typename DType, typename LlamaOperations, typename Context>"
_MODEL_CLAUSE = ("requires ModelConfig<Config> && LlamaOperationsConcept<LlamaOperations, DType, ConfigRuntime<Config>>\n"
                 "         && ContextConcept<Context, DType>")


def _mirror(scratch: Path, rel_dir: str, patched: dict[str, str]) -> None:
    """scratch/<rel_dir> = the reference directory with the given files replaced by adjusted copies; every other
    entry is a symlink, because quoted includes are resolved relative to the including file first."""
    src_dir, dst_dir = REF_ROOT / "src" / rel_dir, scratch / rel_dir
    dst_dir.mkdir(parents=True, exist_ok=True)
    for entry in src_dir.iterdir():
        target = dst_dir / entry.name
        if entry.name in patched:
            target.write_text(patched[entry.name])
        elif not target.exists():
            os.symlink(entry, target)


def _patched_include_dir(scratch: Path, with_model: bool = False) -> Path:
    """A scratch include root holding the headers GCC 13 needs adjusted; everything else resolves to the
    reference tree.  The only edit is the insertion of the class's own `requires` clause after the template head
    of out-of-class member definitions (GCC 13: "redeclaration with different constraints")."""
    ops = (REF_ROOT / "src" / "arch" / "amd64" / "llama2" / "ops.hh").read_text()
    ops, n = re.subn(re.escape(_TEMPLATE_HEAD) + r"\n(?!requires)", _TEMPLATE_HEAD + "\nrequires ModelConfig<Config>\n", ops)
    if n < 6:
        raise RuntimeError(f"expected at least 6 out-of-class definitions to adjust in ops.hh, found {n}")
    _mirror(scratch, "arch/amd64/llama2", {"ops.hh": ops})
    os.symlink(REF_ROOT / "src" / "arch" / "amd64" / "common", scratch / "arch" / "amd64" / "common")  # "../common/ops.hh"
    if with_model:
        model = (REF_ROOT / "src" / "models" / "llama2" / "model.hh").read_text()
        # member definitions only: the head is followed by the member template's own head or by `void Llama2<`
        model, n = re.subn(re.escape(_MODEL_HEAD) + r"\n(?=template<StateConcept StateType>|void Llama2<)",
                           _MODEL_HEAD + "\n" + _MODEL_CLAUSE + "\n", model)
        if n < 13:
            raise RuntimeError(f"expected 13 member definitions to adjust in model.hh, found {n}")
        _mirror(scratch, "models/llama2", {"model.hh": model})
        state = (REF_ROOT / "src" / "models" / "common" / "state.hh").read_text()
        head, marker, impl = state.partition("/*** Implementations ***/")
        impl, n = re.subn(r"template<typename Config>\n(?!requires)",
                          "template<typename Config>\nrequires llama2::ModelConfig<Config>\n", impl)
        if not marker or n < 21:
            raise RuntimeError(f"expected 21 member definitions to adjust in state.hh, found {n}")
        _mirror(scratch, "models/common", {"state.hh": head + marker + impl})
        _mirror(scratch, "models", {})  # "../types.hh"
    return scratch


def ref_available() -> bool:
    return (REF_ROOT / "src" / "arch" / "amd64" / "llama2" / "ops.hh").exists()


def build_ref(force: bool = False) -> list[Path]:
    """Compile the reference's amd64 attention operations behind ref_harness.cc (both flavours)."""
    if not ref_available():
        return sorted(REF_OUT.glob("libghref_*.so"))
    REF_OUT.mkdir(exist_ok=True)
    harness = HERE / "ref_harness.cc"
    outs = {f: REF_OUT / f"libghref_{f}.so" for f in _MARCH}
    if not force and all(_newer(o, harness, HERE / "shim" / "glog" / "logging.h") for o in outs.values()):
        return list(outs.values())
    scratch = Path(tempfile.mkdtemp(prefix="ghref_build_"))
    try:
        inc = _patched_include_dir(scratch)
        extra_srcs = [str(REF_ROOT / "src" / "util" / "demangle.cc")]
        for flavour, out in outs.items():
            cmd = ["g++", *_REF_FLAGS, _MARCH[flavour], f"-I{HERE / 'shim'}", f"-I{inc}", f"-I{REF_ROOT / 'src'}",
                   str(harness), *extra_srcs, "-o", str(out)]
            subprocess.run(cmd, check=True)
        (REF_OUT / "BUILD_INFO.json").write_text(json.dumps({
            "compiler": subprocess.run(["g++", "--version"], capture_output=True, text=True).stdout.splitlines()[0],
            "flags": _REF_FLAGS,
            "native_cpu_flags": _cpu_flags(),
            "sources": "reference tree: src/arch/amd64/llama2/ops.hh, src/models/llama2/context.hh (+ includes)",
        }, indent=1))
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return list(outs.values())


def build_adapter_check(force: bool = False) -> Path | None:
    """Compiles oracle/adapter_check.cc — the C++ adapter header instantiated with the reference's own view types
    and concepts — against the reference tree and links it with the attention library.  The binary travels in
    oracle/_ref like the reference libraries; a GPU test runs it."""
    out = REF_OUT / "adapter_check"
    src = HERE / "adapter_check.cc"
    adapter = HERE.parent / "glinthawk_b200" / "cpp" / "glinthawk_b200_ops.hh"
    lib_dir = HERE.parent / "glinthawk_b200"
    if not ref_available() or not (lib_dir / "libglinthawk_attn.so").exists():
        return out if out.exists() else None
    if not force and _newer(out, src, adapter, HERE.parent / "include" / "glinthawk_attn.h"):
        return out
    REF_OUT.mkdir(exist_ok=True)
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    cmd = ["g++", "-std=c++20", "-O1", "-DNDEBUG", "-DTARGET_PLATFORM_AMD64", "-fopenmp", "-w",
           f"-I{HERE / 'shim'}", f"-I{REF_ROOT / 'src'}", f"-I{HERE.parent / 'include'}", f"-I{adapter.parent}",
           f"-I{cuda / 'include'}", str(src), str(REF_ROOT / "src" / "util" / "demangle.cc"), "-o", str(out),
           f"-L{lib_dir}", "-lglinthawk_attn", f"-L{cuda / 'lib64'}", "-lcudart",
           "-Wl,-rpath,$ORIGIN/../../glinthawk_b200", f"-Wl,-rpath,{cuda / 'lib64'}"]
    subprocess.run(cmd, check=True)
    return out


def build_model_harness(force: bool = False) -> Path | None:
    """Compiles oracle/model_harness.cc: the reference's own Llama2 model class, once with its amd64 backend and
    once with the adapter (attention stage on the GPU through the C ABI).  Travels in oracle/_ref."""
    out = REF_OUT / "model_harness"
    src = HERE / "model_harness.cc"
    adapter = HERE.parent / "glinthawk_b200" / "cpp" / "glinthawk_b200_ops.hh"
    lib_dir = HERE.parent / "glinthawk_b200"
    if not ref_available() or not (lib_dir / "libglinthawk_attn.so").exists():
        return out if out.exists() else None
    if not force and _newer(out, src, adapter, HERE.parent / "include" / "glinthawk_attn.h"):
        return out
    REF_OUT.mkdir(exist_ok=True)
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    scratch = Path(tempfile.mkdtemp(prefix="ghref_model_"))
    try:
        inc = _patched_include_dir(scratch, with_model=True)
        ref_src = REF_ROOT / "src"
        units = [ref_src / "util" / n for n in ("demangle.cc", "ring_buffer.cc", "file_descriptor.cc", "digest.cc")]
        units.append(ref_src / "models" / "types.cc")
        cmd = ["g++", "-std=c++20", "-O3", "-DNDEBUG", "-ffast-math", "-fsingle-precision-constant", "-march=x86-64-v3",
               "-fopenmp", "-DTARGET_PLATFORM_AMD64", "-w",
               f"-I{HERE / 'shim'}", f"-I{inc}", f"-I{ref_src}", f"-I{HERE.parent / 'include'}", f"-I{adapter.parent}",
               f"-I{cuda / 'include'}", str(src), *map(str, units), "-o", str(out),
               f"-L{lib_dir}", "-lglinthawk_attn", f"-L{cuda / 'lib64'}", "-lcudart", "-lcrypto", "-lpthread",
               "-Wl,-rpath,$ORIGIN/../../glinthawk_b200", f"-Wl,-rpath,{cuda / 'lib64'}"]
        subprocess.run(cmd, check=True)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return out


def load_oracle() -> ctypes.CDLL:
    return ctypes.CDLL(str(build_oracle()))


def ref_flavour() -> str | None:
    """Which prebuilt reference library this host can run, or None when there is none."""
    native, v4, v3 = (REF_OUT / f"libghref_{f}.so" for f in ("native", "v4", "v3"))
    info = REF_OUT / "BUILD_INFO.json"
    have = set(_cpu_flags())
    if native.exists() and info.exists():
        need = set(json.loads(info.read_text()).get("native_cpu_flags", [])) & _CODEGEN_FLAGS
        if need and need <= have:
            return "native"
    if v4.exists() and _V4_FLAGS <= have:
        return "v4"
    if v3.exists():
        return "v3"
    return None


def runnable_flavours() -> list[str]:
    """Every prebuilt reference library this host's CPU can run, widest instruction set first."""
    have = set(_cpu_flags())
    out = []
    info = REF_OUT / "BUILD_INFO.json"
    if (REF_OUT / "libghref_native.so").exists() and info.exists():
        need = set(json.loads(info.read_text()).get("native_cpu_flags", [])) & _CODEGEN_FLAGS
        if need and need <= have:
            out.append("native")
    if (REF_OUT / "libghref_v4.so").exists() and _V4_FLAGS <= have:
        out.append("v4")
    if (REF_OUT / "libghref_v3.so").exists():
        out.append("v3")
    return out


def load_ref(flavour: str | None = None) -> ctypes.CDLL | None:
    fl = flavour or ref_flavour()
    return ctypes.CDLL(str(REF_OUT / f"libghref_{fl}.so")) if fl else None


if __name__ == "__main__":
    print("oracle:", build_oracle(force=True))
    print("reference:", [str(p) for p in build_ref(force=True)] or "reference tree absent, nothing built")
    print("adapter check:", build_adapter_check(force=True))
    print("model harness:", build_model_harness(force=True))
