"""In-tree build of the native parts (no JIT cache, no site-packages install).

Produces, next to the Python sources so they travel with a snapshot of the tree:

* ``oxidized_neural_orchestra_b200/lib/libono_kernels.so``  – every ``csrc/kernels/*.cu`` and
  ``csrc/engine/*.cu|*.cpp`` compiled for sm_100a (``-gencode arch=compute_100a,code=sm_100a``)
* ``orchestra/_orchestra*.so``  – the pybind11 extension holding the C++ control plane, CPU oracle
  and bindings (``csrc/core``, ``csrc/oracle``, ``csrc/py``)
* ``bin/ono-node``, ``bin/orchestui``, ``bin/ono-orchestrator`` – the native executables

Run ``python -m oxidized_neural_orchestra_b200.build`` (add ``--force`` to rebuild everything).
nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
LIBDIR = ROOT / "oxidized_neural_orchestra_b200" / "lib"
BINDIR = ROOT / "bin"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O3", "-fopenmp-simd", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _newer(src: Path, dst: Path, extra: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *extra] if p.exists())


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")


def _headers(*dirs: Path) -> list[Path]:
    out: list[Path] = []
    for d in dirs:
        out += list(d.glob("*.h")) + list(d.glob("*.hpp")) + list(d.glob("*.cuh"))
    return out


def build_kernels(force: bool = False) -> Path:
    """nvcc every CUDA source for sm_100a and link libono_kernels.so."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "engine").glob("*.cu"))
    hdrs = _headers(CSRC / "kernels", CSRC / "engine")
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.stem + ".cu.o")
        objs.append(o)
        if force or _newer(s, o, hdrs):
            jobs.append([NVCC, *CUDA_FLAGS, "-I", str(CSRC / "kernels"), "-I", str(CSRC / "engine"),
                         "-c", str(s), "-o", str(o)])
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        list(ex.map(_run, jobs))
    lib = LIBDIR / "libono_kernels.so"
    if force or jobs or not lib.exists():
        _run([NVCC, "-shared", "-o", str(lib), *map(str, objs), "-gencode",
              "arch=compute_100a,code=sm_100a"])
    return lib


def build_core(force: bool = False) -> Path | None:
    """g++ the C++ control plane / oracle / bindings into orchestra/_orchestra.so."""
    import pybind11

    srcs = (sorted((CSRC / "core").glob("*.cpp")) + sorted((CSRC / "oracle").glob("*.cpp")) +
            sorted((CSRC / "py").glob("*.cpp")))
    if not srcs:
        return None
    hdrs = _headers(CSRC / "core", CSRC / "oracle", CSRC / "py")
    OBJ.mkdir(parents=True, exist_ok=True)
    inc = ["-I", str(CSRC), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / (s.parent.name + "_" + s.stem + ".o")
        objs.append(o)
        if force or _newer(s, o, hdrs):
            jobs.append([CXX, *CXX_FLAGS, "-fvisibility=hidden", *inc, "-c", str(s), "-o", str(o)])
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        list(ex.map(_run, jobs))
    ext = ROOT / "orchestra" / ("_orchestra" + sysconfig.get_config_var("EXT_SUFFIX"))
    if force or jobs or not ext.exists():
        _run([CXX, "-shared", "-pthread", "-o", str(ext), *map(str, objs)])
    return ext


SANITIZERS = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "thread": ["-fsanitize=thread"]}


def sanitizer_cxx(kind: str) -> str | None:
    """A C++ compiler on this machine that can link the given sanitizer's runtime (None if there is none)."""
    import tempfile

    seen = []
    for cxx in (CXX, shutil.which("g++"), "/usr/bin/g++", shutil.which("clang++")):
        if not cxx or cxx in seen or not Path(cxx).exists() and shutil.which(cxx) is None:
            continue
        seen.append(cxx)
        with tempfile.TemporaryDirectory() as d:
            src = Path(d) / "probe.cpp"
            src.write_text("int main() { return 0; }\n")
            r = subprocess.run([cxx, *SANITIZERS[kind], str(src), "-o", str(Path(d) / "probe")], capture_output=True)
            if r.returncode == 0:
                return cxx
    return None


def build_bins(force: bool = False, sanitize: str | None = None, only: tuple | None = None) -> list[Path]:
    """Native executables: every csrc/{node,tui,orch_main}/*.cpp with a main().

    ``sanitize="address"`` (ASan + UBSan) or ``"thread"`` (TSan) builds instrumented copies under
    ``bin/<sanitize>/`` for the host-side race and memory checks of the C++ runtime (control plane, sessions,
    dynamic barrier, codec); the reference runs no sanitizer in CI (.github/workflows/test.yml:29-30)."""
    bindir = BINDIR if sanitize is None else BINDIR / sanitize
    # (sanitizer builds: no per-ISA clones of the hot loops, their load-time resolvers run before the sanitizer runtime is up)
    flags = CXX_FLAGS if sanitize is None else ["-O1", "-g1", "-fno-omit-frame-pointer", "-DONO_NO_CLONES", *CXX_FLAGS[1:],
                                                *SANITIZERS[sanitize]]
    cxx = CXX
    if sanitize is not None:
        cxx = sanitizer_cxx(sanitize)
        if cxx is None:
            raise RuntimeError(f"no C++ compiler here links the {sanitize} sanitizer runtime")
    bindir.mkdir(parents=True, exist_ok=True)
    out, jobs = [], []
    core_srcs = sorted((CSRC / "core").glob("*.cpp")) + sorted((CSRC / "oracle").glob("*.cpp"))
    hdrs = _headers(CSRC / "core", CSRC / "oracle", CSRC / "node", CSRC / "tui")
    for name, sub in (("ono-node", "node"), ("orchestui", "tui"), ("ono-orchestrator", "orch_main")):
        mains = sorted((CSRC / sub).glob("*.cpp")) if (CSRC / sub).exists() else []
        if not mains or (only is not None and name not in only):
            continue
        exe = bindir / name
        if force or any(_newer(s, exe, hdrs) for s in mains + core_srcs):
            jobs.append([cxx, *flags, "-I", str(CSRC), "-o", str(exe), *map(str, mains), *map(str, core_srcs), "-ldl"])
        out.append(exe)
    with cf.ThreadPoolExecutor(max_workers=min(4, os.cpu_count() or 2)) as ex:      # one compiler process per executable
        list(ex.map(_run, jobs))
    return out


def build_all(force: bool = False) -> dict:
    return {"kernels": build_kernels(force), "core": build_core(force), "bins": build_bins(force)}


if __name__ == "__main__":
    res = build_all(force="--force" in sys.argv)
    for k, v in res.items():
        print(k, v)
