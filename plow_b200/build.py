"""In-tree build of the native libraries.

Two shared objects are produced under ``plow_b200/lib``:

* ``libplow_cuda.so`` — every ``csrc/cuda/*.cu`` and ``csrc/comm/*.cu`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``; nvcc cross-compiles without a GPU).
* ``libplow_cpu.so``  — the packet reader, the counter-gated CPU interpreter and the golden
  C++ ops from ``csrc/cpu`` (g++), used for the CPU-only serving path and as a numeric oracle.

Objects are cached under ``build/`` keyed by a hash of the source and every header beside it,
so a second call is a no-op.  ``python -m plow_b200.build`` runs the build from the shell.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
# PLOW_LIBDIR / PLOW_EXTRA_NVCC_FLAGS build a variant beside the default one, e.g.
#   PLOW_LIBDIR=/tmp/plow_trace PLOW_EXTRA_NVCC_FLAGS=-DPLOW_DEVICE_TRACE python -m plow_b200.build
LIBDIR = Path(os.environ["PLOW_LIBDIR"]) if os.environ.get("PLOW_LIBDIR") else Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" if not os.environ.get("PLOW_LIBDIR") else \
    ROOT / "build" / ("variant_" + hashlib.sha256(os.environ["PLOW_LIBDIR"].encode()).hexdigest()[:8])

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-march=x86-64-v3", "-fopenmp", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _digest(src: Path, extra: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(extra).encode())
    deps = [src] + sorted(p for d in (src.parent, CSRC / "common", CSRC / "cuda")
                          for p in d.glob("*.h*")) + sorted((CSRC / "cuda").glob("*.cuh"))
    for p in deps:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _compile(cmd_prefix: list[str], src: Path, flags: list[str], verbose: bool) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    obj = OBJDIR / f"{src.parent.name}_{src.stem}.{_digest(src, flags)}.o"
    if obj.exists():
        return obj
    for old in OBJDIR.glob(f"{src.parent.name}_{src.stem}.*.o"):
        old.unlink()
    cmd = cmd_prefix + flags + ["-I", str(CSRC / "common"), "-I", str(CSRC / "cuda"), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, file=sys.stderr)
    return obj


def _link(cmd: list[str], objs: list[Path], out: Path, extra: list[str]) -> None:
    LIBDIR.mkdir(parents=True, exist_ok=True)
    stamp = hashlib.sha256(" ".join(sorted(o.name for o in objs)).encode()).hexdigest()[:16]
    stamp_file = OBJDIR / (out.name + "." + hashlib.sha256(str(out).encode()).hexdigest()[:8] + ".stamp")
    if out.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return
    r = subprocess.run(cmd + ["-shared", "-o", str(out)] + [str(o) for o in objs] + extra,
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {r.stderr}")
    stamp_file.write_text(stamp)


def build_cpu(verbose: bool = False) -> Path:
    """Compile csrc/cpu into libplow_cpu.so (no CUDA needed)."""
    srcs = sorted((CSRC / "cpu").glob("*.cpp"))
    out = LIBDIR / "libplow_cpu.so"
    if not srcs:
        return out
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(["g++"], s, CXX_FLAGS, verbose), srcs))
    _link(["g++"], objs, out, ["-fopenmp"])
    return out


def build_cuda(verbose: bool = False) -> Path | None:
    """Compile every CUDA source for sm_100a into libplow_cuda.so."""
    nvcc = _nvcc()
    out = LIBDIR / "libplow_cuda.so"
    if nvcc is None:
        return out if out.exists() else None
    srcs = sorted((CSRC / "cuda").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + os.environ.get("PLOW_EXTRA_NVCC_FLAGS", "").split()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        objs = list(ex.map(lambda s: _compile([nvcc], s, flags, verbose), srcs))
    _link([nvcc], objs, out, [])
    return out


def build_all(verbose: bool = False) -> dict:
    return {"cpu": build_cpu(verbose), "cuda": build_cuda(verbose)}


if __name__ == "__main__":
    res = build_all(verbose="-v" in sys.argv)
    for k, v in res.items():
        print(f"{k}: {v}")
