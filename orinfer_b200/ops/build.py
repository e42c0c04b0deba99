"""Build the native libraries in-tree with nvcc / g++ (no JIT cache).

``liborinfer_kernels.so`` holds every CUDA kernel, compiled for sm_100a only;
``liborinfer_core.so`` holds the C++ policy core (scheduler, radix prefix cache,
sampling law, MTP controller, ...) and needs no GPU.  Run as
``python -m orinfer_b200.ops.build`` or through ``__graft_entry__.build()``.
"""

from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
OUT = ROOT / "orinfer_b200" / "_native"
OBJ = ROOT / "build" / "obj"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-pthread"]


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(path.parent.glob("*.h")) + sorted(path.parent.glob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile(cmd, obj: Path, stamp: str, log: Path):
    tag = obj.with_suffix(".stamp")
    if obj.exists() and tag.exists() and tag.read_text() == stamp:
        return obj, ""
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError(f"compile failed: {' '.join(map(str, cmd))}\n{res.stdout}{res.stderr}")
    tag.write_text(stamp)
    return obj, res.stderr


def build_kernels(verbose: bool = False) -> Path:
    OUT.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    jobs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        for src in srcs:
            obj = OBJ / (src.stem + ".o")
            cmd = [NVCC, *CUDA_FLAGS, "-I", str(CSRC / "kernels"), "-c", str(src), "-o", str(obj)]
            jobs.append(pool.submit(_compile, cmd, obj, _digest(src, " ".join(CUDA_FLAGS)),
                                    OBJ / (src.stem + ".log")))
        objs = [j.result() for j in jobs]
    lib = OUT / "liborinfer_kernels.so"
    cmd = [NVCC, "-shared", "-o", str(lib), *[str(o) for o, _ in objs], "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError(res.stdout + res.stderr)
    if verbose:
        for _, log in objs:
            sys.stderr.write(log)
    return lib


SANITIZERS = {"asan": "address,undefined", "tsan": "thread"}


def build_core(sanitizer: str = "") -> Path:
    """The C++ policy core.  ``sanitizer`` = "asan" (AddressSanitizer + UBSan) or "tsan"
    builds an instrumented ``liborinfer_core_<sanitizer>.so`` beside the normal one; load it
    with ``ORINFER_CORE_LIB`` and the matching runtime preloaded (see tests/test_sanitizers.py)."""
    OUT.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "core").glob("*.cpp")) + sorted((CSRC / "dist").glob("*.cpp"))
    tag = f"_{sanitizer}" if sanitizer else ""
    lib = OUT / f"liborinfer_core{tag}.so"
    if not srcs:
        return lib
    flags = list(CXX_FLAGS)
    if sanitizer:
        flags = [f for f in flags if not f.startswith("-O")] + [
            "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={SANITIZERS[sanitizer]}",
            "-fno-sanitize-recover=undefined"]
    objs = []
    with cf.ThreadPoolExecutor(max_workers=8) as pool:
        jobs = []
        for src in srcs:
            obj = OBJ / (f"core{tag}_" + src.stem + ".o")
            cmd = ["g++", *flags, "-I", str(CSRC / "core"), "-c", str(src), "-o", str(obj)]
            jobs.append(pool.submit(_compile, cmd, obj, _digest(src, " ".join(flags)),
                                    OBJ / (f"core{tag}_" + src.stem + ".log")))
        objs = [j.result()[0] for j in jobs]
    link = ["g++", "-shared", "-pthread"]
    if sanitizer:
        link.append(f"-fsanitize={SANITIZERS[sanitizer]}")
    res = subprocess.run([*link, "-o", str(lib), *map(str, objs)],
                         capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError(res.stdout + res.stderr)
    return lib


def build_all(verbose: bool = False):
    return build_kernels(verbose), build_core()


if __name__ == "__main__":
    libs = build_all(verbose="-v" in sys.argv)
    print("\n".join(str(p) for p in libs))
