"""Builds the native parts in-tree: the sm_100a kernel library and the C++ host libraries.

Everything is compiled with explicit nvcc / g++ command lines into ``trinity-be_b200/lib`` so
the shared objects travel with the source tree.  nvcc cross-compiles for sm_100a without a GPU.
"""
import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent
REPO = ROOT.parent
CSRC = ROOT / "csrc"
HOST = ROOT / "host"
LIB = ROOT / "lib"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc():
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _stale(target, sources):
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > stamp for s in sources)


def _run(command):
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(map(str, command)),
                                                        result.stdout, result.stderr))
    return result


def build_kernels(force=False):
    """nvcc -> lib/libtrinity_sm100.so (all CUDA kernels + their C ABI)."""
    LIB.mkdir(exist_ok=True)
    target = LIB / "libtrinity_sm100.so"
    sources = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [
        REPO / "include" / "trinity_sm100.h"]
    if force or _stale(target, sources):
        _run([_nvcc(), *NVCC_FLAGS, "-o", str(target), str(CSRC / "libtrinity_sm100.cu")])
    return target


def build_host(force=False):
    """g++ -> lib/libtrinity_host.so (plan model, emitter, artifact runtime; no CUDA headers)."""
    LIB.mkdir(exist_ok=True)
    target = LIB / "libtrinity_host.so"
    sources = sorted(HOST.glob("*.cpp"))
    if not sources:
        return None
    deps = sources + list(HOST.glob("*.hpp")) + list(HOST.glob("*.h")) + list(
        (REPO / "include").glob("*.h"))
    if force or _stale(target, deps):
        cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
        _run(["g++", "-std=c++17", "-O2", "-shared", "-fPIC", "-fvisibility=hidden",
              "-I", str(REPO / "include"), "-I", str(cuda / "include"), "-o", str(target),
              *map(str, sources), "-L", str(cuda / "lib64"), "-lcudart_static", "-ldl", "-lrt",
              "-lpthread"])
    return target


def build_all(force=False):
    built = [build_kernels(force)]
    host = build_host(force)
    if host:
        built.append(host)
    return built


if __name__ == "__main__":
    for path in build_all(force=True):
        print(path)
