"""The shared libraries load without a GPU and export every symbol their C headers declare
(no compute call is made here)."""
import ctypes
import re
from pathlib import Path

from trinity_lowering import _host, kernels

ROOT = Path(__file__).resolve().parents[1]


def declared(header, macro):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(macro + r"\s+[\w\s\*]+?\b(\w+)\s*\(", text)


def test_kernel_library_exports_every_declared_entry_point():
    names = declared("trinity_sm100.h", "TRINITY_SM100_API")
    assert len(names) >= 25 and "trinity_sm100_gemm_bf16" in names and "trinity_sm100_allgather_bf16" in names
    library = ctypes.CDLL(str(kernels.library_path()))
    missing = [name for name in names if not hasattr(library, name)]
    assert not missing, missing
    assert sorted(names) == sorted(kernels.EXPORTS)        # the Python binding lists the same surface
    assert kernels.library().trinity_sm100_abi_version() == 1


def test_host_library_exports_every_declared_entry_point():
    names = declared("trinity_host.h", "TRINITY_HOST_API")
    assert len(names) >= 30 and "th_execution_create_persistent" in names
    library = _host.library()
    missing = [name for name in names if not hasattr(library, name)]
    assert not missing, missing
