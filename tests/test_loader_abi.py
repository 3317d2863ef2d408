"""Loader and ABI layout checks on the CPU: fixture libraries built with g++ from
tests/fixtures/abi_fixture.cpp (the role of the reference's fixtures/library.cpp + core_test.cpp,
python/tests/test_core.py:5-37)."""
import ctypes
import json
import subprocess
from pathlib import Path

import pytest

from trinity_lowering import _host as h

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def fixtures(tmp_path_factory):
    out = tmp_path_factory.mktemp("abi")
    built = {}
    for name, flags in {"good": [], "bad_version": ["-DBAD_VERSION"], "bad_offset": ["-DBAD_OFFSET"],
                        "no_status": ["-DNO_STATUS"]}.items():
        target = out / f"{name}.so"
        subprocess.run(["g++", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", *flags,
                        "-I", str(ROOT / "include"), str(ROOT / "tests" / "fixtures" / "abi_fixture.cpp"),
                        "-o", str(target)], check=True)
        built[name] = target
    return built


def probe(path, mode=1):
    lib = h.library()
    text = lib.th_library_probe(str(path).encode(), mode)
    if not text:
        h.raise_last()
    return json.loads(text.decode())


def test_good_library_is_accepted_and_reports_its_requirements(fixtures):
    req = probe(fixtures["good"])
    assert req["buffers"][0]["input_names"] == ["X"] and req["target"] == "sm100"


@pytest.mark.parametrize("name", ["bad_version", "bad_offset"])
def test_layout_differences_are_refused(fixtures, name):
    with pytest.raises(ValueError, match="descriptor differs"):
        probe(fixtures[name])


def test_missing_symbol_and_wrong_mode_are_refused(fixtures):
    with pytest.raises(ValueError, match="trinity_status"):
        probe(fixtures["no_status"])
    with pytest.raises(ValueError, match="descriptor differs"):
        probe(fixtures["good"], mode=2)
    with pytest.raises(ValueError):
        probe(fixtures["good"].with_name("absent.so"))


def test_each_load_gets_a_private_copy(fixtures):
    """Two loads of one file must not share statics: the loader copies before dlopen
    (src/native/core.hpp:61-77; fixtures/core_test.cpp:15-19 in the reference)."""
    direct = ctypes.CDLL(str(fixtures["good"]))
    direct.trinity_launch(None, None)
    assert direct.fixture_launches() == 1
    probe(fixtures["good"])                      # a private copy is loaded and unloaded
    assert direct.fixture_launches() == 1


def test_abi_struct_layout_is_the_documented_one():
    """Offsets of the launch and error structs (src/native/abi.h:13-50): LP64."""
    code = r'''
#include <cstdio>
#include "trinity_abi.h"
using namespace trinity::abi;
int main() {
  Descriptor d = describe(1, "", 0), p = describe(2, "", 0);
  printf("%u %u %u %u %u %u %u %u|", d.version, d.pointer_size, d.error_size, d.error_alignment, d.launch_size,
         d.launch_alignment, d.field_count, (unsigned)sizeof(Descriptor));
  for (int i = 0; i < 3; ++i) printf("%u ", d.offsets[i]);
  printf("|");
  for (int i = 0; i < 6; ++i) printf("%u ", d.error_offsets[i]);
  printf("|%u %u ", p.launch_size, p.field_count);
  for (int i = 0; i < 9; ++i) printf("%u ", p.offsets[i]);
  return 0;
}'''
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "layout.cpp"
        src.write_text(code)
        subprocess.run(["g++", "-std=c++17", "-I", str(ROOT / "include"), str(src), "-o", str(Path(tmp) / "layout")],
                       check=True)
        out = subprocess.run([str(Path(tmp) / "layout")], capture_output=True, text=True, check=True).stdout
    assert out == "1 8 24 4 24 8 3 112|0 8 16 |0 4 8 12 16 20 |64 9 0 8 16 24 32 40 44 48 56 "


def test_peer_table_bytes_match_the_c_struct():
    """The runtime fills a persistent artifact's peer table from Python; its byte layout must be
    the C struct's (include/trinity_sm100.h), which the kernels read on the device."""
    import struct
    import tempfile
    from trinity_lowering import kernels
    code = r'''
#include <cstddef>
#include <cstdio>
#include "trinity_sm100.h"
int main() {
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %d %d", sizeof(trinity_sm100_peer_table),
         offsetof(trinity_sm100_peer_table, rank), offsetof(trinity_sm100_peer_table, epoch),
         offsetof(trinity_sm100_peer_table, counter), offsetof(trinity_sm100_peer_table, failed),
         offsetof(trinity_sm100_peer_table, workspace), offsetof(trinity_sm100_peer_table, buffers),
         offsetof(trinity_sm100_peer_table, flags), TRINITY_SM100_PEER_BUFFERS, TRINITY_SM100_PEER_TABLE_BYTES);
  return 0;
}'''
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "table.cpp"
        src.write_text(code)
        subprocess.run(["g++", "-std=c++17", "-I", str(ROOT / "include"), str(src), "-o", str(Path(tmp) / "table")],
                       check=True)
        out = subprocess.run([str(Path(tmp) / "table")], capture_output=True, text=True, check=True).stdout
    size, rank, epoch, counter, failed, workspace, buffers, flags, slots, reserved = map(int, out.split())
    assert (slots, reserved) == (kernels.PEER_BUFFERS, kernels.PEER_TABLE_BYTES) and size <= reserved
    table = kernels.peer_table(4, 2, [0x1000, 0x2000, 0x3000, 0x4000], [[0x10, 0x20, 0x30, 0x40], [0x50, 0x60, 0x70, 0x80]])
    assert len(table) == reserved
    assert struct.unpack_from("<i", table, 0)[0] == 4 and struct.unpack_from("<i", table, rank)[0] == 2
    assert struct.unpack_from("<III", table, epoch) == (0, 0, 0) and (counter, failed) == (epoch + 4, epoch + 8)
    assert struct.unpack_from("<4Q", table, workspace) == (0x1000, 0x2000, 0x3000, 0x4000)
    assert struct.unpack_from("<4Q", table, buffers) == (0x10, 0x20, 0x30, 0x40)
    assert struct.unpack_from("<4Q", table, buffers + 64) == (0x50, 0x60, 0x70, 0x80)
    assert not any(table[flags:])            # flags start at zero: a fresh pad reads as call number 0
