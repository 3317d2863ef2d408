"""Host-side failures of a program.so and the bookkeeping that follows (B200 only; no GPU fault is
involved: the fixture's entry points return error codes on the host).  Scenarios of the
reference's runtime tests (python/tests/test_cuda_runtime.py:295-324, :379-394 there, fixture
switches python/tests/fixtures/cuda_library.cu:16-19): a launch that fails after work may have
been submitted, an execution that cannot run again and still closes, a release that fails and is
retried, a prepare that fails before anything was submitted."""
import json
import subprocess
from pathlib import Path

import pytest
import torch

import trinity_lowering as tl

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DEV = "cuda:0"

REQUIREMENTS = {
    "target": "sm100", "world_size": 1,
    "buffers": [{"value": 0, "input_names": ["X"], "output_name": "Y", "shape": [4], "dtype": "fp32",
                 "strides": [1], "bytes": 16, "alignment": 4, "external": True, "symmetric": False}],
    "workspace_bytes": 0, "workspace_alignment": 1, "workspace_symmetric": False,
    "cooperative_launch": False, "shared_memory_bytes": 0, "block_threads": 128, "nvshmem": False,
    "nvls": False,
}


@pytest.fixture(scope="module")
def artifact_directory(tmp_path_factory):
    """An artifact directory around the host-only fixture library."""
    out = tmp_path_factory.mktemp("failing_artifact")
    subprocess.run(["g++", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-I", str(ROOT / "include"),
                    str(ROOT / "tests" / "fixtures" / "abi_fixture.cpp"), "-o", str(out / "program.so")], check=True)
    (out / "source.cu").write_text("// host-only fixture\n")
    manifest = {"schema_version": 1, "host_abi_version": 1, "execution": "streamed", "library": "program.so",
                "source": "source.cu", "requirements": REQUIREMENTS,
                "toolchain": {"nvcc": None, "cuda_major": 12, "kernel_library": None, "cutlass": None,
                              "nvshmem": None, "nvshmem_library_directory": None, "host_compiler": "g++"}}
    (out / "manifest.json").write_text(json.dumps(manifest))
    return out


@torch.inference_mode()
def test_partial_enqueue_error_and_release_retry(artifact_directory, monkeypatch):
    module = tl.load(artifact_directory, DEV)
    x = torch.ones(4, device=DEV, dtype=torch.float32)
    execution = module.prepare({"X": x}, out=x)
    execution.run()
    execution.wait(timeout=30)

    monkeypatch.setenv("TRINITY_FIXTURE_FAILURE", "launch")
    with pytest.raises(tl.RuntimeFailure) as error:
        execution.run()
    assert error.value.code == 719 and error.value.submitted
    monkeypatch.delenv("TRINITY_FIXTURE_FAILURE")

    with pytest.raises(tl.RuntimeFailure):      # a failed execution never runs again
        execution.run()
    with pytest.raises(tl.ResourceBusy):        # and still counts as a live child of its module
        module.close()
    with pytest.raises(tl.RuntimeFailure):      # closing reports the failure ...
        execution.close()
    assert execution._closed                    # ... after the execution has been closed
    execution.close()                           # idempotent

    monkeypatch.setenv("TRINITY_FIXTURE_FAILURE", "release")
    with pytest.raises(tl.RuntimeFailure) as error:
        module.close()
    assert error.value.code == 19
    monkeypatch.delenv("TRINITY_FIXTURE_FAILURE")
    module.close()                              # the module stayed prepared: the retry succeeds


@torch.inference_mode()
def test_prepare_error_leaves_the_module_usable(artifact_directory, monkeypatch):
    module = tl.load(artifact_directory, DEV)
    x = torch.ones(4, device=DEV, dtype=torch.float32)
    monkeypatch.setenv("TRINITY_FIXTURE_FAILURE", "prepare")
    with pytest.raises(tl.RuntimeFailure) as error:
        module.prepare({"X": x}, out=x)
    assert error.value.code == 17 and not error.value.submitted
    monkeypatch.delenv("TRINITY_FIXTURE_FAILURE")
    execution = module.prepare({"X": x}, out=x)
    execution.run()
    execution.wait(timeout=30)
    execution.close()
    module.close()
