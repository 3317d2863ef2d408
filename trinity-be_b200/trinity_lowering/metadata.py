"""Artifact metadata: the requirements JSON embedded in a ``program.so`` and ``manifest.json``.

Everything here is plain data checking and needs no CUDA.  The rules are those the reference
enforces on its artifacts (python/src/trinity_lowering/metadata.py:54-132 there): bindings are
numbered canonically, BF16 or FP32, rank 1 to 3, densely row-major, aligned to a power of two that
is at least the element size, named as inputs or as the single output exactly when they are
external; a streamed (single-GPU) artifact has no control workspace, a persistent (multi-GPU)
one has a symmetric workspace and a cooperative launch.
"""
import json
from dataclasses import dataclass, fields
from types import MappingProxyType

# compute capability per target name; "sm100" is this provider's, the others let metadata of
# artifacts built by the reference be read
TARGET_CAPABILITIES = {"sm100": (10, 0), "hopper": (9, 0), "sm89": (8, 9), "sm120": (12, 0)}
ELEMENT_BYTES = {"bf16": 2, "fp32": 4}
_INT64_MAX = (1 << 63) - 1
_INT32_MAX = (1 << 31) - 1


def freeze(value):
    """A read-only copy of parsed JSON (mappings become mapping proxies, lists tuples)."""
    if isinstance(value, list):
        return tuple(map(freeze, value))
    if isinstance(value, dict):
        return MappingProxyType({key: freeze(item) for key, item in value.items()})
    return value


@dataclass(frozen=True)
class BufferRequirement:
    value: int
    input_names: tuple
    output_name: object
    shape: tuple
    dtype: str
    strides: tuple
    bytes: int
    alignment: int
    external: bool
    symmetric: bool


@dataclass(frozen=True)
class Requirements:
    target: str
    world_size: int
    buffers: tuple
    workspace_bytes: int
    workspace_alignment: int
    workspace_symmetric: bool
    cooperative_launch: bool
    shared_memory_bytes: int
    block_threads: int
    nvshmem: bool
    nvls: bool


def _is_count(value):
    """A JSON integer (not a bool) in (0, 2^63)."""
    return type(value) is int and 0 < value <= _INT64_MAX


def _dense_strides(shape):
    strides, run = [], 1
    for extent in reversed(shape):
        strides.append(run)
        run *= extent
    return tuple(reversed(strides)), run


class _BindingChecker:
    """Checks the buffer list entry by entry and keeps what spans entries (names, outputs)."""

    def __init__(self, single_gpu):
        self.single_gpu = single_gpu
        self.input_names = set()
        self.output_count = 0

    def check(self, slot, raw):
        entry = {**raw, "shape": tuple(raw["shape"]), "strides": tuple(raw["strides"]),
                 "input_names": tuple(raw["input_names"])}
        buffer = BufferRequirement(**{f.name: entry[f.name] for f in fields(BufferRequirement)})
        width = ELEMENT_BYTES.get(buffer.dtype)
        if buffer.value != slot or width is None or len(buffer.shape) not in (1, 2, 3):
            raise ValueError("invalid canonical binding/dtype/shape")
        if not all(_is_count(extent) for extent in buffer.shape):
            raise ValueError("invalid shape extent")
        if not _is_count(buffer.alignment):
            raise ValueError("invalid alignment")
        expected_strides, elements = _dense_strides(buffer.shape)
        power_of_two = buffer.alignment & (buffer.alignment - 1) == 0
        if not power_of_two or buffer.alignment < width or buffer.strides != expected_strides:
            raise ValueError("invalid alignment/strides")
        if elements > _INT32_MAX or buffer.bytes != elements * width:
            raise ValueError("invalid buffer bytes")
        named = bool(buffer.input_names) or buffer.output_name is not None
        if named != buffer.external:
            raise ValueError("invalid external binding")
        for name in buffer.input_names:
            if not isinstance(name, str) or name in self.input_names:
                raise ValueError("invalid or duplicate input name")
            self.input_names.add(name)
        if buffer.output_name is not None:
            if not isinstance(buffer.output_name, str):
                raise ValueError("invalid output name")
            self.output_count += 1
        if buffer.symmetric and self.single_gpu:
            raise ValueError("streamed allocation cannot be symmetric")
        return buffer


def requirements(data):
    """Validates a requirements mapping; returns it as frozen dataclasses."""
    if data["target"] not in TARGET_CAPABILITIES:
        raise ValueError("unsupported artifact target")
    if not _is_count(data["world_size"]):
        raise ValueError("invalid world_size")
    multi_gpu = data["world_size"] > 1
    checker = _BindingChecker(single_gpu=not multi_gpu)
    buffers = tuple(checker.check(slot, raw) for slot, raw in enumerate(data["buffers"]))
    if checker.output_count != 1:
        raise ValueError("exactly one output binding required")
    # execution mode: world size, transport and workspace must tell the same story
    if data["nvshmem"] != multi_gpu or data["workspace_symmetric"] != multi_gpu:
        raise ValueError("inconsistent world/workspace mode")
    if not _is_count(data["workspace_alignment"]):
        raise ValueError("invalid workspace alignment")
    if multi_gpu:
        if not _is_count(data["workspace_bytes"]):
            raise ValueError("invalid workspace bytes")
        if not data["cooperative_launch"]:
            raise ValueError("persistent launch must be cooperative")
    elif data["workspace_bytes"] != 0 or data["cooperative_launch"]:
        raise ValueError("streamed execution cannot have a control workspace")
    return Requirements(**{f.name: (buffers if f.name == "buffers" else data[f.name]) for f in fields(Requirements)})


def manifest(text):
    """Parses and validates ``manifest.json``; returns (parsed manifest, Requirements)."""
    parsed = json.loads(text)
    versions = (parsed.get("schema_version"), parsed.get("host_abi_version"))
    if versions != (1, 1):
        raise ValueError("unsupported artifact/ABI version; recompile the artifact")
    if (parsed.get("library"), parsed.get("source")) != ("program.so", "source.cu"):
        raise ValueError("invalid artifact bundle paths")
    needs = requirements(parsed["requirements"])
    if parsed.get("execution") != ("persistent" if needs.nvshmem else "streamed"):
        raise ValueError("inconsistent execution mode")
    if parsed["toolchain"]["cuda_major"] < 12:
        raise ValueError("artifacts need CUDA 12.8 or newer (the first toolkit with sm_100a)")
    return parsed, needs
