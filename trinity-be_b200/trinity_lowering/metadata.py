"""CUDA-independent validation of artifact metadata (requirements and manifest)."""
import json
import math
from dataclasses import dataclass
from types import MappingProxyType

# sm100 is this provider's target; the others are kept so that metadata of reference artifacts
# is still recognised.
TARGET_CAPABILITIES = {"sm100": (10, 0), "hopper": (9, 0), "sm89": (8, 9), "sm120": (12, 0)}
_WIDTH = {"bf16": 2, "fp32": 4}


def freeze(value):
    """Recursively read-only view of JSON data."""
    if isinstance(value, dict):
        return MappingProxyType({k: freeze(v) for k, v in value.items()})
    if isinstance(value, list):
        return tuple(freeze(v) for v in value)
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


def _positive(value, what):
    if type(value) is not int or not 0 < value <= 2 ** 63 - 1:
        raise ValueError(f"invalid {what}")


def requirements(data):
    """Validates a requirements mapping and returns it as frozen dataclasses."""
    if data["target"] not in TARGET_CAPABILITIES:
        raise ValueError("unsupported artifact target")
    _positive(data["world_size"], "world_size")
    seen, outputs, buffers = set(), 0, []
    for slot, raw in enumerate(data["buffers"]):
        fields = dict(raw)
        for key in ("shape", "strides", "input_names"):
            fields[key] = tuple(fields[key])
        b = BufferRequirement(**fields)
        if b.value != slot or b.dtype not in _WIDTH or not 1 <= len(b.shape) <= 3:
            raise ValueError("invalid canonical binding/dtype/shape")
        for extent in b.shape:
            _positive(extent, "shape extent")
        _positive(b.alignment, "alignment")
        row_major = tuple(math.prod(b.shape[axis + 1:]) for axis in range(len(b.shape)))
        if b.alignment < _WIDTH[b.dtype] or b.alignment & (b.alignment - 1) or b.strides != row_major:
            raise ValueError("invalid alignment/strides")
        elements = math.prod(b.shape)
        if b.bytes != elements * _WIDTH[b.dtype] or elements > 2 ** 31 - 1:
            raise ValueError("invalid buffer bytes")
        if bool(b.input_names or b.output_name is not None) != b.external:
            raise ValueError("invalid external binding")
        for name in b.input_names:
            if not isinstance(name, str) or name in seen:
                raise ValueError("invalid or duplicate input name")
            seen.add(name)
        if b.output_name is not None:
            if not isinstance(b.output_name, str):
                raise ValueError("invalid output name")
            outputs += 1
        if b.symmetric and data["world_size"] == 1:
            raise ValueError("streamed allocation cannot be symmetric")
        buffers.append(b)
    if outputs != 1:
        raise ValueError("exactly one output binding required")
    persistent = data["world_size"] > 1
    if data["nvshmem"] != persistent or data["workspace_symmetric"] != persistent:
        raise ValueError("inconsistent world/workspace mode")
    _positive(data["workspace_alignment"], "workspace alignment")
    if persistent:
        _positive(data["workspace_bytes"], "workspace bytes")
        if not data["cooperative_launch"]:
            raise ValueError("persistent launch must be cooperative")
    elif data["workspace_bytes"] != 0 or data["cooperative_launch"]:
        raise ValueError("streamed execution cannot have a control workspace")
    return Requirements(**{**data, "buffers": tuple(buffers)})


def manifest(text):
    """Parses and validates manifest.json; returns (data, Requirements)."""
    data = json.loads(text)
    if data.get("schema_version") != 1 or data.get("host_abi_version") != 1:
        raise ValueError("unsupported artifact/ABI version; recompile the artifact")
    if data.get("library") != "program.so" or data.get("source") != "source.cu":
        raise ValueError("invalid artifact bundle paths")
    req = requirements(data["requirements"])
    if data.get("execution") != ("persistent" if req.nvshmem else "streamed"):
        raise ValueError("inconsistent execution mode")
    if data["toolchain"]["cuda_major"] < 12:
        raise ValueError("artifacts need CUDA 12.8 or newer (the first toolkit with sm_100a)")
    return data, req
