"""Planning, emission and compilation: Python face of the C++ host library.

Same names and call shapes as the reference's ``trinity_lowering.compiler`` (which wraps a PyO3
module): ``PhysicalPlanBuilder``, ``PhysicalPlan``, ``lower_ir``, ``emit``, ``compile``,
``CudaSource``, ``CudaArtifact``, ``CompileConfig``, the ``*_implementations`` enumerations.
The Triton / Quack Python-source paths of the reference are not part of this provider.
"""
import ctypes
import json
import threading
from dataclasses import dataclass, field
from pathlib import Path

from . import _host as h
from .errors import CompileError  # noqa: F401  (re-exported)
from .metadata import freeze, manifest, requirements

DEFAULT_TARGET = "sm100"


class PhysicalPlan:
    """A validated, canonical plan (immutable)."""

    def __init__(self, handle):
        self._handle = handle

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_plan_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass

    def metadata_json(self):
        return h.text(h.library().th_plan_metadata_json(self._handle))

    @property
    def symbols(self):
        return json.loads(h.text(h.library().th_plan_symbols_json(self._handle)))

    @property
    def world_size(self):
        return h.library().th_plan_world_size(self._handle)

    def bind_symbols(self, bindings):
        names = [str(k).encode() for k in bindings]
        for value in bindings.values():
            if type(value) is not int:
                raise ValueError("symbol bindings must be integers")
        array = (ctypes.c_char_p * max(1, len(names)))(*names)
        values = (ctypes.c_int64 * max(1, len(names)))(*bindings.values())
        return PhysicalPlan(h.check_ptr(h.library().th_plan_bind_symbols(self._handle, array, values,
                                                                         len(names))))

    def same_body(self, other):
        return self._structure() == other._structure()

    def _structure(self):
        return h.text(h.library().th_plan_structure(self._handle))

    def __eq__(self, other):
        return isinstance(other, PhysicalPlan) and self._structure() == other._structure()

    def __hash__(self):
        return int(h.library().th_plan_hash(self._handle))


def _index_text(value):
    if type(value) is int:
        return str(value).encode()
    if isinstance(value, str):
        return value.encode()
    raise TypeError("loop bounds are integers or index expressions")


class PhysicalPlanBuilder:
    """Registers values, operations and explicit loops; ``build`` validates and canonicalises."""

    def __init__(self, world_size=1, target_name=DEFAULT_TARGET):
        if world_size == 0:
            raise ValueError("world_size must be positive")
        self._handle = h.check_ptr(h.library().th_builder_new(world_size, target_name.encode()))

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_builder_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass

    def add_value(self, dtype_name, shape, storage_name, *, name=None):
        shape = list(shape)
        if not shape or any(type(d) is not int or d <= 0 for d in shape):
            raise ValueError("positive shape required")
        array = (ctypes.c_int64 * len(shape))(*shape)
        return h.check_int(h.library().th_builder_add_value(
            self._handle, dtype_name.encode(), array, len(shape), storage_name.encode(),
            name.encode() if name is not None else None))

    def bind_input(self, name, value):
        h.check_int(h.library().th_builder_bind_input(self._handle, name.encode(), value))

    def add_operation(self, inflows, outflows, *, expression):
        ins, n_in = h.int_array(inflows)
        outs, n_out = h.int_array(outflows)
        return h.check_int(h.library().th_builder_add_operation(self._handle, ins, n_in, outs, n_out,
                                                               expression.encode()))

    def add_loop(self, kind, variable, start, stop, step, body):
        ids, n = h.int_array(body)
        return h.check_int(h.library().th_builder_add_loop(
            self._handle, kind.encode(), variable.encode(), _index_text(start), _index_text(stop),
            _index_text(step), ids, n))

    def build(self, statements, output_name, output):
        ids, n = h.int_array(statements)
        return PhysicalPlan(h.check_ptr(h.library().th_builder_build(self._handle, ids, n,
                                                                     output_name.encode(), output)))


def lower_ir(text, symbols, dtypes, target_name=DEFAULT_TARGET, world_size=1):
    """Reads loop/tensor IR text into plans (a list with one plan)."""
    sym_names = (ctypes.c_char_p * max(1, len(symbols)))(*[k.encode() for k in symbols])
    sym_values = (ctypes.c_int64 * max(1, len(symbols)))(*symbols.values())
    names = (ctypes.c_char_p * max(1, len(dtypes)))(*[k.encode() for k in dtypes])
    kinds = (ctypes.c_char_p * max(1, len(dtypes)))(*[v.encode() for v in dtypes.values()])
    out = (ctypes.c_void_p * 8)()
    count = h.check_int(h.library().th_lower_ir(text.encode(), sym_names, sym_values, len(symbols), names,
                                                kinds, len(dtypes), target_name.encode(), world_size,
                                                out, 8))
    return [PhysicalPlan(out[i]) for i in range(count)]


class _NativeSource:
    def __init__(self, handle):
        self._handle = handle

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_source_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass

    @property
    def code(self):
        return h.text(h.library().th_source_code(self._handle))

    def requirements_json(self):
        return h.text(h.library().th_source_requirements_json(self._handle))

    @property
    def launch_count(self):
        return h.library().th_source_launch_count(self._handle)


class CudaSource:
    """Emitted host program plus its buffer / launch requirements."""

    def __init__(self, native):
        self._native = native
        self._requirements = requirements(json.loads(native.requirements_json()))

    @property
    def code(self):
        return self._native.code

    @property
    def requirements(self):
        return self._requirements

    @property
    def launch_count(self):
        return self._native.launch_count


def emit(plan):
    """Selects sm_100a kernels for every region of ``plan`` and renders the host program."""
    return CudaSource(_NativeSource(h.check_ptr(h.library().th_emit(plan._handle))))


def kernel_candidates(plan):
    """Per-operation candidates and rejections of the native provider."""
    return json.loads(h.text(h.library().th_kernel_candidates_json(plan._handle)))


@dataclass
class CompileConfig:
    """Where the toolchain pieces live; there are no free-form compiler flags."""
    host_compiler: str = None
    library_dir: str = None
    cuda_root: str = None
    cutlass_root: str = None
    nvshmem_root: str = None
    extra: dict = field(default_factory=dict)


class CudaArtifact:
    """A compiled plan: directory with source.cu, exports.map, program.so, manifest.json,
    diagnostics.json.  The directory is removed on close() unless persist() was called."""

    def __init__(self, handle):
        self._handle = handle
        self._lock = threading.RLock()
        lib = h.library()
        data, self._requirements = manifest(h.text(lib.th_artifact_manifest_json(handle)))
        self._manifest = freeze(data)

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_artifact_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass

    @property
    def requirements(self):
        return self._requirements

    @property
    def manifest(self):
        return self._manifest

    @property
    def directory(self):
        with self._lock:
            return Path(h.text(h.library().th_artifact_directory(self._handle)))

    @property
    def artifact_path(self):
        with self._lock:
            return Path(h.text(h.library().th_artifact_path(self._handle)))

    @property
    def diagnostics(self):
        with self._lock:
            return freeze(json.loads(h.text(h.library().th_artifact_diagnostics_json(self._handle))))

    @property
    def code(self):
        with self._lock:
            return h.text(h.library().th_artifact_code(self._handle))

    def close(self):
        with self._lock:
            h.library().th_artifact_close(self._handle)

    def persist(self):
        with self._lock:
            return Path(h.text(h.library().th_artifact_persist(self._handle)))


def compile(source, config=None):
    """Builds program.so for an emitted source."""
    config = config or CompileConfig()
    return CudaArtifact(h.check_ptr(h.library().th_compile(
        source._native._handle,
        config.host_compiler.encode() if config.host_compiler else None,
        config.library_dir.encode() if config.library_dir else None)))


# ---------------------------------------------------------------- implementation enumeration
@dataclass(frozen=True)
class Implementation:
    """An implementation id with its static attributes (what the reference enumerates in
    src/emit/implementation/definitions/*.rs, plus the sm_100a ids of this provider)."""
    id: str
    attributes: dict

    def enumerate(self, dtypes, shapes, **attrs):
        arity = self.attributes.get("arity")
        if arity is not None and len(dtypes) != arity + 1:
            raise ValueError(f"{self.id} takes {arity} operand(s) and one result")
        if len(dtypes) != len(shapes):
            raise ValueError("one shape per dtype is required")
        if self.attributes.get("scalar") and "scalar" not in attrs:
            raise ValueError(f"{self.id} needs a scalar attribute")
        if not self.attributes.get("scalar") and "scalar" in attrs:
            raise ValueError(f"{self.id} takes no scalar attribute")
        family = self.attributes["family"]
        if family == "pointwise":
            if any(list(s) != list(shapes[0]) for s in shapes):
                raise ValueError("pointwise operands and result share one shape")
            return [self]
        if family == "reduce_sum":
            if len(shapes[0]) != 2 or list(shapes[1]) not in ([shapes[0][0]], [shapes[0][1]]):
                raise ValueError("reduce_sum maps [M,N] to [M]")
            ok = attrs.get("axis", 1) == 1 and dtypes[1] == "fp32" and list(shapes[1]) == [shapes[0][0]]
            return [self] if ok else []
        if family == "broadcast":
            if dtypes[0] != dtypes[1] or len(shapes[0]) != 1 or len(shapes[1]) != 2 or \
                    shapes[1][0] != shapes[0][0]:
                raise ValueError("broadcast maps [M] to [M,N] of the same dtype")
            return [self]
        return [self]


def gemm_implementations(target_name=DEFAULT_TARGET):
    return [
        Implementation("blackwell.tcgen05.bf16", {
            "family": "gemm", "tile": (128, 256, 64), "stages": 4, "accumulator": "tmem fp32 x2",
            "epilogue": ("bias_col", "bias_row", "bias_matrix", "relu", "silu", "silu_gate")}),
        Implementation("hopper.wgmma.bf16", {"family": "gemm", "tile": (128, 128, 64), "legacy": True}),
    ]


def pointwise_implementations(target_name=DEFAULT_TARGET):
    unary = ("square", "sqrt", "sigmoid", "relu")
    out = [Implementation(f"cuda.{n}", {"family": "pointwise", "arity": 2}) for n in ("add", "mul", "div")]
    out.append(Implementation("cuda.scalar_div", {"family": "pointwise", "arity": 1, "scalar": True}))
    out += [Implementation(f"cuda.{n}", {"family": "pointwise", "arity": 1}) for n in unary]
    return out


def reduce_sum_implementations(target_name=DEFAULT_TARGET):
    return [Implementation("cuda.reduce_sum", {"family": "reduce_sum", "arity": 1})]


def broadcast_implementations(target_name=DEFAULT_TARGET):
    return [Implementation("cuda.broadcast", {"family": "broadcast", "arity": 1})]


def all_gather_implementations(target_name=DEFAULT_TARGET):
    return [
        Implementation("sm100.peer_memory.two_shot_allreduce", {"family": "collective", "vector_bytes": 16}),
        Implementation("nvls.one_shot_push_nbi", {"family": "collective", "chunk": 128, "legacy": True}),
        Implementation("nvshmem.peer_push", {"family": "collective", "tile": (64, 64), "legacy": True}),
        Implementation("nvshmem.peer_pull", {"family": "collective", "tile": (64, 64), "legacy": True}),
    ]


# ---------------------------------------------------------------- names kept for importers
class TritonProgram:
    """The reference's Triton provider result (src/python.rs:726-753 there).  This provider has no
    Triton path; the name exists so that ``from trinity_lowering import TritonProgram`` keeps
    importing, and it cannot be constructed."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError("UnsupportedExecution: the sm_100a provider has no Triton path")


def _no_triton(name):
    def refuse(*args, **kwargs):
        raise NotImplementedError(f"UnsupportedExecution: {name} belongs to the Triton provider, "
                                  "which the sm_100a provider does not have")
    refuse.__name__ = name
    refuse.__doc__ = f"``{name}`` of the reference's Triton provider: refused here."
    return refuse


emit_python = _no_triton("emit_python")
emit_triton = _no_triton("emit_triton")
lower_triton = _no_triton("lower_triton")
