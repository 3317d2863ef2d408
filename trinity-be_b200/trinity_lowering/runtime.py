"""Loading compiled plans and running them on PyTorch tensors and streams.

Importing this module does not initialise CUDA.  PyTorch supplies device memory, streams and
events; validation of tensors against the artifact's buffer metadata happens here, everything
after that (launch, completion, graph capture) in the C++ runtime.
"""
import ctypes
import hashlib
import json
import threading
from collections.abc import Mapping
from dataclasses import dataclass
from pathlib import Path
from types import MappingProxyType

from . import _host as h
from .compiler import CudaArtifact
from .errors import ResourceBusy
from .metadata import TARGET_CAPABILITIES, freeze, manifest

_TORCH_DTYPE = {"bf16": "bfloat16", "fp32": "float32"}


def native():
    """The host library (kept under the reference's accessor name)."""
    return _Native


class _Native:
    @staticmethod
    def collect_local():
        return int(h.library().th_collect_local())

    @staticmethod
    def retire_pending():
        return int(h.library().th_retire_pending())

    @staticmethod
    def cuda_version():
        return h.library().th_cuda_runtime_version()


def device_of(device, target="sm100"):
    """The execution device as a torch.device with an index; it must be a CUDA device of the
    compute capability the artifact was built for."""
    import torch
    chosen = torch.device(device)
    if chosen.type != "cuda":
        raise ValueError("a CUDA device is required")
    if chosen.index is None:
        chosen = torch.device("cuda", torch.cuda.current_device())
    capability = TARGET_CAPABILITIES.get(target)
    if capability is None:
        raise ValueError("unsupported artifact target")
    if tuple(torch.cuda.get_device_capability(chosen)) != capability:
        raise ValueError(f"this artifact requires a {target} device")
    return chosen


def stream_of(device, stream=None, wait_for=()):
    """The stream a launch goes to (the current one by default), after making it wait for the
    caller's events."""
    import torch
    chosen = torch.cuda.current_stream(device) if stream is None else stream
    if not (isinstance(chosen, torch.cuda.Stream) and chosen.device == device):
        raise ValueError("stream must be a torch.cuda.Stream on the execution device")
    pending = list(wait_for)
    for event in pending:
        if not isinstance(event, torch.cuda.Event):
            raise ValueError("wait_for must contain recorded CUDA events on the execution device")
    for event in pending:
        chosen.wait_event(event)
    return chosen


def tensor_check(tensor, b, device, world=None):
    """dtype, shape, stride, device, alignment and storage size against one buffer requirement."""
    import torch
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"binding {b.value} requires a Tensor")
    wanted = getattr(torch, _TORCH_DTYPE[b.dtype])
    layout_ok = (tensor.layout == torch.strided and tuple(tensor.shape) == b.shape
                 and tuple(tensor.stride()) == b.strides)
    if not (layout_ok and tensor.dtype == wanted and tensor.device == device):
        raise ValueError(f"binding {b.value}: dtype/shape/stride/device mismatch")
    if tensor.requires_grad and torch.is_grad_enabled():
        raise ValueError("use no_grad or inference_mode for gradient Tensors")
    behind = tensor.untyped_storage().nbytes() - tensor.storage_offset() * tensor.element_size()
    if behind < b.bytes or tensor.data_ptr() % b.alignment != 0:
        raise ValueError(f"binding {b.value}: alignment/storage mismatch")
    if b.symmetric and (world is None or world.symmetric_buffer_of(tensor) is None):
        raise ValueError(f"binding {b.value} requires this world's symmetric allocation")


def _overlapping(first, second):
    (a0, a_len), (b0, b_len) = first, second
    return a0 < b0 + b_len and b0 < a0 + a_len


def resolve_bindings(req, inputs, out, device, world=None, allow_missing=False):
    """Maps buffer slots to the caller's tensors: every input name must be known (and, unless
    ``allow_missing``, present), aliases of one value must be one region, distinct values must not
    overlap."""
    if not isinstance(inputs, Mapping):
        raise TypeError("inputs must be a mapping of binding names to Tensors")
    known = set()
    for requirement in req.buffers:
        known.update(requirement.input_names)
    given = set(inputs)
    if not given <= known or (given != known and not allow_missing):
        raise ValueError(f"expected exactly input names {sorted(known)}")
    bound = {}
    for requirement in req.buffers:
        tensors = [inputs[name] for name in requirement.input_names if name in inputs]
        if out is not None and requirement.output_name is not None:
            tensors.append(out)
        if not tensors:
            continue
        for tensor in tensors:
            tensor_check(tensor, requirement, device, world)
        first = tensors[0]
        if any(other.data_ptr() != first.data_ptr() for other in tensors[1:]):
            raise ValueError("names referring to the same value must share one Tensor region")
        bound[requirement.value] = first
    spans = [(tensor.data_ptr(), req.buffers[slot].bytes) for slot, tensor in bound.items()]
    for position, span in enumerate(spans):
        if any(_overlapping(span, earlier) for earlier in spans[:position]):
            raise ValueError("different canonical values overlap")
    return bound


@dataclass(frozen=True)
class IOBuffers:
    inputs: Mapping
    output: object


def outside_capture(device):
    import torch
    with torch.cuda.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise ResourceBusy("load, prepare and Trinity allocation must finish before capture")


class LoadedModule:
    def __init__(self, handle, data, req, device, fingerprint, world=None):
        self._handle, self._requirements, self._device = handle, req, device
        self._manifest, self._fingerprint = freeze(data), fingerprint
        self._closed = False
        self._lock = threading.RLock()
        self._world = world

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_module_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass

    requirements = property(lambda self: self._requirements)
    manifest = property(lambda self: self._manifest)
    device = property(lambda self: self._device)
    world = property(lambda self: self._world)
    fingerprint = property(lambda self: self._fingerprint)

    def _open(self):
        if self._closed:
            raise RuntimeError("module is closed")

    def _allocate(self, b):
        import torch
        if b.symmetric:
            # every rank's copy is mapped into every process (a collective step of the world)
            return self._world.allocate(b.shape, getattr(torch, _TORCH_DTYPE[b.dtype])).tensor
        # Over-allocated byte storage supports alignments stronger than the allocator's.
        owner = torch.empty(b.bytes + b.alignment - 1, dtype=torch.uint8, device=self.device)
        offset = (-owner.data_ptr()) % b.alignment
        dtype = getattr(torch, _TORCH_DTYPE[b.dtype])
        return owner[offset:offset + b.bytes].view(dtype).view(b.shape)

    def _bindings(self, inputs, out, allow_missing=False):
        self._open()
        outside_capture(self.device)
        return resolve_bindings(self.requirements, inputs, out, self.device, self._world, allow_missing)

    def allocate_io(self, inputs=None):
        with self._lock:
            bound = self._bindings({} if inputs is None else inputs, None, True)
            for b in self.requirements.buffers:
                if b.external and b.value not in bound:
                    bound[b.value] = self._allocate(b)
            return IOBuffers(
                MappingProxyType({name: bound[b.value] for b in self.requirements.buffers
                                  for name in b.input_names}),
                next(bound[b.value] for b in self.requirements.buffers if b.output_name is not None))

    def prepare(self, inputs, out=None, workers=None):
        import torch
        with self._lock:
            bound = self._bindings(inputs, out)
            lib = h.library()
            maximum = ctypes.c_uint(0)
            with torch.cuda.device(self.device):
                if lib.th_module_prepare(self._handle, ctypes.byref(maximum)) != 0:
                    h.raise_last()
            chosen = maximum.value if workers is None else workers
            if type(chosen) is not int or not 1 <= chosen <= maximum.value:
                raise ValueError(f"workers must be within [1, {maximum.value}]")
            for b in self.requirements.buffers:
                if b.value not in bound:
                    bound[b.value] = self._allocate(b)
            tensors = [bound[b.value] for b in self.requirements.buffers]
            pointers = (ctypes.c_void_p * max(1, len(tensors)))(*[t.data_ptr() for t in tensors])
            stream = torch.cuda.current_stream(self.device)
            workspace = None
            if self._world is None:
                handle = h.check_ptr(lib.th_execution_create(self._handle, pointers, len(tensors),
                                                             ctypes.c_void_p(stream.cuda_stream)))
            else:
                workspace = self._peer_workspace(tensors)
                handle = h.check_ptr(lib.th_execution_create_persistent(
                    self._handle, pointers, len(tensors), ctypes.c_void_p(workspace.tensor.data_ptr()),
                    workspace.tensor.numel(), chosen, ctypes.c_void_p(stream.cuda_stream)))
            output = next(bound[b.value] for b in self.requirements.buffers if b.output_name is not None)
            named = {n: bound[b.value] for b in self.requirements.buffers for n in b.input_names}
            return PreparedExecution(self, handle, named, tensors, output, workspace)

    def _peer_workspace(self, tensors):
        """The execution's workspace in symmetric memory, its first bytes the peer table the
        kernels read: every rank's workspace and every rank's copy of the symmetric plan buffers,
        as mapped into this process.  All ranks finish this step before any of them launches."""
        import torch
        from . import kernels
        world, req = self._world, self.requirements
        size = max(req.workspace_bytes, kernels.PEER_TABLE_BYTES)
        workspace = world.allocate((size,), torch.uint8)
        peers = []
        for b, tensor in zip(req.buffers, tensors):
            if b.symmetric:
                owner = world.symmetric_buffer_of(tensor)
                peers.append(owner.peer_ptrs)
        table = kernels.peer_table(world.size, world.rank, workspace.peer_ptrs, peers)
        workspace.tensor.zero_()
        workspace.tensor[:len(table)].copy_(torch.frombuffer(bytearray(table), dtype=torch.uint8))
        torch.cuda.synchronize(self.device)
        world.barrier()
        return workspace

    def close(self, wait=True):
        with self._lock:
            if not self._closed:
                if h.library().th_module_close(self._handle) != 0:
                    h.raise_last()
                self._closed = True


class PreparedExecution:
    """A module bound to concrete tensors.  The tensors are kept alive here; their addresses and
    storages must not change while the execution is open."""

    def __init__(self, module, handle, inputs, tensors, output, workspace=None):
        self._module, self._handle = module, handle
        self._workspace = workspace      # persistent modules: the symmetric workspace with the peer table
        self._inputs = MappingProxyType(inputs)
        self._tensors, self._output = tensors, output
        self._snapshot = [(t.data_ptr(), t.untyped_storage().data_ptr()) for t in tensors]
        self._closed = False
        self._graph = None

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_execution_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass

    module = property(lambda self: self._module)
    inputs = property(lambda self: self._inputs)
    output = property(lambda self: self._output)
    world = property(lambda self: self._module.world)

    def _validate(self):
        if self._closed:
            raise RuntimeError("execution is closed")
        for tensor, (address, storage) in zip(self._tensors, self._snapshot):
            if tensor.data_ptr() != address or tensor.untyped_storage().data_ptr() != storage:
                raise ValueError("a bound tensor's storage was replaced after prepare")

    def run(self, stream=None, wait_for=()):
        self._validate()
        st = stream_of(self._module.device, stream, wait_for)
        if h.library().th_execution_run(self._handle, ctypes.c_void_p(st.cuda_stream)) != 0:
            h.raise_last()
        return self._output

    def wait(self, timeout=None):
        if self._closed:
            return
        if h.library().th_execution_wait(self._handle, -1.0 if timeout is None else float(timeout)) != 0:
            h.raise_last()

    def close(self, wait=True):
        if self._closed:
            return
        failed = h.library().th_execution_close(self._handle, 1 if wait else 0) != 0
        if not failed or h.library().th_execution_closed(self._handle):
            # an execution that failed earlier closes all the same and then reports the failure
            self._closed = True
            self._inputs = MappingProxyType({})
        if failed:
            h.raise_last()


def load(artifact_or_directory, device, world=None):
    """Loads an artifact (or a persisted artifact directory) onto ``device``."""
    artifact = artifact_or_directory
    directory = artifact.directory if isinstance(artifact, CudaArtifact) else Path(artifact)
    data, req = manifest((directory / "manifest.json").read_text())
    d = device_of(device, req.target)
    outside_capture(d)
    if req.nvshmem != (world is not None):
        raise ValueError("artifact requires a matching world" if req.nvshmem else
                         "a streamed artifact is loaded without a world")
    if world is not None and (world.size != req.world_size or world.device != d):
        raise ValueError("the world's size and device must be the artifact's")
    fingerprint = hashlib.sha256((directory / "source.cu").read_bytes()
                                 + json.dumps(data["requirements"], sort_keys=True).encode()).hexdigest()
    lib = h.library()
    handle = h.check_ptr(lib.th_module_load(str(directory / "program.so").encode(), d.index,
                                            2 if world is not None else 1))
    if json.loads(h.text(lib.th_module_requirements_json(handle))) != data["requirements"]:
        lib.th_module_free(handle)
        raise ValueError("artifact manifest differs from the loaded module")
    return LoadedModule(handle, data, req, d, fingerprint, world)
