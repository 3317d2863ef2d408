"""ctypes binding of the C++ host library (``include/trinity_host.h``): planner, emitter,
artifact builder and runtime.  Failing calls are turned into the exceptions the reference's
Python package raises."""
import ctypes
import json
import threading
from pathlib import Path

from .errors import CompileError, ResourceBusy, RuntimeFailure

_ROOT = Path(__file__).resolve().parents[1]
_LIB_PATH = _ROOT / "lib" / "libtrinity_host.so"
_lock = threading.Lock()
_lib = None

P = ctypes.c_void_p
S = ctypes.c_char_p
I = ctypes.c_int
I64P = ctypes.POINTER(ctypes.c_int64)
IP = ctypes.POINTER(ctypes.c_int)

_SIGNATURES = {
    "th_last_error_kind": (I, []),
    "th_last_error_message": (S, []),
    "th_last_error_info": (None, [ctypes.POINTER(ctypes.c_int32)]),
    "th_last_error_diagnostics": (S, []),
    "th_configure": (None, [S, S]),
    "th_builder_new": (P, [I, S]),
    "th_builder_free": (None, [P]),
    "th_builder_add_value": (I, [P, S, I64P, I, S, S]),
    "th_builder_bind_input": (I, [P, S, I]),
    "th_builder_add_operation": (I, [P, IP, I, IP, I, S]),
    "th_builder_add_loop": (I, [P, S, S, S, S, S, IP, I]),
    "th_builder_build": (P, [P, IP, I, S, I]),
    "th_plan_free": (None, [P]),
    "th_plan_metadata_json": (S, [P]),
    "th_plan_symbols_json": (S, [P]),
    "th_plan_structure": (S, [P]),
    "th_plan_hash": (ctypes.c_uint64, [P]),
    "th_plan_world_size": (I, [P]),
    "th_plan_bind_symbols": (P, [P, ctypes.POINTER(S), I64P, I]),
    "th_lower_ir": (I, [S, ctypes.POINTER(S), I64P, I, ctypes.POINTER(S), ctypes.POINTER(S), I, S, I,
                        ctypes.POINTER(P), I]),
    "th_emit": (P, [P]),
    "th_source_free": (None, [P]),
    "th_source_code": (S, [P]),
    "th_source_requirements_json": (S, [P]),
    "th_source_launch_count": (I, [P]),
    "th_kernel_candidates_json": (S, [P]),
    "th_compile": (P, [P, S, S]),
    "th_artifact_free": (None, [P]),
    "th_artifact_directory": (S, [P]),
    "th_artifact_path": (S, [P]),
    "th_artifact_manifest_json": (S, [P]),
    "th_artifact_diagnostics_json": (S, [P]),
    "th_artifact_code": (S, [P]),
    "th_artifact_close": (I, [P]),
    "th_artifact_persist": (S, [P]),
    "th_library_probe": (S, [S, I]),
    "th_module_load": (P, [S, I, I]),
    "th_module_free": (None, [P]),
    "th_module_requirements_json": (S, [P]),
    "th_module_prepare": (I, [P, ctypes.POINTER(ctypes.c_uint)]),
    "th_module_close": (I, [P]),
    "th_module_live_executions": (I, [P]),
    "th_execution_create": (P, [P, ctypes.POINTER(P), ctypes.c_size_t, P]),
    "th_execution_create_persistent": (P, [P, ctypes.POINTER(P), ctypes.c_size_t, P, ctypes.c_size_t,
                                           ctypes.c_uint, P]),
    "th_execution_free": (None, [P]),
    "th_execution_run": (I, [P, P]),
    "th_execution_wait": (I, [P, ctypes.c_double]),
    "th_execution_close": (I, [P, I]),
    "th_execution_closed": (I, [P]),
    "th_graph_create": (P, [ctypes.POINTER(P), ctypes.c_size_t, I]),
    "th_graph_free": (None, [P]),
    "th_graph_begin": (I, [P, P, I]),
    "th_graph_end_warmup": (I, [P]),
    "th_graph_end_capture": (I, [P]),
    "th_graph_abort": (I, [P]),
    "th_graph_replay": (I, [P, P]),
    "th_graph_wait": (I, [P, ctypes.c_double]),
    "th_graph_close": (I, [P]),
    "th_collect_local": (ctypes.c_size_t, []),
    "th_retire_pending": (ctypes.c_size_t, []),
    "th_cuda_runtime_version": (I, []),
}
EXPORTS = tuple(_SIGNATURES)


def library():
    global _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise RuntimeError(f"{_LIB_PATH} is missing: build it with `python -m __graft_entry__`")
            lib = ctypes.CDLL(str(_LIB_PATH))
            for name, (restype, argtypes) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = restype, argtypes
            lib.th_configure(str(_ROOT.parent / "include").encode(), str(_ROOT / "lib").encode())
            _lib = lib
    return _lib


def raise_last():
    lib = library()
    kind = lib.th_last_error_kind()
    message = (lib.th_last_error_message() or b"").decode(errors="replace")
    if kind == 1:
        raise ValueError(message)
    if kind == 2:
        raise NotImplementedError(message)
    if kind == 4:
        raise TypeError(message)
    if kind == 5:
        info = (ctypes.c_int32 * 6)()
        lib.th_last_error_info(info)
        raise RuntimeFailure(message, *list(info))
    if kind == 6:
        raise ResourceBusy(message)
    if kind == 7:
        text = (lib.th_last_error_diagnostics() or b"").decode(errors="replace")
        raise CompileError(message, json.loads(text) if text else None)
    raise RuntimeError(message)


def check_ptr(value):
    if not value:
        raise_last()
    return value


def check_int(value):
    if value < 0:
        raise_last()
    return value


def text(value):
    return (value or b"").decode()


def int_array(values):
    values = list(values)
    return (ctypes.c_int * max(1, len(values)))(*values), len(values)
