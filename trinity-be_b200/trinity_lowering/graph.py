"""CUDA-Graph capture and replay of prepared executions."""
import ctypes

from . import _host as h
from .errors import ResourceBusy


class Graph:
    def __init__(self, handle, executions, stream, output):
        self._handle, self._executions, self._stream, self._output = handle, list(executions), stream, output
        self._closed = False

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        try:
            if handle:
                h.library().th_graph_free(handle)
        except Exception:  # interpreter shutdown: the library wrapper is already gone
            pass  # pending replays are handed to the retire queue

    @property
    def output(self):
        return self._output

    @classmethod
    def capture(cls, fn, executions, stream=None, warmup=3):
        """Runs ``fn`` ``warmup`` times on ``stream``, then once more under stream capture.
        ``fn`` must launch every execution of ``executions`` (and nothing that allocates)."""
        import torch
        executions = list(executions)
        if not executions:
            raise ValueError("at least one execution is required")
        device = executions[0].module.device
        if stream is None:
            stream = torch.cuda.current_stream(device)
        if stream == torch.cuda.default_stream(device) or stream.cuda_stream == 0:
            raise ValueError("graph capture needs a non-default stream")
        with torch.cuda.device(device):
            if torch.cuda.is_current_stream_capturing():
                raise ResourceBusy("a capture is already active on this thread")
        for e in executions:
            e._validate()
        lib = h.library()
        pointers = (ctypes.c_void_p * len(executions))(*[e._handle for e in executions])
        handle = h.check_ptr(lib.th_graph_create(pointers, len(executions), device.index))
        raw = ctypes.c_void_p(stream.cuda_stream)
        result = None
        try:
            with torch.cuda.stream(stream):
                for _ in range(warmup):
                    if lib.th_graph_begin(handle, raw, 0) != 0:
                        h.raise_last()
                    try:
                        fn()
                    finally:
                        if lib.th_graph_end_warmup(handle) != 0:
                            h.raise_last()
                if lib.th_graph_begin(handle, raw, 1) != 0:
                    h.raise_last()
                try:
                    result = fn()
                except BaseException:
                    lib.th_graph_abort(handle)
                    raise
                if lib.th_graph_end_capture(handle) != 0:
                    h.raise_last()
        except BaseException:
            lib.th_graph_close(handle)
            lib.th_graph_free(handle)
            raise
        return cls(handle, executions, stream, result if result is not None else executions[-1].output)

    def replay(self, stream=None):
        import torch
        if self._closed:
            raise RuntimeError("graph is closed")
        for e in self._executions:
            e._validate()
        st = stream if stream is not None else torch.cuda.current_stream(self._executions[0].module.device)
        if h.library().th_graph_replay(self._handle, ctypes.c_void_p(st.cuda_stream)) != 0:
            h.raise_last()
        return self._output

    def wait(self, timeout=None):
        if self._closed:
            return
        if h.library().th_graph_wait(self._handle, -1.0 if timeout is None else float(timeout)) != 0:
            h.raise_last()

    def close(self):
        if not self._closed:
            if h.library().th_graph_close(self._handle) != 0:
                h.raise_last()
            self._closed = True
