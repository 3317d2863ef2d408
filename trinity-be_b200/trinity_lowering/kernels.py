"""ctypes binding of the sm_100a kernel library (``include/trinity_sm100.h``).

This is the only route from Python to the CUDA kernels.  There is no CPU or PyTorch
fallback: when the shared library is missing or a call fails, an exception is raised.
PyTorch tensors are used for device memory and streams only; the C ABI sees raw pointers.
"""
import ctypes
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parents[1] / "lib" / "libtrinity_sm100.so"

BIAS_NONE, BIAS_COL_VECTOR, BIAS_ROW_VECTOR, BIAS_MATRIX = 0, 1, 2, 3
ACT_NONE, ACT_RELU, ACT_SILU, ACT_SILU_GATE = 0, 1, 2, 3
DT_BF16, DT_FP32 = 0, 1

EXPORTS = (
    "trinity_sm100_gemm_bf16",
    "trinity_sm100_gemm_batched_bf16",
    "trinity_sm100_gemm_pair_capacity",
    "trinity_sm100_rmsnorm_bf16",
    "trinity_sm100_softmax_bf16",
    "trinity_sm100_mla_scratch_bytes",
    "trinity_sm100_mla_default_splits",
    "trinity_sm100_mla_balanced_slots",
    "trinity_sm100_mla_schedule",
    "trinity_sm100_mla_schedule_segment",
    "trinity_sm100_mla_decode_bf16",
    "trinity_sm100_mla_decode_bf16_noalloc",
    "trinity_sm100_allreduce_flag_words",
    "trinity_sm100_allreduce_bf16",
    "trinity_sm100_allgather_bf16",
    "trinity_sm100_gemm_allreduce_flag_words",
    "trinity_sm100_gemm_allreduce_bf16",
    "trinity_sm100_gemm_allreduce_stamps",
    "trinity_sm100_gemm_allreduce_workspace_bytes",
    "trinity_sm100_gemm_allreduce_workspace_bf16",
    "trinity_sm100_pointwise",
    "trinity_sm100_row_reduce_sum",
    "trinity_sm100_prepare_device",
    "trinity_sm100_current_device",
    "trinity_sm100_stream_synchronize",
    "trinity_sm100_device_status",
    "trinity_sm100_set_wait_budget",
    "trinity_sm100_abi_version",
    "trinity_sm100_last_error",
    "trinity_sm100_launch_count",
)


class KernelError(RuntimeError):
    """A kernel-library call returned a non-zero code."""

    def __init__(self, code, message):
        super().__init__(f"trinity_sm100 error {code}: {message}")
        self.code = code


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("b2", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldo", ctypes.c_int64),
        ("ld_bias", ctypes.c_int64),
        ("bias_mode", ctypes.c_int32), ("activation", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class GemmBatchArgs(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int64), ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64),
                ("stride_out", ctypes.c_int64), ("stride_bias", ctypes.c_int64)]


class MlaArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("cache", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seq", ctypes.c_int32),
        ("d_qk", ctypes.c_int32), ("d_v", ctypes.c_int32), ("kv_splits", ctypes.c_int32),
        ("scale", ctypes.c_float), ("reserved", ctypes.c_int32),
    ]


class AllReduceArgs(ctypes.Structure):
    _fields_ = [
        ("peers", ctypes.POINTER(ctypes.c_void_p)), ("flags", ctypes.POINTER(ctypes.c_void_p)),
        ("rows", ctypes.c_int64), ("cols", ctypes.c_int64),
        ("world", ctypes.c_int32), ("rank", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("reserved", ctypes.c_int32),
    ]


_lock = threading.Lock()
_lib = None


def library_path():
    return _LIB_PATH


def library():
    """Loads the kernel library once; raises if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise RuntimeError(
                    f"{_LIB_PATH} is missing: build it with `python -m __graft_entry__` "
                    "(there is no fallback path)")
            lib = ctypes.CDLL(str(_LIB_PATH))
            lib.trinity_sm100_gemm_bf16.argtypes = [ctypes.POINTER(GemmArgs), ctypes.c_void_p]
            lib.trinity_sm100_rmsnorm_bf16.argtypes = [
                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                ctypes.c_float, ctypes.c_void_p]
            lib.trinity_sm100_softmax_bf16.argtypes = [
                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
            lib.trinity_sm100_mla_scratch_bytes.argtypes = [ctypes.c_int32] * 4
            lib.trinity_sm100_mla_scratch_bytes.restype = ctypes.c_size_t
            lib.trinity_sm100_mla_default_splits.argtypes = [ctypes.c_int32] * 2
            lib.trinity_sm100_mla_balanced_slots.argtypes = [ctypes.c_int32] * 2
            lib.trinity_sm100_mla_decode_bf16.argtypes = [ctypes.POINTER(MlaArgs), ctypes.c_void_p]
            lib.trinity_sm100_mla_decode_bf16_noalloc.argtypes = [
                ctypes.POINTER(MlaArgs), ctypes.c_void_p]
            lib.trinity_sm100_allreduce_flag_words.restype = ctypes.c_size_t
            lib.trinity_sm100_allreduce_bf16.argtypes = [
                ctypes.POINTER(AllReduceArgs), ctypes.c_void_p]
            lib.trinity_sm100_allgather_bf16.argtypes = [
                ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
            lib.trinity_sm100_gemm_allreduce_flag_words.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int32]
            lib.trinity_sm100_gemm_allreduce_flag_words.restype = ctypes.c_size_t
            lib.trinity_sm100_gemm_allreduce_bf16.argtypes = [
                ctypes.POINTER(GemmArgs), ctypes.POINTER(AllReduceArgs), ctypes.c_void_p]
            lib.trinity_sm100_device_status.argtypes = [
                ctypes.POINTER(ctypes.c_uint32), ctypes.c_int]
            lib.trinity_sm100_set_wait_budget.argtypes = [ctypes.c_uint64]
            lib.trinity_sm100_last_error.restype = ctypes.c_char_p
            lib.trinity_sm100_launch_count.restype = ctypes.c_uint64
            _lib = lib
    return _lib


def _check(code):
    if code != 0:
        raise KernelError(code, library().trinity_sm100_last_error().decode())


def _stream(stream=None):
    if stream is None:
        stream = torch.cuda.current_stream()
    return ctypes.c_void_p(stream.cuda_stream)


def _require(t, dtype, name):
    if not t.is_cuda or t.dtype != dtype:
        raise ValueError(f"{name}: expected a CUDA tensor of {dtype}, got {t.device} {t.dtype}")


def launch_count():
    return int(library().trinity_sm100_launch_count())


def device_status(clear=False):
    value = ctypes.c_uint32(0)
    _check(library().trinity_sm100_device_status(ctypes.byref(value), int(clear)))
    return value.value


def gemm_pair_capacity():
    """CTA pairs the current device keeps resident at once in the GEMM's pair mode."""
    value = ctypes.c_int32(0)
    _check(library().trinity_sm100_gemm_pair_capacity(ctypes.byref(value)))
    return value.value


def set_wait_budget(cycles):
    """Budget of every bounded in-kernel wait on the current device, in SM clock cycles
    (0 restores the default of about two seconds)."""
    _check(library().trinity_sm100_set_wait_budget(int(cycles)))


def gemm(a, b, *, bias=None, bias_mode=None, activation=ACT_NONE, b2=None, out=None,
         out_dtype=torch.bfloat16, stream=None):
    """out = act(a @ b + bias); see ``trinity_sm100_gemm_bf16``.  Row-major 2-D tensors."""
    _require(a, torch.bfloat16, "a")
    _require(b, torch.bfloat16, "b")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("gemm: a must be [m,k] and b [k,n]")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("gemm: operands must be row-major with unit inner stride")
    m, k = a.shape
    n = b.shape[1]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if out.shape != (m, n) or out.stride(1) != 1:
        raise ValueError("gemm: out must be a row-major [m,n] tensor")
    args = GemmArgs()
    args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k = m, n, k
    args.lda, args.ldb, args.ldo = a.stride(0), b.stride(0), out.stride(0)
    args.activation = activation
    args.out_dtype = DT_FP32 if out.dtype == torch.float32 else DT_BF16
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("gemm: out dtype must be bf16 or fp32")
    if b2 is not None:
        _require(b2, torch.bfloat16, "b2")
        if b2.shape != b.shape or b2.stride() != b.stride():
            raise ValueError("gemm: b2 must match b")
        args.b2 = b2.data_ptr()
    if bias is not None:
        _require(bias, torch.bfloat16, "bias")
        if bias_mode is None:
            bias_mode = BIAS_MATRIX if bias.dim() == 2 else BIAS_COL_VECTOR
        expected = {BIAS_COL_VECTOR: (n,), BIAS_ROW_VECTOR: (m,), BIAS_MATRIX: (m, n)}[bias_mode]
        if tuple(bias.shape) != expected or bias.stride(-1) != 1:
            raise ValueError(f"gemm: bias shape {tuple(bias.shape)} does not fit mode {bias_mode}")
        args.bias = bias.data_ptr()
        args.ld_bias = bias.stride(0) if bias.dim() == 2 else 0
        args.bias_mode = bias_mode
    with torch.cuda.device(a.device):
        _check(library().trinity_sm100_gemm_bf16(ctypes.byref(args), _stream(stream)))
    return out


def gemm_batched(a, b, *, bias=None, activation=ACT_NONE, out=None, out_dtype=torch.bfloat16, stream=None):
    """out[z] = act(a[z] @ b[z] + bias[z]) for every batch entry z in one launch; see
    ``trinity_sm100_gemm_batched_bf16``.  ``a`` is [batch, m, k] and ``out`` [batch, m, n], any
    strides with a unit inner stride (so ``x.permute(1, 0, 2)`` of a [tokens, heads, k] tensor is
    fine); ``b`` is [batch, k, n] or a shared [k, n]; ``bias`` is [batch, n] or a shared [n]."""
    _require(a, torch.bfloat16, "a")
    _require(b, torch.bfloat16, "b")
    if a.dim() != 3 or b.dim() not in (2, 3) or a.shape[2] != b.shape[-2] or a.stride(2) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm_batched: a must be [batch,m,k], b [batch,k,n] or [k,n], unit inner strides")
    batch, m, k = a.shape
    n = b.shape[-1]
    if b.dim() == 3 and b.shape[0] != batch:
        raise ValueError("gemm_batched: a and b disagree on the batch")
    if out is None:
        out = torch.empty((batch, m, n), dtype=out_dtype, device=a.device)
    if tuple(out.shape) != (batch, m, n) or out.stride(2) != 1 or out.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("gemm_batched: out must be [batch,m,n] with a unit inner stride, bf16 or fp32")
    args = GemmArgs()
    args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k = m, n, k
    args.lda, args.ldb, args.ldo = a.stride(1), b.stride(-2), out.stride(1)
    args.activation = activation
    args.out_dtype = DT_FP32 if out.dtype == torch.float32 else DT_BF16
    how = GemmBatchArgs()
    how.batch = batch
    how.stride_a, how.stride_out = a.stride(0), out.stride(0)
    how.stride_b = b.stride(0) if b.dim() == 3 else 0
    if bias is not None:
        _require(bias, torch.bfloat16, "bias")
        if tuple(bias.shape) not in ((n,), (batch, n)) or bias.stride(-1) != 1:
            raise ValueError("gemm_batched: bias must be [n] or [batch,n]")
        args.bias = bias.data_ptr()
        args.bias_mode = BIAS_COL_VECTOR
        how.stride_bias = bias.stride(0) if bias.dim() == 2 else 0
    with torch.cuda.device(a.device):
        _check(library().trinity_sm100_gemm_batched_bf16(ctypes.byref(args), ctypes.byref(how), _stream(stream)))
    return out


def rmsnorm(x, gain=None, eps=0.0, out=None, stream=None):
    _require(x, torch.bfloat16, "x")
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("rmsnorm: x must be a contiguous [rows, cols] tensor")
    if out is None:
        out = torch.empty_like(x)
    if gain is not None:
        _require(gain, torch.bfloat16, "gain")
        if tuple(gain.shape) != (x.shape[1],) or not gain.is_contiguous():
            raise ValueError("rmsnorm: gain must be [cols]")
    with torch.cuda.device(x.device):
        _check(library().trinity_sm100_rmsnorm_bf16(
            x.data_ptr(), gain.data_ptr() if gain is not None else None, out.data_ptr(),
            x.shape[0], x.shape[1], float(eps), _stream(stream)))
    return out


def softmax(x, out=None, stream=None):
    _require(x, torch.bfloat16, "x")
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("softmax: x must be a contiguous [rows, cols] tensor")
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _check(library().trinity_sm100_softmax_bf16(
            x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _stream(stream)))
    return out


def mla_default_splits(batch, seq):
    return int(library().trinity_sm100_mla_default_splits(batch, seq))


def mla_balanced_slots(batch, seq):
    return int(library().trinity_sm100_mla_balanced_slots(batch, seq))


def mla_scratch_bytes(batch, heads, d_v, kv_splits):
    return int(library().trinity_sm100_mla_scratch_bytes(batch, heads, d_v, kv_splits))


def mla_decode(q, cache, scale, d_v=512, kv_splits=0, out=None, scratch=None, stream=None):
    """out[b,h,:] = softmax_s(scale * q[b,h] . cache[b,s]) @ cache[b,:,:d_v]."""
    _require(q, torch.bfloat16, "q")
    _require(cache, torch.bfloat16, "cache")
    if q.dim() != 3 or cache.dim() != 3 or not q.is_contiguous() or not cache.is_contiguous():
        raise ValueError("mla_decode: q [batch,heads,d_qk] and cache [batch,seq,d_qk], contiguous")
    batch, heads, d_qk = q.shape
    if cache.shape[0] != batch or cache.shape[2] != d_qk:
        raise ValueError("mla_decode: q and cache disagree on batch or width")
    seq = cache.shape[1]
    if out is None:
        out = torch.empty((batch, heads, d_v), dtype=torch.bfloat16, device=q.device)
    # kv_splits == 0 leaves the schedule to the library, kv_splits < 0 asks for the balanced one;
    # either way the library says how many partial slots per sequence it needs scratch for.
    slots = kv_splits if kv_splits > 0 else (
        mla_default_splits(batch, seq) if kv_splits == 0 else mla_balanced_slots(batch, seq))
    need = mla_scratch_bytes(batch, heads, d_v, slots)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    args = MlaArgs()
    args.q, args.cache, args.out = q.data_ptr(), cache.data_ptr(), out.data_ptr()
    args.scratch, args.scratch_bytes = scratch.data_ptr(), scratch.numel() * scratch.element_size()
    args.batch, args.heads, args.seq, args.d_qk, args.d_v = batch, heads, seq, d_qk, d_v
    args.kv_splits = kv_splits
    args.scale = float(scale)
    with torch.cuda.device(q.device):
        _check(library().trinity_sm100_mla_decode_bf16(ctypes.byref(args), _stream(stream)))
    return out


MLA_STATIC_SCRATCH_BYTES = 32 << 20


def mla_decode_noalloc(q, cache, scale, d_v=512, kv_splits=0, out=None, stream=None):
    """``mla_decode`` for callers that cannot bring or allocate scratch memory: the split
    partials live in a fixed array inside the kernel library (``MLA_STATIC_SCRATCH_BYTES`` per
    GPU).  ``out`` must be passed by such callers; it is created here only as a convenience for
    tests.  Calls that overlap on one GPU race on the shared array."""
    _require(q, torch.bfloat16, "q")
    _require(cache, torch.bfloat16, "cache")
    if q.dim() != 3 or cache.dim() != 3 or not q.is_contiguous() or not cache.is_contiguous():
        raise ValueError("mla_decode: q [batch,heads,d_qk] and cache [batch,seq,d_qk], contiguous")
    batch, heads, d_qk = q.shape
    if cache.shape[0] != batch or cache.shape[2] != d_qk:
        raise ValueError("mla_decode: q and cache disagree on batch or width")
    if out is None:
        out = torch.empty((batch, heads, d_v), dtype=torch.bfloat16, device=q.device)
    args = MlaArgs()
    args.q, args.cache, args.out = q.data_ptr(), cache.data_ptr(), out.data_ptr()
    args.batch, args.heads, args.seq, args.d_qk, args.d_v = batch, heads, cache.shape[1], d_qk, d_v
    args.kv_splits = kv_splits
    args.scale = float(scale)
    with torch.cuda.device(q.device):
        _check(library().trinity_sm100_mla_decode_bf16_noalloc(ctypes.byref(args), _stream(stream)))
    return out


def allreduce_flag_words():
    return int(library().trinity_sm100_allreduce_flag_words())


def allreduce(peer_ptrs, flag_ptrs, rows, cols, rank, epoch, stream=None):
    """In-place sum all-reduce over peer-mapped BF16 buffers (see the C header)."""
    world = len(peer_ptrs)
    peers = (ctypes.c_void_p * world)(*peer_ptrs)
    flags = (ctypes.c_void_p * world)(*flag_ptrs)
    args = AllReduceArgs()
    args.peers = ctypes.cast(peers, ctypes.POINTER(ctypes.c_void_p))
    args.flags = ctypes.cast(flags, ctypes.POINTER(ctypes.c_void_p))
    args.rows, args.cols, args.world, args.rank, args.epoch = rows, cols, world, rank, epoch
    _check(library().trinity_sm100_allreduce_bf16(ctypes.byref(args), _stream(stream)))


PEER_TABLE_BYTES = 1024
PEER_BUFFERS = 4


def peer_table(world, rank, workspace_ptrs, buffer_ptrs):
    """The bytes of a ``trinity_sm100_peer_table`` (see the C header): ``workspace_ptrs[r]`` is
    rank r's workspace as mapped into this process, ``buffer_ptrs[i][r]`` rank r's copy of the
    i-th symmetric plan buffer."""
    import struct
    if len(buffer_ptrs) > PEER_BUFFERS or world > 8:
        raise ValueError("at most %d symmetric buffers and 8 ranks" % PEER_BUFFERS)
    words = struct.pack("<iiIIIIII", world, rank, 0, 0, 0, 0, 0, 0)
    words += struct.pack("<8Q", *(list(workspace_ptrs) + [0] * (8 - world)))
    for i in range(PEER_BUFFERS):
        ptrs = list(buffer_ptrs[i]) if i < len(buffer_ptrs) else []
        words += struct.pack("<8Q", *(ptrs + [0] * (8 - len(ptrs))))
    words += bytes(64 * 4)
    return words + bytes(PEER_TABLE_BYTES - len(words))


def allgather(workspace_ptr, source, out, rows, cols, axis, world, stream=None):
    """out = rank-major all-gather of the [rows, cols] BF16 shards held in symmetric buffer
    ``source`` of the peer table at ``workspace_ptr`` (see ``trinity_sm100_allgather_bf16``)."""
    _require(out, torch.bfloat16, "out")
    with torch.cuda.device(out.device):
        _check(library().trinity_sm100_allgather_bf16(ctypes.c_void_p(workspace_ptr), source, out.data_ptr(),
                                                      rows, cols, axis, world, _stream(stream)))
    return out


def gemm_allreduce_stamps():
    """Milestones (ns of the device timer) of the most recent fused launch's first thread block:
    start, last MMA committed, last partial tile handed over, last owned rows reduced, retired."""
    values = (ctypes.c_uint64 * 5)()
    _check(library().trinity_sm100_gemm_allreduce_stamps(values))
    return list(values)


def gemm_allreduce_flag_words(m, n, world):
    return int(library().trinity_sm100_gemm_allreduce_flag_words(m, n, world))


def gemm_allreduce(a, b, out, peer_ptrs, flag_ptrs, rank, epoch, stream=None):
    """out (on every rank) = sum over ranks of a_rank @ b_rank, reduced inside the GEMM's
    epilogue over peer-mapped memory (see ``trinity_sm100_gemm_allreduce_bf16``).  ``out`` is this
    rank's symmetric buffer, ``peer_ptrs[rank] == out.data_ptr()``."""
    _require(a, torch.bfloat16, "a")
    _require(b, torch.bfloat16, "b")
    _require(out, torch.bfloat16, "out")
    m, kk = a.shape
    n = b.shape[1]
    args = GemmArgs()
    args.a, args.b, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.m, args.n, args.k = m, n, kk
    args.lda, args.ldb, args.ldo = a.stride(0), b.stride(0), out.stride(0)
    world = len(peer_ptrs)
    peers = (ctypes.c_void_p * world)(*peer_ptrs)
    flags = (ctypes.c_void_p * world)(*flag_ptrs)
    red = AllReduceArgs()
    red.peers = ctypes.cast(peers, ctypes.POINTER(ctypes.c_void_p))
    red.flags = ctypes.cast(flags, ctypes.POINTER(ctypes.c_void_p))
    red.rows, red.cols, red.world, red.rank, red.epoch = m, n, world, rank, epoch
    with torch.cuda.device(a.device):
        _check(library().trinity_sm100_gemm_allreduce_bf16(ctypes.byref(args), ctypes.byref(red),
                                                           _stream(stream)))
    return out
