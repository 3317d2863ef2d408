"""One process per GPU: control plane over Gloo, data plane over NVLink peer-mapped memory.

Takes the role of the reference's NVSHMEM ``World`` (src/native/world.cpp,
python/src/trinity_lowering/world.py) without NVSHMEM:

* control plane (works on CPU ranks): a Gloo group for agreement.  Every collective-sensitive step
  runs through ``_stage``: ranks agree on the step's signature, run it, then exchange success or
  the failure text; if any rank failed, every rank raises ``DistributedFailure`` and the world is
  terminal (no re-formation), as in the reference.  A heartbeat on a store key lets ranks notice
  a peer that stopped between steps.
* data plane (needs GPUs): buffers from ``torch.distributed._symmetric_memory`` mapped into every
  rank's address space; collectives are this library's own kernels over plain peer loads and
  stores with bounded flag waits (``trinity_sm100_allreduce_bf16``).  NCCL is used only by the
  symmetric-memory rendezvous, never for the data path.  The kernels need no multicast object,
  and none is bound: TORCH_SYMM_MEM_DISABLE_MULTICAST=1 is set before the first rendezvous (a
  rank that died while its memory was bound to an NVLink multicast object could fault its peers).
"""
import os
import threading
import time

from .errors import DistributedFailure

# Read by torch's symmetric-memory allocator at its first rendezvous in the process.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class World:
    def __init__(self, group, rank, size, device=None, timeout=60.0, store=None):
        self._group, self.rank, self.size = group, rank, size
        self.device, self.timeout = device, timeout
        self._control_lock = threading.RLock()
        self._failed = None
        self._closed = False
        self._store = store
        self._stop = threading.Event()
        self._heartbeat = None
        self._epoch = 0
        self._buffers = []
        if store is not None:
            self._heartbeat = threading.Thread(target=self._beat, daemon=True)
            self._heartbeat.start()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_torchrun(cls, timeout=60.0, backend=None):
        """Builds the world from RANK / WORLD_SIZE / LOCAL_RANK (torchrun's environment)."""
        import torch
        import torch.distributed as dist
        rank = int(os.environ["RANK"])
        size = int(os.environ["WORLD_SIZE"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        use_cuda = torch.cuda.is_available()
        device = None
        if use_cuda:
            torch.cuda.set_device(local)
            device = torch.device("cuda", local)
        if not dist.is_initialized():
            chosen = backend or ("cpu:gloo,cuda:nccl" if use_cuda else "gloo")
            kwargs = {"device_id": device} if use_cuda else {}
            dist.init_process_group(chosen, **kwargs)
        control = dist.new_group(backend="gloo")
        store = dist.PrefixStore("trinity-world", dist.distributed_c10d._get_default_store())
        hosts = [None] * size
        dist.all_gather_object(hosts, os.uname().nodename, group=control)
        if len(set(hosts)) != 1:
            raise DistributedFailure("all ranks of a world must be on one host (one NVLink domain)")
        return cls(control, rank, size, device, timeout, store)

    # ------------------------------------------------------------------ control plane
    def _beat(self):
        while True:
            try:
                self._store.set(f"beat{self.rank}", str(time.time()))
            except Exception:
                return
            if self._stop.wait(min(1.0, self.timeout / 4)):
                return

    def check_peers(self):
        """Raises if a peer's heartbeat is older than the timeout."""
        if self._store is None:
            return
        now = time.time()
        for peer in range(self.size):
            if peer == self.rank:
                continue
            try:
                if not self._store.check([f"beat{peer}"]):
                    continue  # the peer has not published yet (a plain get would block)
                seen = float(self._store.get(f"beat{peer}"))
            except Exception:
                continue
            if now - seen > self.timeout:
                self._fail(f"rank {peer} stopped responding")
                raise DistributedFailure(self._failed)

    def _check(self):
        if self._closed:
            raise RuntimeError("world is closed")
        if self._failed:
            raise DistributedFailure(self._failed)

    def _fail(self, reason):
        if not self._failed:
            self._failed = reason

    def _exchange(self, name, value):
        import torch.distributed as dist
        out = [None] * self.size
        dist.all_gather_object(out, (name, value), group=self._group)
        names = {n for n, _ in out}
        if len(names) != 1:
            self._fail(f"ranks disagree on the step: {sorted(map(str, names))}")
            raise DistributedFailure(self._failed)
        return [v for _, v in out]

    def _stage(self, name, fn, signature=None):
        """Agree on (name, signature), run fn, agree on the outcome."""
        with self._control_lock:
            self._check()
            signatures = self._exchange(name + ".enter", signature)
            if any(s != signatures[0] for s in signatures):
                self._fail(f"ranks disagree on {name}")
                raise DistributedFailure(self._failed)
            error, result = None, None
            try:
                result = fn()
            except Exception as caught:  # reported to every rank below
                error = caught
            outcomes = self._exchange(name + ".exit", None if error is None else f"rank {self.rank}: {error}")
            failures = [o for o in outcomes if o is not None]
            if failures:
                self._fail(f"{name} failed: " + "; ".join(failures))
                if error is not None:
                    raise DistributedFailure(self._failed) from error
                raise DistributedFailure(self._failed)
            return result

    def barrier(self):
        self._stage("barrier", lambda: None)

    # ------------------------------------------------------------------ data plane
    def allocate(self, shape, dtype=None, flag_words=None):
        """A symmetric buffer: same shape on every rank, every rank's copy mapped everywhere.
        ``flag_words`` sizes the flag pad that travels with it (default: the all-reduce kernel's)."""
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch
        import torch.distributed._symmetric_memory as symm
        from . import kernels

        def make():
            tensor = symm.empty(*shape, dtype=dtype or torch.bfloat16, device=self.device)
            handle = symm.rendezvous(tensor, group=torch.distributed.group.WORLD)
            flags = symm.empty(max(flag_words or 0, kernels.allreduce_flag_words()), dtype=torch.int32,
                               device=self.device)
            flags.zero_()
            flag_handle = symm.rendezvous(flags, group=torch.distributed.group.WORLD)
            torch.cuda.synchronize(self.device)
            return SymmetricBuffer(self, tensor, list(handle.buffer_ptrs), flags, list(flag_handle.buffer_ptrs))

        buffer = self._stage("allocate", make, [list(shape), str(dtype), flag_words])
        self._stage("allocate.ready", lambda: None)
        self._buffers.append(buffer)
        return buffer

    def symmetric_buffer_of(self, tensor):
        """The symmetric allocation of this world that `tensor` is (same address and size), or None."""
        for buffer in self._buffers:
            if buffer.tensor.data_ptr() == tensor.data_ptr() and buffer.tensor.numel() * buffer.tensor.element_size() >= \
                    tensor.numel() * tensor.element_size():
                return buffer
        return None

    def record_stream(self, tensor):
        """Kept for the reference's surface (python/src/trinity_lowering/world.py): symmetric
        allocations of this world are owned by the world until `collect()` or `close()`, so there
        is no allocator stream to record."""
        return None

    def collect(self):
        """Releases symmetric allocations that nothing outside the world refers to any more.  A
        collective step: every rank calls it at the same point."""
        import sys

        def sweep():
            keep = [b for b in self._buffers if sys.getrefcount(b) > 3 or sys.getrefcount(b.tensor) > 2]
            dropped = len(self._buffers) - len(keep)
            self._buffers[:] = keep
            return dropped
        return self._stage("collect", sweep)

    def all_reduce(self, buffer, stream=None):
        """In-place sum all-reduce of a symmetric BF16 matrix through peer memory."""
        from . import kernels
        self._check()
        self._epoch += 1
        rows = buffer.tensor.shape[0] if buffer.tensor.dim() > 1 else 1
        cols = buffer.tensor.numel() // rows
        kernels.allreduce(buffer.peer_ptrs, buffer.flag_ptrs, rows, cols, self.rank, self._epoch, stream=stream)
        return buffer.tensor

    def gemm_all_reduce(self, a, b, buffer, stream=None):
        """buffer.tensor (on every rank) = sum over ranks of a @ b, reduced in the GEMM epilogue."""
        from . import kernels
        self._check()
        self._epoch += 1
        kernels.gemm_allreduce(a, b, buffer.tensor, buffer.peer_ptrs, buffer.flag_ptrs, self.rank,
                               self._epoch, stream=stream)
        return buffer.tensor

    def close(self):
        self._stop.set()
        self._closed = True
        self._buffers.clear()


class SymmetricBuffer:
    def __init__(self, world, tensor, peer_ptrs, flags, flag_ptrs):
        self.world, self.tensor, self.peer_ptrs = world, tensor, peer_ptrs
        self.flags, self.flag_ptrs = flags, flag_ptrs
