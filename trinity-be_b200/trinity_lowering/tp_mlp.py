"""Tensor-parallel SwiGLU MLP over a World:  Y = (silu(X Wg) * (X Wu)) Wd.

Each rank holds column shards of W_gate / W_up ([d_model, d_ff / n]) and the matching row shard
of W_down ([d_ff / n, d_model]); X is replicated.  Per step a rank launches
  1. the gated GEMM (two accumulators, SiLU-gate epilogue) -> H[M, d_ff / n] in BF16,
  2. the row-parallel down GEMM -> its partial Y[M, d_model] into a symmetric buffer,
  3. the peer-memory sum all-reduce of Y (skipped when the world has one rank),
all on one stream, with no host synchronisation in between.  With ``fused=True`` (the default)
steps 2 and 3 are one kernel: the down GEMM's epilogue warps exchange and add the partial tiles
over NVLink while the tensor cores work on the following tiles.
The plan-level spelling of the two GEMMs is `plans.gated_gemm` (a streamed, single-GPU plan per
rank) and `plans.row_parallel_gemm` (a multi-GPU plan: `all_reduce` of the accumulator), which the
provider emits as a persistent artifact whose one launch is the same fused kernel this class calls
directly; this class is the hand-written launch sequence over the kernel library.
"""
import torch

from . import kernels as k


class TensorParallelMLP:
    def __init__(self, world, m, d_model, d_ff, w_gate, w_up, w_down, device=None, fused=True):
        self.world = world
        self.size = world.size if world is not None else 1
        self.rank = world.rank if world is not None else 0
        if d_ff % self.size:
            raise ValueError("d_ff must divide by the world size")
        shard = d_ff // self.size
        for name, t, shape in (("w_gate", w_gate, (d_model, shard)), ("w_up", w_up, (d_model, shard)),
                               ("w_down", w_down, (shard, d_model))):
            if tuple(t.shape) != shape or t.dtype != torch.bfloat16 or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous bf16 shard of shape {shape}")
        self.m, self.d_model, self.shard = m, d_model, shard
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down
        device = device or w_gate.device
        self.hidden = torch.empty((m, shard), dtype=torch.bfloat16, device=device)
        self.fused = fused
        if world is not None and self.size > 1:
            self.buffer = world.allocate((m, d_model), torch.bfloat16,
                                         flag_words=k.gemm_allreduce_flag_words(m, d_model, self.size))
            self.output = self.buffer.tensor
        else:
            self.buffer = None
            self.output = torch.empty((m, d_model), dtype=torch.bfloat16, device=device)

    def forward(self, x, stream=None):
        """Launches the step on `stream` (default: current); returns the output tensor, which
        holds the all-reduced result once the stream has run."""
        k.gemm(x, self.w_up, b2=self.w_gate, activation=k.ACT_SILU_GATE, out=self.hidden, stream=stream)
        if self.fused is None:   # timing baseline only: per-rank partial, no exchange
            k.gemm(self.hidden, self.w_down, out=self.output, stream=stream)
            return self.output
        if self.buffer is not None and self.fused:
            self.world.gemm_all_reduce(self.hidden, self.w_down, self.buffer, stream=stream)
            return self.output
        k.gemm(self.hidden, self.w_down, out=self.output, stream=stream)
        if self.buffer is not None:
            self.world.all_reduce(self.buffer, stream=stream)
        return self.output

    @staticmethod
    def shard_weights(w_gate, w_up, w_down, rank, size):
        """Column shards of the gate / up projections and the row shard of the down projection."""
        shard = w_gate.shape[1] // size
        cols = slice(rank * shard, (rank + 1) * shard)
        return (w_gate[:, cols].contiguous(), w_up[:, cols].contiguous(), w_down[cols, :].contiguous())
