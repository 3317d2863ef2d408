"""B200-native provider for Trinity Lowering's CUDA path.

Host-side mirror of the reference's ``trinity_lowering`` package: plans are built with
``PhysicalPlanBuilder`` or ``lower_ir``, ``emit`` selects sm_100a kernels, ``compile`` builds a
``program.so`` with the five-symbol artifact ABI, ``load`` / ``prepare`` / ``run`` / ``Graph`` execute
it on PyTorch tensors.  ``trinity_lowering.kernels`` is the direct ctypes binding of the kernel
library (``include/trinity_sm100.h``).
"""
from . import kernels  # noqa: F401
from .compiler import (CompileConfig, CompileError, CudaArtifact, CudaSource, Implementation,
                       PhysicalPlan, PhysicalPlanBuilder, TritonProgram, all_gather_implementations,
                       broadcast_implementations, compile, emit, emit_python, emit_triton,
                       gemm_implementations, kernel_candidates, lower_ir, lower_triton,
                       pointwise_implementations, reduce_sum_implementations)
from .errors import DistributedFailure, ResourceBusy, RuntimeFailure
from .graph import Graph
from .runtime import IOBuffers, LoadedModule, PreparedExecution, load
from .world import World

__all__ = [
    "CompileConfig", "CompileError", "CudaArtifact", "CudaSource", "Implementation", "PhysicalPlan",
    "PhysicalPlanBuilder", "TritonProgram", "emit_python", "emit_triton", "lower_triton",
    "all_gather_implementations", "pointwise_implementations",
    "reduce_sum_implementations", "broadcast_implementations", "compile", "emit", "gemm_implementations",
    "kernel_candidates", "lower_ir", "DistributedFailure", "ResourceBusy", "RuntimeFailure", "Graph",
    "IOBuffers", "LoadedModule", "PreparedExecution", "load", "World", "kernels",
]
