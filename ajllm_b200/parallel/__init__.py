"""Parallel runtime: process mesh, tensor / expert / pipeline / fully-sharded data parallelism, symmetric memory."""

from ajllm_b200.parallel.context_parallel import ContextParallel
from ajllm_b200.parallel.mesh import AxisGroup, ParallelMesh, init_distributed
from ajllm_b200.parallel.pipeline import PipelineOptimizer, PipelineParallel, pp_optimizer_classes
from ajllm_b200.parallel.tensor_parallel import TensorParallel, tp_optimizer_classes

__all__ = ["ContextParallel", "AxisGroup", "ParallelMesh", "init_distributed", "TensorParallel", "tp_optimizer_classes",
           "PipelineParallel", "PipelineOptimizer", "pp_optimizer_classes"]
