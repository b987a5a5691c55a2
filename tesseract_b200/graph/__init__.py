"""Graph IR: record eager code into an SSA ``Graph`` (``GraphScope``), replay it (``run``, ``GraphExecutor`` with
CUDA-graph replay on a GPU), differentiate it as a graph transform (``build_backward``), and print / read it as
``tesseract``-dialect text (``emit_mlir`` / ``parse_mlir``). The role of the reference's C++ graph layer
(include/tesseract/graph/*.hpp, src/graph/*.cpp); its MLIR passes and JIT engines (src/ir) are not part of this
framework.
"""
from .autograd import BackwardResult, build_backward, differentiable_ops
from .interpreter import GraphExecutor, reduce_to_shape, run, supported_ops
from .ir import Graph, Op, Value, ValueId, ValueKind, kInvalidValueId
from .mlir import emit_mlir, parse_mlir
from .scope import GraphScope, active_scope, is_recording, maybe_record
from .train import GraphTrainStep

__all__ = ["Graph", "Op", "Value", "ValueId", "ValueKind", "kInvalidValueId", "GraphScope", "active_scope",
           "is_recording", "maybe_record", "run", "GraphExecutor", "reduce_to_shape", "supported_ops",
           "build_backward", "BackwardResult", "differentiable_ops", "emit_mlir", "parse_mlir", "GraphTrainStep"]
