"""Visual-builder core: block graphs (``.tsb``), the block catalog, static analysis with shape inference, source
generation, and an executor that trains / generates / evaluates what the graph describes
(the reference's studio/core). ``python -m tesseract_b200.studio.server`` serves the same functions over HTTP as a
JSON API with a small page on top.
"""
from .analysis import AnalysisResult, Diagnostic, analyze
from .catalog import BlockCatalog, BlockSpec, ParamSpec, PortSpec
from .codegen import extract_tsb, generate_ir, generate_python
from .executor import Executor, RunEvent, RunOptions
from .graph import BlockGraph, Edge, Endpoint, Node, PortType

__all__ = ["AnalysisResult", "Diagnostic", "analyze", "BlockCatalog", "BlockSpec", "ParamSpec", "PortSpec", "extract_tsb",
           "generate_ir", "generate_python", "Executor", "RunEvent", "RunOptions", "BlockGraph", "Edge", "Endpoint", "Node",
           "PortType"]
