from .engine import ServingEngine, argmax_rows, sample_top_p_rows

__all__ = ["ServingEngine", "argmax_rows", "sample_top_p_rows"]
