from .engine import ServingEngine, TPServe, argmax_rows, sample_top_p_rows

__all__ = ["ServingEngine", "TPServe", "argmax_rows", "sample_top_p_rows"]
