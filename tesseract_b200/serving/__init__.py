from .engine import ServingEngine, TPServe, argmax_rows, sample_rows, sample_top_p_rows
from .replicas import ReplicaPlan, default_tp, make_replica_plan, split_requests

__all__ = ["ServingEngine", "TPServe", "argmax_rows", "sample_rows", "sample_top_p_rows", "ReplicaPlan", "default_tp",
           "make_replica_plan", "split_requests"]
