"""drone_b200 — B200-native sparse aggregation for DRONE's EBV-partitioned graphs.

Host-side Python mirror of the C ABI (include/drone_b200.h).  torch is imported
first so that its bundled NCCL is the one the CUDA library binds to.
"""
import torch  # noqa: F401  (must precede loading libdrone_b200.so)

from ._lib import OP_A, OP_AT, PLAN_A, PLAN_AT, PLAN_BOTH, DroneError, lib  # noqa: F401
from .plan import AggregationPlan, compute_csr_values, degree_scales  # noqa: F401
from . import graphgen  # noqa: F401

__all__ = ["AggregationPlan", "compute_csr_values", "degree_scales", "graphgen", "lib", "DroneError",
           "OP_A", "OP_AT", "PLAN_A", "PLAN_AT", "PLAN_BOTH"]
