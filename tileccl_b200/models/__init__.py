"""Model-level blocks built from the fused operators."""

from .tp_mlp import TPMLP, pack_gate_up, reference_forward

__all__ = ["TPMLP", "pack_gate_up", "reference_forward"]
