"""B200 (sm_100a) implementation of the sparse message-passing operator library that sits under
Graphiler's MP-DFG compiler: SpMM, SDDMM, segment softmax, typed linear, broadcasts and the fused
attention operator, behind a C ABI (include/gphl.h) and the reference's TorchScript registrations."""
from .graph import GraphArrays, prepare_graph, attach_types, debug_graph, debug_hetero_graph  # noqa: F401

__all__ = ["GraphArrays", "prepare_graph", "attach_types", "debug_graph", "debug_hetero_graph"]
