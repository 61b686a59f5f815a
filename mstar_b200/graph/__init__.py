from .ir import (EMIT_TO_CLIENT, EMPTY_DESTINATION, GraphEdge, GraphNode, GraphSection, Loop, Parallel, Sequential,
                 TensorPointerInfo)
from .walk_state import Completion, WalkState

__all__ = ["EMIT_TO_CLIENT", "EMPTY_DESTINATION", "GraphEdge", "GraphNode", "GraphSection", "Loop", "Parallel",
           "Sequential", "TensorPointerInfo", "Completion", "WalkState"]
