"""Circuit tracing: node-labelled tensors, hooks that splice dictionaries into a model, attribution graphs."""

from .attribution import (
    AttributionResult,
    IntermediateRefs,
    NodeRefs,
    QKTracingResult,
    attribute,
    compute_hessian_matrix,
    compute_intermediates_attribution,
    get_normalized_matrix,
    prune_attribution,
    qk_trace,
)
from .hooks import apply_saes, detach_at, replace_model_biases_with_leaves, replace_sae_biases_with_leaves
from .indexed_tensor import NodeDimension, NodeIndexed, NodeIndexedMatrix, NodeIndexedTensor, NodeIndexedVector, NodeInfo

__all__ = [
    "AttributionResult", "IntermediateRefs", "NodeDimension", "NodeIndexed", "NodeIndexedMatrix", "NodeIndexedTensor",
    "NodeIndexedVector", "NodeInfo", "NodeRefs", "QKTracingResult", "apply_saes", "attribute", "compute_hessian_matrix",
    "compute_intermediates_attribution", "detach_at", "get_normalized_matrix", "prune_attribution", "qk_trace",
    "replace_model_biases_with_leaves", "replace_sae_biases_with_leaves",
]  # fmt: skip
