"""Import shim for code written against the reference's `model.qwen_36` (model/qwen_36.py:172-184, 242-351).

The reference patches HuggingFace layers in place; here the model is an explicit executor, so only the helpers
that make sense on their own are re-exported: the INT8 weight format and the model classes."""
from tileinfer_b200.models.hybrid_b200 import B200HybridModel  # noqa: F401
from tileinfer_b200.models.reference_cpu import TorchHybridModel  # noqa: F401
from tileinfer_b200.models.weights import quantize_int8_rowwise


def quantize_weight_int8(weight):
    """Symmetric per-output-row INT8: returns (int8 weights, per-row scales) with scale = amax / 127, as the
    reference's function of the same name (rows are not padded here: the kernel layout pads when it tiles)."""
    return quantize_int8_rowwise(weight)
