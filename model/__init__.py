"""Import shim: the reference keeps its model code in a top-level `model` package (model/qwen_36.py,
model/generate.py).  The implementation lives in `tileinfer_b200.models`."""
