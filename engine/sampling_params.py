from tileinfer_b200.engine.sampling_params import SamplingParams  # noqa: F401
