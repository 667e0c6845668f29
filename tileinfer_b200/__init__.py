"""tileinfer_b200: a Blackwell (sm_100a) inference engine for hybrid gated-DeltaNet + GQA models."""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name == "SamplingParams":
        from .engine.sampling_params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
