from .config import Config
from .sampling_params import SamplingParams
from .sequence import Sequence, SequenceStatus

__all__ = ["Config", "SamplingParams", "Sequence", "SequenceStatus", "LLM"]


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM
        return LLM
    raise AttributeError(name)
