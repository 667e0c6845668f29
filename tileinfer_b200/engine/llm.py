"""`LLM`: the user-facing class (reference: engine/llm.py:18-24, an alias of the engine)."""
from .llm_engine import LLMEngine


class LLM(LLMEngine):
    pass
