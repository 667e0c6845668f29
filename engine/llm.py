from tileinfer_b200.engine.llm import LLM  # noqa: F401
