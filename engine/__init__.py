"""Import-compatibility package: `from engine.llm import LLM` as with the reference."""
