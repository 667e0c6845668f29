from tileinfer_b200.engine.llm_engine import *  # noqa: F401,F403
