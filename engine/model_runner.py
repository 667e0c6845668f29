from tileinfer_b200.engine.model_runner import *  # noqa: F401,F403
