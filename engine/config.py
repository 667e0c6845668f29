from tileinfer_b200.engine.config import *  # noqa: F401,F403
