from tileinfer_b200.engine.scheduler import *  # noqa: F401,F403
