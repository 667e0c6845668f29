from tileinfer_b200.engine.constraints import *  # noqa: F401,F403
