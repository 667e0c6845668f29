from tileinfer_b200.engine.sequence import *  # noqa: F401,F403
