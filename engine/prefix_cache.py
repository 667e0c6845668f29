from tileinfer_b200.engine.prefix_cache import *  # noqa: F401,F403
