from tileinfer_b200.engine.block_manager import *  # noqa: F401,F403
