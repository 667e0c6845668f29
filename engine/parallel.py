from tileinfer_b200.parallel.comm import init_distributed, get_comm, shutdown_distributed  # noqa: F401
