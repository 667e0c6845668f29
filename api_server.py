"""Entry point kept at the repository root like the reference's api_server.py."""
from tileinfer_b200.server.api_server import main

if __name__ == "__main__":
    main()
