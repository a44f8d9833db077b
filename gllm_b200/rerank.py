"""Re-export of the rerank builder types (they live with the client that executes them)."""
from .client import *  # noqa: F401,F403
