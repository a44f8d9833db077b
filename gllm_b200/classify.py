"""Re-export of the classify builder types (they live with the client that executes them)."""
from .client import *  # noqa: F401,F403
