"""CPU oracle (test infrastructure, never imported by the product package)."""
from .na2d_oracle import *  # noqa: F401,F403
