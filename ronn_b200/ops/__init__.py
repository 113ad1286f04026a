"""Python entry points of the hand-written sm_100a kernels."""
from .kernels import *  # noqa: F401,F403
