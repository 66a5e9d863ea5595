from .marlin_24 import *  # noqa: F401,F403
