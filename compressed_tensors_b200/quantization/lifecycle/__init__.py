from .forward import *  # noqa: F401,F403
