from .compressed_linear import *  # noqa: F401,F403
