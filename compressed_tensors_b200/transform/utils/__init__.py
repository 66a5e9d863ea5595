from .hadamard import *  # noqa: F401,F403
from .matrix import *  # noqa: F401,F403
