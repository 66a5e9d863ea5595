from .base import *  # noqa: F401,F403
from .hadamard import *  # noqa: F401,F403
from .random_hadamard import *  # noqa: F401,F403
