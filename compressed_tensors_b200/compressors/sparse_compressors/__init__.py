from .base import *  # noqa: F401,F403
from .dense import *  # noqa: F401,F403
from .sparse_24_bitmask import *  # noqa: F401,F403
from .sparse_bitmask import *  # noqa: F401,F403
