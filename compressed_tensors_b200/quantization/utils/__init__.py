from .helpers import *  # noqa: F401,F403
from .mxfp4_utils import *  # noqa: F401,F403
