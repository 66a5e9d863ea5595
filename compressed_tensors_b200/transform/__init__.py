from .transform_args import *  # noqa: F401,F403
from .transform_scheme import *  # noqa: F401,F403
from .transform_config import *  # noqa: F401,F403
from .factory import *  # noqa: F401,F403
from .utils import *  # noqa: F401,F403
from .apply import *  # noqa: F401,F403
