from .quant_args import *  # noqa: F401,F403
from .quant_scheme import *  # noqa: F401,F403
from .utils.helpers import *  # noqa: F401,F403
from .lifecycle.forward import *  # noqa: F401,F403
from .lifecycle.initialize import *  # noqa: F401,F403
from .lifecycle.compressed import *  # noqa: F401,F403
from .lifecycle.helpers import *  # noqa: F401,F403
from .quant_config import *  # noqa: F401,F403
