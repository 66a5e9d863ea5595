from .base import *  # noqa: F401,F403
from .fp4_quantized import *  # noqa: F401,F403
from .naive_quantized import *  # noqa: F401,F403
from .pack_quantized import *  # noqa: F401,F403
