from .base import *  # noqa: F401,F403
from .quantized_compressors import *  # noqa: F401,F403
from .sparse_compressors import *  # noqa: F401,F403
from .sparse_quantized_compressors import *  # noqa: F401,F403
from .model_compressors import *  # noqa: F401,F403
