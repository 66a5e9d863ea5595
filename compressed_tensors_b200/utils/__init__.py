from .helpers import *  # noqa: F401,F403
from .safetensors_load import *  # noqa: F401,F403
