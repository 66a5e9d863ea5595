from .helpers import *  # noqa: F401,F403
from .safetensors_load import *  # noqa: F401,F403
from .semi_structured_conversions import *  # noqa: F401,F403
from .permutations_24 import *  # noqa: F401,F403
