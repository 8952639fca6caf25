"""Drop-in replacement of the `adafactor8bit` package for NVIDIA B200: the same
public names (reference __init__.py:4-8), backed by libaf8's sm_100a kernels."""
from .optimizer import Adafactor8Bit
from .routing import build_param_groups
from .zero import ShardedAdafactor8Bit

__version__ = "0.4.6+b200.1"
__all__ = ["Adafactor8Bit", "build_param_groups", "ShardedAdafactor8Bit", "__version__"]
