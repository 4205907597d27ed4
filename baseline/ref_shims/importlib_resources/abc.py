from importlib.resources.abc import *  # noqa: F401,F403
from importlib.resources.abc import Traversable  # noqa: F401
