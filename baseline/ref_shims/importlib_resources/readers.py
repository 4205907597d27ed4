from importlib.resources.readers import *  # noqa: F401,F403
from importlib.resources.readers import MultiplexedPath  # noqa: F401
