"""Stand-in that forwards to the standard library's importlib.resources."""
from importlib.resources import *  # noqa: F401,F403
from importlib.resources import as_file, files  # noqa: F401

try:
    from importlib.resources.abc import Traversable  # noqa: F401
except ImportError:  # pragma: no cover
    from importlib.abc import Traversable  # noqa: F401
