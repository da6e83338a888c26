from .exceptions import *  # noqa: F401,F403
from .local import LocalScheduler

__all__ = ["LocalScheduler"]
