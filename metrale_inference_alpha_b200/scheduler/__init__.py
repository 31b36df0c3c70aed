from .core import SchedulerCore  # noqa: F401
from .policy import SchedulerConfig  # noqa: F401
from .types import *  # noqa: F401,F403
