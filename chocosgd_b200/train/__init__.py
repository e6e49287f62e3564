"""Training loops, LR scheduler and metrics."""
from .metrics import Metrics
from .scheduler import Scheduler
