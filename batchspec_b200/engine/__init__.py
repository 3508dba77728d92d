from .engine import Engine, parse_dtype
from .scheduler import Scheduler, Workload
from .sequence import Sequence, Status
from .step import GroupTables, StepContext, StepEntry, StepRunner

__all__ = ["Engine", "parse_dtype", "Scheduler", "Workload", "Sequence", "Status", "GroupTables", "StepContext",
           "StepEntry", "StepRunner"]
