from .engine import Engine, parse_dtype
from .step import GroupTables, StepContext, StepEntry, StepRunner

__all__ = ["Engine", "parse_dtype", "GroupTables", "StepContext", "StepEntry", "StepRunner"]
