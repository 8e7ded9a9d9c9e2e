from .step import Engine, GroupMeta, StepContext, StepEntry, Workspace

__all__ = ["Engine", "StepEntry", "StepContext", "GroupMeta", "Workspace"]
