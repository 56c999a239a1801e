"""Alignment pre-processing workflows (the reference's ``fastfold.workflow``, on a local scheduler instead of Ray)."""
from .dag import TaskNode, WorkflowError, run_dag  # noqa: F401
from .workflow_run import batch_run  # noqa: F401
