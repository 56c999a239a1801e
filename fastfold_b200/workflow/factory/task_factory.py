"""Import-path alias (fastfold/workflow/factory/task_factory.py)."""
from . import TaskFactory  # noqa: F401
