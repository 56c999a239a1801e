"""Import-path alias (fastfold/workflow/template/fastfold_data_workflow.py)."""
from . import FastFoldDataWorkFlow  # noqa: F401
