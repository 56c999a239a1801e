"""Import-path alias (fastfold/workflow/template/fastfold_multimer_data_workflow.py)."""
from . import FastFoldMultimerDataWorkFlow  # noqa: F401
