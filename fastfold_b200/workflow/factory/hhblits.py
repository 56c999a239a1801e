"""Import-path alias (fastfold/workflow/factory/hhblits.py)."""
from . import HHBlitsFactory  # noqa: F401
