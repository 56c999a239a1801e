"""Import-path alias (fastfold/workflow/factory/hhfilter.py)."""
from . import HHfilterFactory  # noqa: F401
