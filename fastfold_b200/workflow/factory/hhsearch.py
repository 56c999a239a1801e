"""Import-path alias (fastfold/workflow/factory/hhsearch.py)."""
from . import HHSearchFactory  # noqa: F401
