"""Import-path alias (fastfold/workflow/factory/jackhmmer.py)."""
from . import JackHmmerFactory  # noqa: F401
