"""Import-path alias (fastfold/workflow/factory/hmmsearch.py)."""
from . import HmmSearchFactory  # noqa: F401
