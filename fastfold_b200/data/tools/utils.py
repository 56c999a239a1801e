"""Import-path alias (fastfold/data/tools/utils.py): the code lives in the package module."""
from . import tmpdir_manager, timing, to_date  # noqa: F401
