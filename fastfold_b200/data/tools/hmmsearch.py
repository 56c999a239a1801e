"""Import-path alias (fastfold/data/tools/hmmsearch.py): the code lives in the package module."""
from . import Hmmsearch  # noqa: F401
