"""Import-path alias (fastfold/data/tools/jackhmmer.py): the code lives in the package module."""
from . import Jackhmmer  # noqa: F401
