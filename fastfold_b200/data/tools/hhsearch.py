"""Import-path alias (fastfold/data/tools/hhsearch.py): the code lives in the package module."""
from . import HHSearch  # noqa: F401
