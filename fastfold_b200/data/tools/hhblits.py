"""Import-path alias (fastfold/data/tools/hhblits.py): the code lives in the package module."""
from . import HHBlits  # noqa: F401
