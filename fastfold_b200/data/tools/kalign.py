"""Import-path alias (fastfold/data/tools/kalign.py): the code lives in the package module."""
from . import Kalign  # noqa: F401
