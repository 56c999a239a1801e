"""Import-path alias (fastfold/data/tools/hmmbuild.py): the code lives in the package module."""
from . import Hmmbuild  # noqa: F401
