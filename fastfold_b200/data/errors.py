"""Exception types of the data pipeline (import path of fastfold/data/errors.py:17-22)."""
from .templates import Error, MultipleChainsError          # noqa: F401
