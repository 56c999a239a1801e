"""Optimal rigid superposition (Kabsch, via SVD) of one point set onto another under a mask.
Import path of fastfold/utils/superimposition.py:1-99; the implementation sits with the validation metrics."""
from .validation_utils import superimpose          # noqa: F401
