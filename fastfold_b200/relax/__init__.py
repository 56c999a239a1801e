"""Structure relaxation (role of fastfold/relax): OpenMM Amber minimisation when OpenMM is installed, otherwise a
self-contained violation minimiser in PyTorch."""
from .relax import AmberRelaxation  # noqa: F401
