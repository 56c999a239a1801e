"""Species identifiers of MSA rows (UniProt-style descriptions), used to pair rows of different chains.
Import path of fastfold/data/msa_identifiers.py:50-91; the parser lives beside the pairing code."""
from .msa_pairing import Identifiers, get_identifiers          # noqa: F401
