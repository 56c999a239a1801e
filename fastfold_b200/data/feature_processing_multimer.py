"""Multimer feature processing entry points: per-chain clean-up, MSA pairing, cropping and merging of the chains of a
complex into one example (``pair_and_merge``), and the final filtering / mask fix-up (``process_final``).

The implementation shares its tables and helpers with the pairing code and lives in ``msa_pairing``; this module gives
it the import path of fastfold/data/feature_processing_multimer.py:41-244.
"""
from .msa_pairing import (REQUIRED_FEATURES, crop_chains, pair_and_merge, process_final, process_unmerged_features,       # noqa: F401
                          _is_homomer_or_monomer)
