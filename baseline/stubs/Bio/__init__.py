"""Stand-in for BioPython (not installed here).  The reference imports ``Bio.PDB.PDBParser`` at module level in
``fastfold/common/protein.py``; nothing on the benchmarked path calls it."""
