"""Ready-made alignment workflows: monomer and multimer (fastfold/workflow/template/*.py).

Monomer graph:   jackhmmer(uniref90) -> hhsearch(pdb70)   ||   jackhmmer(mgnify)   ||   hhblits(bfd) | jackhmmer(small bfd)
Multimer graph:  jackhmmer(uniref90, sto) -> hmmsearch(pdb seqres)   ||   jackhmmer(mgnify)   ||   bfd   ||   jackhmmer(uniprot)
"""
from .fastfold_data_workflow import FastFoldDataWorkFlow
from .fastfold_multimer_data_workflow import FastFoldMultimerDataWorkFlow

__all__ = ["FastFoldDataWorkFlow", "FastFoldMultimerDataWorkFlow"]
