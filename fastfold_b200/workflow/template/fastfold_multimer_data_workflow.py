"""Multimer alignment workflow (fastfold/workflow/template/fastfold_multimer_data_workflow.py:17-192):
jackhmmer(uniref90, sto) -> hmmsearch(pdb seqres)   ||   jackhmmer(mgnify)   ||   bfd   ||   jackhmmer(uniprot)."""
import os
import time
from typing import Optional

from ..factory import HmmSearchFactory, JackHmmerFactory
from ..workflow_run import batch_run
from .fastfold_data_workflow import FastFoldDataWorkFlow, _check


class FastFoldMultimerDataWorkFlow(FastFoldDataWorkFlow):
    """Per-chain multimer searches with Stockholm outputs, a UniProt search and an hmmsearch template search
    (fastfold/workflow/template/fastfold_multimer_data_workflow.py:12-192)."""

    def __init__(self, jackhmmer_binary_path: Optional[str] = None, hhblits_binary_path: Optional[str] = None,
                 hmmsearch_binary_path: Optional[str] = None, hmmbuild_binary_path: Optional[str] = None,
                 uniref90_database_path: Optional[str] = None, mgnify_database_path: Optional[str] = None,
                 bfd_database_path: Optional[str] = None, uniref30_database_path: Optional[str] = None,
                 uniprot_database_path: Optional[str] = None, pdb_seqres_database_path: Optional[str] = None,
                 use_small_bfd: Optional[bool] = None, no_cpus: Optional[int] = None, uniref_max_hits: int = 10000,
                 mgnify_max_hits: int = 5000, uniprot_max_hits: int = 50000):
        super().__init__(jackhmmer_binary_path=jackhmmer_binary_path, hhblits_binary_path=hhblits_binary_path,
                         uniref90_database_path=uniref90_database_path, mgnify_database_path=mgnify_database_path,
                         bfd_database_path=bfd_database_path, uniref30_database_path=uniref30_database_path, use_small_bfd=use_small_bfd,
                         no_cpus=no_cpus, uniref_max_hits=uniref_max_hits, mgnify_max_hits=mgnify_max_hits)
        _check({"hmmsearch": (hmmsearch_binary_path, [pdb_seqres_database_path]), "jackhmmer": (jackhmmer_binary_path, [uniprot_database_path])},
               pdb_seqres_database_path is not None, uniref90_database_path)
        n_cpu = no_cpus or os.cpu_count() or 1
        self.jackhmmer_uniprot_factory = None
        if uniprot_database_path is not None:
            self.jackhmmer_uniprot_factory = JackHmmerFactory(config={"binary_path": jackhmmer_binary_path, "database_path": uniprot_database_path,
                                                                      "n_cpu": n_cpu, "uniref_max_hits": uniprot_max_hits})
        self.hmmsearch_pdb_factory = None
        if pdb_seqres_database_path is not None:
            self.hmmsearch_pdb_factory = HmmSearchFactory(config={"binary_path": hmmsearch_binary_path, "hmmbuild_binary_path": hmmbuild_binary_path,
                                                                  "database_path": pdb_seqres_database_path, "n_cpu": n_cpu})

    def run(self, fasta_path: str, alignment_dir: Optional[str] = None, storage_dir: Optional[str] = None) -> None:
        os.makedirs(alignment_dir, exist_ok=True)
        targets = []
        if self.jackhmmer_uniref90_factory is not None:
            uniref = os.path.join(alignment_dir, "uniref90_hits.sto")
            node = self.jackhmmer_uniref90_factory.gen_node(fasta_path, uniref, output_format="sto")
            if self.hmmsearch_pdb_factory is not None:
                node = self.hmmsearch_pdb_factory.gen_node(uniref, output_dir=alignment_dir, after=[node])
            targets.append(node)
        if self.jackhmmer_mgnify_factory is not None:
            targets.append(self.jackhmmer_mgnify_factory.gen_node(fasta_path, os.path.join(alignment_dir, "mgnify_hits.sto"), output_format="sto"))
        bfd = self._bfd_node(fasta_path, alignment_dir, "bfd_uniref_hits.sto")
        if bfd is not None:
            targets.append(bfd)
        if self.jackhmmer_uniprot_factory is not None:
            targets.append(self.jackhmmer_uniprot_factory.gen_node(fasta_path, os.path.join(alignment_dir, "uniprot_hits.sto"), output_format="sto"))
        batch_run(workflow_id="fastfold_multimer_data_workflow " + time.asctime(), dags=targets)
