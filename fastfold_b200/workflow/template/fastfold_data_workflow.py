"""Monomer alignment workflow (fastfold/workflow/template/fastfold_data_workflow.py:16-169):
jackhmmer(uniref90) -> hhsearch(pdb70)   ||   jackhmmer(mgnify)   ||   hhblits(bfd) | jackhmmer(small bfd)."""
import os
import time
from typing import Optional

from ..factory import HHBlitsFactory, HHSearchFactory, JackHmmerFactory
from ..workflow_run import batch_run


def _check(groups, need_uniref_for_templates, uniref90_database_path):
    for name, (binary, dbs) in groups.items():
        if binary is None and any(d is not None for d in dbs):
            raise ValueError("%s DBs provided but %s binary is None" % (name, name))
    if need_uniref_for_templates and uniref90_database_path is None:
        raise ValueError("uniref90_database_path must be specified in order to perform template search")


class FastFoldDataWorkFlow:
    """Writes ``uniref90_hits.a3m``, ``pdb70_hits.hhr``, ``mgnify_hits.a3m`` and ``bfd_uniref_hits.a3m`` into
    ``alignment_dir`` (fastfold/workflow/template/fastfold_data_workflow.py:10-169)."""

    def __init__(self, jackhmmer_binary_path: Optional[str] = None, hhblits_binary_path: Optional[str] = None,
                 hhsearch_binary_path: Optional[str] = None, uniref90_database_path: Optional[str] = None,
                 mgnify_database_path: Optional[str] = None, bfd_database_path: Optional[str] = None,
                 uniref30_database_path: Optional[str] = None, pdb70_database_path: Optional[str] = None,
                 use_small_bfd: Optional[bool] = None, no_cpus: Optional[int] = None, uniref_max_hits: int = 10000,
                 mgnify_max_hits: int = 5000):
        _check({"jackhmmer": (jackhmmer_binary_path, [uniref90_database_path, mgnify_database_path, bfd_database_path if use_small_bfd else None]),
                "hhblits": (hhblits_binary_path, [bfd_database_path if not use_small_bfd else None]),
                "hhsearch": (hhsearch_binary_path, [pdb70_database_path])}, pdb70_database_path is not None, uniref90_database_path)
        self.use_small_bfd = use_small_bfd
        n_cpu = no_cpus or os.cpu_count() or 1
        jack = lambda db, hits: JackHmmerFactory(config={"binary_path": jackhmmer_binary_path, "database_path": db, "n_cpu": n_cpu,
                                                         "uniref_max_hits": hits})
        self.jackhmmer_uniref90_factory = jack(uniref90_database_path, uniref_max_hits) if uniref90_database_path else None
        self.jackhmmer_mgnify_factory = jack(mgnify_database_path, mgnify_max_hits) if mgnify_database_path else None
        self.jackhmmer_small_bfd_factory = jack(bfd_database_path, uniref_max_hits) if (bfd_database_path and use_small_bfd) else None
        self.hhblits_bfd_factory = None
        if bfd_database_path is not None and not use_small_bfd:
            dbs = [bfd_database_path] + ([uniref30_database_path] if uniref30_database_path else [])
            self.hhblits_bfd_factory = HHBlitsFactory(config={"binary_path": hhblits_binary_path, "databases": dbs, "n_cpu": n_cpu})
        self.hhsearch_pdb_factory = None
        if pdb70_database_path is not None:
            self.hhsearch_pdb_factory = HHSearchFactory(config={"binary_path": hhsearch_binary_path, "databases": [pdb70_database_path],
                                                                "n_cpu": n_cpu})

    def _bfd_node(self, fasta_path, alignment_dir, small_name):
        if self.use_small_bfd and self.jackhmmer_small_bfd_factory is not None:
            return self.jackhmmer_small_bfd_factory.gen_node(fasta_path, os.path.join(alignment_dir, small_name), output_format="sto")
        if self.hhblits_bfd_factory is not None:
            return self.hhblits_bfd_factory.gen_node(fasta_path, os.path.join(alignment_dir, "bfd_uniref_hits.a3m"))
        return None

    def run(self, fasta_path: str, alignment_dir: Optional[str] = None, storage_dir: Optional[str] = None) -> None:
        os.makedirs(alignment_dir, exist_ok=True)
        targets = []
        if self.jackhmmer_uniref90_factory is not None:
            uniref = os.path.join(alignment_dir, "uniref90_hits.a3m")
            node = self.jackhmmer_uniref90_factory.gen_node(fasta_path, uniref)
            if self.hhsearch_pdb_factory is not None:
                node = self.hhsearch_pdb_factory.gen_node(uniref, os.path.join(alignment_dir, "pdb70_hits.hhr"), after=[node])
            targets.append(node)
        if self.jackhmmer_mgnify_factory is not None:
            targets.append(self.jackhmmer_mgnify_factory.gen_node(fasta_path, os.path.join(alignment_dir, "mgnify_hits.a3m")))
        bfd = self._bfd_node(fasta_path, alignment_dir, "bfd_uniref_hits.a3m")
        if bfd is not None:
            targets.append(bfd)
        batch_run(workflow_id="fastfold_data_workflow " + time.asctime(), dags=targets)
