"""hmmsearch (HMMER) wrapper: profile search of PDB seqres, the multimer template search (fastfold/data/tools/hmmsearch.py:27-139)."""
import logging
import os
from typing import Optional, Sequence

from .utils import _need_binary, _run, tmpdir_manager

from .hmmbuild import Hmmbuild

log = logging.getLogger(__name__)


class Hmmsearch:
    """Search a profile HMM against a sequence database (fastfold/data/tools/hmmsearch.py:27-139)."""

    def __init__(self, *, binary_path: str, hmmbuild_binary_path: str, database_path: str, n_cpu: int = 8,
                 flags: Optional[Sequence[str]] = None):
        self.binary_path = _need_binary(binary_path, "hmmsearch")
        self.hmmbuild_runner = Hmmbuild(binary_path=hmmbuild_binary_path)
        if not os.path.exists(database_path):
            raise ValueError("Could not find hmmsearch database %s" % database_path)
        self.database_path = database_path
        self.n_cpu = n_cpu
        if flags is None:      # defaults of the multimer template search
            flags = ["--F1", "0.1", "--F2", "0.1", "--F3", "0.1", "--incE", "100", "-E", "100", "--domE", "100", "--incdomE", "100"]
        self.flags = list(flags)

    output_format = property(lambda self: "sto")
    input_format = property(lambda self: "sto")

    def query(self, msa_sto: str, output_dir: Optional[str] = None) -> str:
        return self.query_with_hmm(self.hmmbuild_runner.build_profile_from_sto(msa_sto, model_construction="hand"), output_dir)

    def query_with_hmm(self, hmm: str, output_dir: Optional[str] = None) -> str:
        with tmpdir_manager() as tmp:
            hmm_path = os.path.join(tmp, "query.hmm")
            out_dir = tmp if output_dir is None else output_dir
            sto = os.path.join(out_dir, "hmm_output.sto")
            with open(hmm_path, "w") as f:
                f.write(hmm)
            cmd = [self.binary_path, "--noali", "--cpu", str(self.n_cpu)] + self.flags + ["-A", sto, hmm_path, self.database_path]
            _run(cmd, "hmmsearch (%s)" % os.path.basename(self.database_path))
            return open(sto).read()

    def get_template_hits(self, output_string: str, input_sequence: str):
        from .. import parsers
        a3m = parsers.convert_stockholm_to_a3m(output_string, remove_first_row_gaps=False)
        return parsers.parse_hmmsearch_a3m(query_sequence=input_sequence, a3m_string=a3m, skip_first=False)
