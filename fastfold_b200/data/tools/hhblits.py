"""hhblits (HH-suite) wrapper: iterative HMM-HMM search of one or several databases (fastfold/data/tools/hhblits.py:28-181)."""
import glob
import logging
import os
from typing import Any, Mapping, Optional, Sequence

from .utils import _need_binary, _run, tmpdir_manager

log = logging.getLogger(__name__)


class HHBlits:
    """Iterative HMM-HMM search against HH-suite databases (fastfold/data/tools/hhblits.py:30-181)."""

    def __init__(self, *, binary_path: str, databases: Sequence[str], n_cpu: int = 4, n_iter: int = 3, e_value: float = 0.001,
                 maxseq: int = 1_000_000, realign_max: int = 100_000, maxfilt: int = 100_000, min_prefilter_hits: int = 1000,
                 all_seqs: bool = False, alt: Optional[int] = None, p: int = 20, z: int = 500, cov: int = 0):
        self.binary_path = _need_binary(binary_path, "hhblits")
        self.databases = list(databases)
        for db in self.databases:
            if not glob.glob(db + "_*"):
                raise ValueError("Could not find HHBlits database %s" % db)
        self.n_cpu, self.n_iter, self.e_value, self.maxseq = n_cpu, n_iter, e_value, maxseq
        self.realign_max, self.maxfilt, self.min_prefilter_hits = realign_max, maxfilt, min_prefilter_hits
        self.all_seqs, self.alt, self.p, self.z = all_seqs, alt, p, z
        self.cov = cov              # minimum coverage of the query (%), 0 = no filter

    def query(self, input_fasta_path: str) -> Mapping[str, Any]:
        with tmpdir_manager() as tmp:
            a3m = os.path.join(tmp, "output.a3m")
            cmd = [self.binary_path, "-i", input_fasta_path, "-cpu", str(self.n_cpu), "-oa3m", a3m, "-o", "/dev/null", "-n", str(self.n_iter),
                   "-e", str(self.e_value), "-maxseq", str(self.maxseq), "-realign_max", str(self.realign_max), "-maxfilt", str(self.maxfilt),
                   "-min_prefilter_hits", str(self.min_prefilter_hits)]
            if self.all_seqs:
                cmd.append("-all")
            if self.alt:
                cmd += ["-alt", str(self.alt)]
            if self.p != 20:
                cmd += ["-p", str(self.p)]
            if self.z != 500:
                cmd += ["-Z", str(self.z)]
            if self.cov:
                cmd += ["-cov", str(self.cov)]
            for db in self.databases:
                cmd += ["-d", db]
            stdout, stderr = _run(cmd, "HHblits")
            a3m_text = open(a3m).read()
        return dict(a3m=a3m_text, output=stdout, stderr=stderr, n_iter=self.n_iter, e_value=self.e_value)
