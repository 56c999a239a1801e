"""hhsearch (HH-suite) wrapper: template search of an alignment against PDB70 (fastfold/data/tools/hhsearch.py:26-164)."""
import glob
import logging
import os
from typing import Sequence, Union

from .utils import _need_binary, _run, tmpdir_manager

log = logging.getLogger(__name__)


class HHSearch:
    """Template search of an A3M profile against HH-suite databases (fastfold/data/tools/hhsearch.py:26-164)."""

    def __init__(self, *, binary_path: str, databases: Sequence[str], n_cpu: int = 2, maxseq: int = 1_000_000):
        self.binary_path = _need_binary(binary_path, "hhsearch")
        self.databases = list(databases)
        for db in self.databases:
            if not glob.glob(db + "_*"):
                raise ValueError("Could not find HHsearch database %s" % db)
        self.n_cpu, self.maxseq = n_cpu, maxseq

    output_format = property(lambda self: "hhr")
    input_format = property(lambda self: "a3m")

    def query(self, a3m: str, gen_atab: bool = False) -> Union[str, tuple]:
        with tmpdir_manager() as tmp:
            inp, hhr, atab = os.path.join(tmp, "query.a3m"), os.path.join(tmp, "output.hhr"), os.path.join(tmp, "output.atab")
            with open(inp, "w") as f:
                f.write(a3m)
            cmd = [self.binary_path, "-i", inp, "-o", hhr, "-maxseq", str(self.maxseq), "-cpu", str(self.n_cpu)]
            for db in self.databases:
                cmd += ["-d", db]
            if gen_atab:
                cmd += ["-atab", atab]
            _run(cmd, "HHsearch")
            hhr_text = open(hhr).read()
            atab_text = open(atab).read() if gen_atab else None
        return (hhr_text, atab_text) if gen_atab else hhr_text

    def get_template_hits(self, output_string: str, input_sequence: str):
        from .. import parsers
        return parsers.parse_hhr(output_string)
