"""hhsearch (HH-suite) wrapper: template search of an alignment against PDB70 (fastfold/data/tools/hhsearch.py:26-164)."""
import glob
import logging
import os
from typing import Sequence, Union

from .utils import _need_binary, _run, tmpdir_manager

log = logging.getLogger(__name__)


class HHSearch:
    """Template search of an A3M profile against HH-suite databases (fastfold/data/tools/hhsearch.py:26-164)."""

    def __init__(self, *, binary_path: str, databases: Sequence[str], n_cpu: int = 2, maxseq: int = 1_000_000, mact: float = 0.35,
                 min_align: int = 10, max_align: int = 500, min_lines: int = 10, max_lines: int = 500, aliw: int = 100000,
                 e_value: float = 0.001, min_prob: float = 20.0):
        """``mact``: posterior threshold of the realignment (greediness at alignment ends); ``min_align`` / ``max_align``:
        bounds on the alignment list (-b / -B); ``min_lines`` / ``max_lines``: bounds on the summary list (-z / -Z);
        ``aliw``: columns per alignment line; ``e_value``: inclusion cutoff; ``min_prob``: minimum probability listed."""
        self.binary_path = _need_binary(binary_path, "hhsearch")
        self.databases = list(databases)
        for db in self.databases:
            if not glob.glob(db + "_*"):
                raise ValueError("Could not find HHsearch database %s" % db)
        self.n_cpu, self.maxseq = n_cpu, maxseq
        self.mact, self.min_align, self.max_align, self.min_lines, self.max_lines = mact, min_align, max_align, min_lines, max_lines
        self.aliw, self.e_value, self.min_prob = aliw, e_value, min_prob

    output_format = property(lambda self: "hhr")
    input_format = property(lambda self: "a3m")

    def query(self, a3m: str, gen_atab: bool = False) -> Union[str, tuple]:
        with tmpdir_manager() as tmp:
            inp, hhr, atab = os.path.join(tmp, "query.a3m"), os.path.join(tmp, "output.hhr"), os.path.join(tmp, "output.atab")
            with open(inp, "w") as f:
                f.write(a3m)
            cmd = [self.binary_path, "-i", inp, "-o", hhr, "-maxseq", str(self.maxseq), "-cpu", str(self.n_cpu),
                   "-b", str(self.min_align), "-B", str(self.max_align), "-z", str(self.min_lines), "-Z", str(self.max_lines),
                   "-mact", str(self.mact), "-aliw", str(self.aliw), "-e", str(self.e_value), "-p", str(self.min_prob)]
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
