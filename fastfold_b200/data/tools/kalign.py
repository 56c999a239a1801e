"""kalign wrapper: realignment of a template sequence to the query (fastfold/data/tools/kalign.py:24-115)."""
import logging
import os
from typing import Sequence

from .utils import _need_binary, _run, tmpdir_manager

log = logging.getLogger(__name__)


class Kalign:
    """Multiple alignment of a few sequences, returned as A3M (fastfold/data/tools/kalign.py:26-115)."""

    def __init__(self, *, binary_path: str):
        self.binary_path = _need_binary(binary_path, "kalign")

    def align(self, sequences: Sequence[str]) -> str:
        for s in sequences:
            if len(s) < 6:
                raise ValueError("Kalign requires all sequences to be at least 6 residues long. Got %s (%d residues)." % (s, len(s)))
        with tmpdir_manager() as tmp:
            inp, out = os.path.join(tmp, "input.fasta"), os.path.join(tmp, "output.a3m")
            with open(inp, "w") as f:
                f.write("".join(">sequence %d\n%s\n" % (i, s) for i, s in enumerate(sequences, 1)))
            _run([self.binary_path, "-i", inp, "-o", out, "-format", "fasta"], "Kalign")
            return open(out).read()
