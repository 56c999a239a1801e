"""hmmbuild (HMMER) wrapper: profile HMM from an alignment (fastfold/data/tools/hmmbuild.py:25-137)."""
import logging
import os

from .utils import _need_binary, _run, tmpdir_manager

log = logging.getLogger(__name__)


class Hmmbuild:
    """Profile HMM from an alignment (fastfold/data/tools/hmmbuild.py:25-137)."""

    def __init__(self, *, binary_path: str, singlemx: bool = False):
        """``singlemx``: use the substitution score matrix also for alignments of more than one sequence."""
        self.binary_path = _need_binary(binary_path, "hmmbuild")
        self.singlemx = singlemx

    def build_profile_from_sto(self, sto: str, model_construction: str = "fast") -> str:
        return self._build(sto, model_construction)

    def build_profile_from_a3m(self, a3m: str) -> str:
        # drop insert columns (lower case) so that the A3M becomes an aligned FASTA hmmbuild accepts
        lines = [ln if ln.startswith(">") else "".join(c for c in ln if not c.islower()) for ln in a3m.splitlines()]
        return self._build("\n".join(lines) + "\n", "fast")

    def _build(self, msa: str, model_construction: str) -> str:
        if model_construction not in ("hand", "fast"):
            raise ValueError("Invalid model_construction %r - only hand and fast supported." % model_construction)
        with tmpdir_manager() as tmp:
            inp, out = os.path.join(tmp, "query.msa"), os.path.join(tmp, "output.hmm")
            with open(inp, "w") as f:
                f.write(msa)
            cmd = [self.binary_path]
            if model_construction == "hand":
                cmd.append("--hand")
            if self.singlemx:
                cmd.append("--singlemx")
            _run(cmd + ["--amino", out, inp], "hmmbuild")
            return open(out).read()
