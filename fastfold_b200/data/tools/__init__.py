"""Subprocess wrappers around the external alignment tools (HMMER, HH-suite, kalign).

Each wrapper builds the command line, runs the binary in a scratch directory and returns the text it produced; none of
them is on the GPU path.  A missing binary raises ``ToolNotFound`` at construction time, so that a pipeline can decide
early to fall back to pre-computed alignments.  Same roles as fastfold/data/tools/{jackhmmer,hhblits,hhsearch,
hmmsearch,hmmbuild,kalign,utils}.py; the reference's per-tool module names are importable too
(``fastfold_b200.data.tools.jackhmmer`` ...).
"""
from .hhblits import HHBlits
from .hhfilter import HHFilter
from .hhsearch import HHSearch
from .hmmbuild import Hmmbuild
from .hmmsearch import Hmmsearch
from .jackhmmer import Jackhmmer
from .kalign import Kalign
from .utils import ToolFailed, ToolNotFound, timing, tmpdir_manager, to_date, _need_binary, _run          # noqa: F401

__all__ = ["Jackhmmer", "HHBlits", "HHSearch", "HHFilter", "Hmmbuild", "Hmmsearch", "Kalign", "ToolNotFound", "ToolFailed", "tmpdir_manager", "timing",
           "to_date"]
