"""hhfilter (HH-suite) wrapper: thins an alignment by sequence identity / coverage (used by the alignment workflow)."""
import logging

from .utils import _need_binary, _run

log = logging.getLogger(__name__)


class HHFilter:
    """Redundancy filter of an A3M (``hhfilter -id``); used by the workflow between search stages."""

    def __init__(self, *, binary_path: str, id: int = 90, cov: int = 0):
        self.binary_path = _need_binary(binary_path, "hhfilter")
        self.id, self.cov = id, cov

    def query(self, a3m_path: str, output_path: str) -> str:
        _run([self.binary_path, "-i", a3m_path, "-o", output_path, "-id", str(self.id), "-cov", str(self.cov)], "HHfilter")
        return output_path
