"""jackhmmer (HMMER) wrapper: iterative protein sequence search, optionally streamed over database chunks
(fastfold/data/tools/jackhmmer.py:30-249)."""
import contextlib
import glob
import logging
import os
import shutil
from concurrent import futures
from typing import Any, Callable, Mapping, Optional, Sequence
from urllib import request

from .utils import _need_binary, _run, tmpdir_manager

log = logging.getLogger(__name__)


class Jackhmmer:
    """Iterative profile search of one sequence against a FASTA database (fastfold/data/tools/jackhmmer.py:30-249).

    A database too large for the page cache can be searched in ``num_streamed_chunks`` pieces named
    ``<database_path>.<i>`` (1-based): the next piece is copied to ``/tmp/ramdisk`` by a helper thread while the
    current one is searched.
    """

    def __init__(self, *, binary_path: str, database_path: str, n_cpu: int = 8, n_iter: int = 1, e_value: float = 1e-4,
                 z_value: Optional[int] = None, get_tblout: bool = False, filter_f1: float = 5e-4, filter_f2: float = 5e-5,
                 filter_f3: float = 5e-7, incdom_e: Optional[float] = None, dom_e: Optional[float] = None,
                 num_streamed_chunks: Optional[int] = None, streaming_callback: Optional[Callable[[int], None]] = None):
        self.binary_path = _need_binary(binary_path, "jackhmmer")
        self.database_path = database_path
        self.num_streamed_chunks = num_streamed_chunks
        if not os.path.exists(database_path) and num_streamed_chunks is None:
            raise ValueError("Could not find Jackhmmer database %s" % database_path)
        self.n_cpu, self.n_iter, self.e_value, self.z_value = n_cpu, n_iter, e_value, z_value
        self.filter_f1, self.filter_f2, self.filter_f3 = filter_f1, filter_f2, filter_f3
        self.incdom_e, self.dom_e, self.get_tblout = incdom_e, dom_e, get_tblout
        self.streaming_callback = streaming_callback

    def _command(self, fasta, database, sto, tbl):
        cmd = [self.binary_path, "-o", "/dev/null", "-A", sto, "--noali", "--F1", str(self.filter_f1), "--F2", str(self.filter_f2),
               "--F3", str(self.filter_f3), "--incE", str(self.e_value), "-E", str(self.e_value), "--cpu", str(self.n_cpu), "-N",
               str(self.n_iter)]
        if self.get_tblout:
            cmd += ["--tblout", tbl]
        if self.z_value:
            cmd += ["-Z", str(self.z_value)]
        if self.dom_e is not None:
            cmd += ["--domE", str(self.dom_e)]
        if self.incdom_e is not None:
            cmd += ["--incdomE", str(self.incdom_e)]
        return cmd + [fasta, database]

    def _query_chunk(self, input_fasta_path: str, database_path: str, max_sequences: Optional[int] = None) -> Mapping[str, Any]:
        with tmpdir_manager() as tmp:
            sto, tbl = os.path.join(tmp, "output.sto"), os.path.join(tmp, "tblout.txt")
            _, stderr = _run(self._command(input_fasta_path, database_path, sto, tbl), "Jackhmmer (%s)" % os.path.basename(database_path))
            tbl_text = open(tbl).read() if self.get_tblout else ""
            if max_sequences is None:
                sto_text = open(sto).read()
            else:
                from .. import parsers
                sto_text = parsers.truncate_stockholm_msa(sto, max_sequences)
        return dict(sto=sto_text, tbl=tbl_text, stderr=stderr, n_iter=self.n_iter, e_value=self.e_value)

    def query(self, input_fasta_path: str, max_sequences: Optional[int] = None) -> Sequence[Mapping[str, Any]]:
        if self.num_streamed_chunks is None:
            return [self._query_chunk(input_fasta_path, self.database_path, max_sequences)]
        name = os.path.basename(self.database_path)
        remote = lambda i: "%s.%d" % (self.database_path, i)
        local = lambda i: "/tmp/ramdisk/%s.%d" % (name, i)
        for stale in glob.glob("/tmp/ramdisk/%s.[0-9]*" % name):
            with contextlib.suppress(OSError):
                os.remove(stale)
        out = []
        with futures.ThreadPoolExecutor(max_workers=2) as pool:
            fetch = lambda i: request.urlretrieve(remote(i), local(i)) if "://" in remote(i) else shutil.copyfile(remote(i), local(i))
            os.makedirs("/tmp/ramdisk", exist_ok=True)
            pending = pool.submit(fetch, 1)
            for i in range(1, self.num_streamed_chunks + 1):
                pending.result()
                if i < self.num_streamed_chunks:
                    pending = pool.submit(fetch, i + 1)
                out.append(self._query_chunk(input_fasta_path, local(i), max_sequences))
                os.remove(local(i))
                if self.streaming_callback:
                    self.streaming_callback(i)
        return out
