"""Subprocess wrappers around the external alignment tools (HMMER, HH-suite, kalign).

Each wrapper builds the command line, runs the binary in a scratch directory and returns the text it produced; none of
them is on the GPU path.  A missing binary raises ``ToolNotFound`` at construction time, so that a pipeline can decide
early to fall back to pre-computed alignments.  Same roles as fastfold/data/tools/{jackhmmer,hhblits,hhsearch,
hmmsearch,hmmbuild,kalign,utils}.py; the reference's per-tool module names are importable too
(``fastfold_b200.data.tools.jackhmmer`` ...).
"""
import contextlib
import datetime
import glob
import logging
import os
import shutil
import subprocess
import tempfile
import time
from concurrent import futures
from typing import Any, Callable, Mapping, Optional, Sequence, Union
from urllib import request

log = logging.getLogger(__name__)


class ToolNotFound(RuntimeError):
    pass


class ToolFailed(RuntimeError):
    def __init__(self, tool, returncode, stderr):
        super().__init__("%s failed (exit %s)\nstderr tail:\n%s" % (tool, returncode, stderr[-2000:]))
        self.returncode = returncode
        self.stderr = stderr


@contextlib.contextmanager
def tmpdir_manager(base_dir: Optional[str] = None):
    """A scratch directory that disappears when the block ends (fastfold/data/tools/utils.py:27-34)."""
    d = tempfile.mkdtemp(dir=base_dir)
    try:
        yield d
    finally:
        shutil.rmtree(d, ignore_errors=True)


@contextlib.contextmanager
def timing(msg: str):
    log.info("Started %s", msg)
    t0 = time.perf_counter()
    yield
    log.info("Finished %s in %.3f seconds", msg, time.perf_counter() - t0)


def to_date(s: str):
    return datetime.datetime(year=int(s[:4]), month=int(s[5:7]), day=int(s[8:10]))


def _need_binary(path, name):
    found = shutil.which(path) if path else None
    if not found:
        raise ToolNotFound("%s binary not found at %r" % (name, path))
    return found


def _run(cmd, tool, stdin_text=None):
    log.info("Launching subprocess %s", " ".join(cmd))
    with timing(tool):
        p = subprocess.run(cmd, input=stdin_text, capture_output=True, text=True)
    if p.returncode != 0:
        raise ToolFailed(tool, p.returncode, p.stderr)
    return p.stdout, p.stderr


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


class HHBlits:
    """Iterative HMM-HMM search against HH-suite databases (fastfold/data/tools/hhblits.py:30-181)."""

    def __init__(self, *, binary_path: str, databases: Sequence[str], n_cpu: int = 4, n_iter: int = 3, e_value: float = 0.001,
                 maxseq: int = 1_000_000, realign_max: int = 100_000, maxfilt: int = 100_000, min_prefilter_hits: int = 1000,
                 all_seqs: bool = False, alt: Optional[int] = None, p: int = 20, z: int = 500):
        self.binary_path = _need_binary(binary_path, "hhblits")
        self.databases = list(databases)
        for db in self.databases:
            if not glob.glob(db + "_*"):
                raise ValueError("Could not find HHBlits database %s" % db)
        self.n_cpu, self.n_iter, self.e_value, self.maxseq = n_cpu, n_iter, e_value, maxseq
        self.realign_max, self.maxfilt, self.min_prefilter_hits = realign_max, maxfilt, min_prefilter_hits
        self.all_seqs, self.alt, self.p, self.z = all_seqs, alt, p, z

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
            for db in self.databases:
                cmd += ["-d", db]
            stdout, stderr = _run(cmd, "HHblits")
            a3m_text = open(a3m).read()
        return dict(a3m=a3m_text, output=stdout, stderr=stderr, n_iter=self.n_iter, e_value=self.e_value)


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


class HHFilter:
    """Redundancy filter of an A3M (``hhfilter -id``); used by the workflow between search stages."""

    def __init__(self, *, binary_path: str, id: int = 90, cov: int = 0):
        self.binary_path = _need_binary(binary_path, "hhfilter")
        self.id, self.cov = id, cov

    def query(self, a3m_path: str, output_path: str) -> str:
        _run([self.binary_path, "-i", a3m_path, "-o", output_path, "-id", str(self.id), "-cov", str(self.cov)], "HHfilter")
        return output_path


class Hmmbuild:
    """Profile HMM from an alignment (fastfold/data/tools/hmmbuild.py:25-137)."""

    def __init__(self, *, binary_path: str, singlemer: bool = False):
        self.binary_path = _need_binary(binary_path, "hmmbuild")
        self.singlemer = singlemer

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
            if self.singlemer:
                cmd.append("--singlemx")
            _run(cmd + ["--amino", out, inp], "hmmbuild")
            return open(out).read()


class Hmmsearch:
    """Search a profile HMM against a sequence database (fastfold/data/tools/hmmsearch.py:27-139)."""

    def __init__(self, *, binary_path: str, hmmbuild_binary_path: str, database_path: str, flags: Optional[Sequence[str]] = None):
        self.binary_path = _need_binary(binary_path, "hmmsearch")
        self.hmmbuild_runner = Hmmbuild(binary_path=hmmbuild_binary_path)
        if not os.path.exists(database_path):
            raise ValueError("Could not find hmmsearch database %s" % database_path)
        self.database_path = database_path
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
            cmd = [self.binary_path, "--noali", "--cpu", "8"] + self.flags + ["-A", sto, hmm_path, self.database_path]
            _run(cmd, "hmmsearch (%s)" % os.path.basename(self.database_path))
            return open(sto).read()

    def get_template_hits(self, output_string: str, input_sequence: str):
        from .. import parsers
        a3m = parsers.convert_stockholm_to_a3m(output_string, remove_first_row_gaps=False)
        return parsers.parse_hmmsearch_a3m(query_sequence=input_sequence, a3m_string=a3m, skip_first=False)


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
