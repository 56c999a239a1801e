"""Shared helpers of the tool wrappers: scratch directories, timing, date parsing, locating a binary and running it
(fastfold/data/tools/utils.py:27-48)."""
import contextlib
import datetime
import logging
import shutil
import subprocess
import tempfile
import time
from typing import Optional

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
