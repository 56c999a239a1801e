"""Per-module tracing: NVTX ranges and device-timed module calls, reduced over ranks.

The reference offers a ``torch.profiler`` trace (benchmark/perf.py:122-132) and wall-clock prints around whole phases
(inference.py:150-152, data/tools/utils.py:37).  Two finer tools here:

* ``annotate(model)`` wraps the forward of every selected sub-module in an NVTX range named by its path in the model,
  so a timeline viewer shows which module a kernel belongs to.  Free when no tool listens.
* ``ModuleTimer(model)`` times every call of the selected sub-modules with CUDA events on the current stream (host clock
  for CPU tensors) and reports, per module path or per module class, calls / total / mean milliseconds as the MAX over
  the ranks of the process group - the number that bounds a step when ranks wait for one another.

Both select modules by depth below the root, by class, or by a predicate, and both are removed with ``.remove()`` (or by
leaving the ``with`` block).  Events are not recorded while a CUDA graph is being captured: a captured event has no
timestamp, so a timer that is active during capture records nothing for those calls.
"""
import contextlib
import time
from collections import OrderedDict

import torch

__all__ = ["annotate", "ModuleTimer", "select_modules", "nvtx_range", "timed_region"]


def select_modules(model, max_depth=None, classes=None, predicate=None, include_root=False):
    """``[(path, module)]`` of the sub-modules to instrument.  ``max_depth``: dots in the path + 1 (1 = direct children);
    ``classes``: tuple of types or class names; ``predicate(path, module) -> bool``.  Containers without a forward of
    their own (``ModuleList`` / ``ModuleDict`` / ``Sequential`` shells are kept: they do run) are skipped."""
    names = tuple(c for c in (classes or ()) if isinstance(c, str))
    types = tuple(c for c in (classes or ()) if not isinstance(c, str))
    out = []
    for path, mod in model.named_modules():
        if path == "":
            if include_root:
                out.append((type(model).__name__, mod))
            continue
        if isinstance(mod, (torch.nn.ModuleList, torch.nn.ModuleDict)):
            continue
        if max_depth is not None and path.count(".") + 1 > max_depth:
            continue
        if classes and not (isinstance(mod, types) or type(mod).__name__ in names):
            continue
        if predicate is not None and not predicate(path, mod):
            continue
        out.append((path, mod))
    return out


def _nvtx_ok():
    return torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name):
    """NVTX range around a block of host code (no-op without CUDA)."""
    if _nvtx_ok():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class _Handles:
    def __init__(self):
        self._handles = []

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove()
        return False


class annotate(_Handles):
    """``with annotate(model, max_depth=3): model(batch)`` - one NVTX range per selected module call, named by module path
    and class (``evoformer.blocks.0.msa [MSAStack]``).  Ranges nest as the modules do."""

    def __init__(self, model, **select):
        super().__init__()
        self.active = _nvtx_ok()
        self.names = []
        for path, mod in select_modules(model, **select):
            label = "%s [%s]" % (path, type(mod).__name__)
            self.names.append(label)
            if not self.active:
                continue
            self._handles.append(mod.register_forward_pre_hook(self._push(label)))
            self._handles.append(mod.register_forward_hook(self._pop, always_call=True))

    @staticmethod
    def _push(label):
        def hook(module, args):
            torch.cuda.nvtx.range_push(label)
        return hook

    @staticmethod
    def _pop(module, args, output):
        torch.cuda.nvtx.range_pop()


class _Span:
    __slots__ = ("start", "stop", "host")

    def __init__(self, start, stop=None, host=False):
        self.start, self.stop, self.host = start, stop, host


def _on_device(args):
    for a in args:
        if torch.is_tensor(a):
            return a.is_cuda
        if isinstance(a, (list, tuple)):
            for b in a:
                if torch.is_tensor(b):
                    return b.is_cuda
    return torch.cuda.is_available()


class ModuleTimer(_Handles):
    """Times the calls of the selected sub-modules.

    ``summary(by="path" | "class", group=None)`` synchronises the device, converts the recorded event pairs to
    milliseconds and returns ``OrderedDict(name -> {"calls", "total_ms", "mean_ms"})`` where the times are the maximum over
    the ranks of ``group`` (the default group when ``torch.distributed`` is initialised; this rank alone otherwise).
    Nested modules are each timed in full, so a parent's time includes its children's.  ``reset()`` drops what was
    recorded; ``table()`` formats the summary.
    """

    def __init__(self, model, **select):
        super().__init__()
        self._open = {}
        self.spans = OrderedDict()
        self._cls = {}
        self.skipped_in_capture = 0
        for path, mod in select_modules(model, **select):
            self.spans[path] = []
            self._cls[path] = type(mod).__name__
            self._handles.append(mod.register_forward_pre_hook(self._begin(path)))
            self._handles.append(mod.register_forward_hook(self._end(path), always_call=True))

    def _begin(self, path):
        def hook(module, args):
            if _on_device(args):
                if torch.cuda.is_current_stream_capturing():
                    self.skipped_in_capture += 1
                    return
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self._open.setdefault(path, []).append(_Span(ev))
            else:
                self._open.setdefault(path, []).append(_Span(time.perf_counter(), host=True))
        return hook

    def _end(self, path):
        def hook(module, args, output):
            stack = self._open.get(path)
            if not stack:
                return
            span = stack.pop()                      # recursion-safe: innermost call of this module closes first
            if span.host:
                span.stop = time.perf_counter()
            else:
                span.stop = torch.cuda.Event(enable_timing=True)
                span.stop.record()
            self.spans[path].append(span)
        return hook

    def reset(self):
        for v in self.spans.values():
            del v[:]
        self._open.clear()
        self.skipped_in_capture = 0

    def _local(self, by):
        if torch.cuda.is_available() and any(not s.host for v in self.spans.values() for s in v):
            torch.cuda.synchronize()
        acc = OrderedDict()
        for path, spans in self.spans.items():
            key = path if by == "path" else self._cls[path]
            calls, total = acc.get(key, (0, 0.0))
            for s in spans:
                total += (s.stop - s.start) * 1e3 if s.host else s.start.elapsed_time(s.stop)
            acc[key] = (calls + len(spans), total)
        return acc

    def summary(self, by="path", group=None):
        assert by in ("path", "class")
        acc = self._local(by)
        names = list(acc)
        calls = torch.tensor([acc[n][0] for n in names], dtype=torch.float64)
        total = torch.tensor([acc[n][1] for n in names], dtype=torch.float64)
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1 and names:
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
            both = torch.stack([calls, total]).to(dev)
            dist.all_reduce(both, op=dist.ReduceOp.MAX, group=group)
            calls, total = both.cpu()
        out = OrderedDict()
        for n, c, t in zip(names, calls.tolist(), total.tolist()):
            out[n] = {"calls": int(c), "total_ms": t, "mean_ms": t / c if c else 0.0}
        return out

    def table(self, by="class", group=None, top=None):
        rows = sorted(self.summary(by, group).items(), key=lambda kv: -kv[1]["total_ms"])
        if top:
            rows = rows[:top]
        width = max([len(n) for n, _ in rows] + [6])
        lines = ["%-*s %8s %12s %10s" % (width, "module", "calls", "total ms", "mean ms")]
        for n, r in rows:
            lines.append("%-*s %8d %12.3f %10.4f" % (width, n, r["calls"], r["total_ms"], r["mean_ms"]))
        return "\n".join(lines)


@contextlib.contextmanager
def timed_region(result, key="ms", sync=True):
    """``with timed_region(d): ...`` stores the elapsed milliseconds of the block in ``d[key]``: CUDA events on the current
    stream with a synchronise on both sides when a GPU is present, host clock otherwise.  (The reference reads the host
    clock without synchronising, inference.py:150-152, which under-reports asynchronous GPU work.)"""
    if torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
        if sync:
            torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        b.synchronize()
        result[key] = a.elapsed_time(b)
    else:
        t0 = time.perf_counter()
        yield
        result[key] = (time.perf_counter() - t0) * 1e3
