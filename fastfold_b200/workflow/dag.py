"""A small dependency-graph executor for the pre-processing workflow.

The reference builds its alignment workflow from ``ray.remote`` function nodes and runs it with ``ray.workflow``
(fastfold/workflow/workflow_run.py:7-14, factory/task_factory.py:8-50).  Every task there is one long-running
subprocess on the local machine, so this framework schedules the same graphs with a thread pool: a node starts as soon
as all of its predecessors have finished; independent nodes run side by side; the first failure cancels whatever has
not started and is re-raised with the name of the failing node.
"""
import threading
from concurrent.futures import FIRST_COMPLETED, ThreadPoolExecutor, wait
from typing import Callable, Iterable, List, Optional, Sequence


class TaskNode:
    """One unit of work: ``fn()`` runs after every node in ``after`` has finished."""

    _ids = iter(range(1 << 62))
    _lock = threading.Lock()

    def __init__(self, fn: Callable[[], object], after: Optional[Sequence["TaskNode"]] = None, name: Optional[str] = None):
        with TaskNode._lock:
            self.id = next(TaskNode._ids)
        self.fn = fn
        self.after: List[TaskNode] = [a for a in (after or []) if a is not None]
        self.name = name or getattr(fn, "__name__", "task")
        self.result = None
        self.done = False

    def __repr__(self):
        return "TaskNode(%s#%d, after=%s)" % (self.name, self.id, [a.name for a in self.after])


class WorkflowError(RuntimeError):
    pass


def collect(targets: Iterable[TaskNode]) -> List[TaskNode]:
    """Every node reachable from ``targets`` through ``after`` edges, predecessors first; raises on a cycle."""
    order, state = [], {}

    def visit(n, path):
        s = state.get(n.id)
        if s == 2:
            return
        if s == 1:
            raise WorkflowError("dependency cycle through %s" % " -> ".join(p.name for p in path + [n]))
        state[n.id] = 1
        for a in n.after:
            visit(a, path + [n])
        state[n.id] = 2
        order.append(n)

    for t in targets:
        visit(t, [])
    return order


def run_dag(targets: Sequence[TaskNode], max_workers: Optional[int] = None) -> List[object]:
    """Run the graph that ends in ``targets``; returns the targets' results in order."""
    nodes = collect(targets)
    pending = {n.id: n for n in nodes if not n.done}
    running = {}
    with ThreadPoolExecutor(max_workers=max_workers or max(1, len(nodes))) as pool:
        while pending or running:
            ready = [n for n in pending.values() if all(a.done for a in n.after)]
            for n in ready:
                del pending[n.id]
                running[pool.submit(n.fn)] = n
            if not running:
                raise WorkflowError("no runnable task left; unfinished: %s" % [n.name for n in pending.values()])
            finished, _ = wait(list(running), return_when=FIRST_COMPLETED)
            for fut in finished:
                n = running.pop(fut)
                err = fut.exception()
                if err is not None:
                    for other in running:
                        other.cancel()
                    raise WorkflowError("task %s failed: %s" % (n.name, err)) from err
                n.result, n.done = fut.result(), True
    return [t.result for t in targets]
