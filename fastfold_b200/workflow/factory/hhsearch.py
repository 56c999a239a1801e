"""Task nodes that run hhsearch on an alignment and keep its HHR output (fastfold/workflow/factory/hhsearch.py:11-42)."""
from typing import List, Optional

from ...data import tools
from ..dag import TaskNode
from .task_factory import TaskFactory

class HHSearchFactory(TaskFactory):
    keywords = ["binary_path", "databases", "n_cpu"]

    def gen_node(self, a3m_path: str, output_path: str, atab_path: Optional[str] = None, after: Optional[List[TaskNode]] = None) -> TaskNode:
        self.isReady()
        cfg = dict(self.config)

        def hhsearch_node_func():
            runner = tools.HHSearch(binary_path=cfg["binary_path"], databases=cfg["databases"], n_cpu=cfg["n_cpu"])
            a3m = open(a3m_path).read()
            if atab_path:
                hhr, atab = runner.query(a3m, gen_atab=True)
                with open(atab_path, "w") as f:
                    f.write(atab)
            else:
                hhr = runner.query(a3m)
            with open(output_path, "w") as f:
                f.write(hhr)
            return output_path

        return TaskNode(hhsearch_node_func, after, name="hhsearch:%s" % output_path)
