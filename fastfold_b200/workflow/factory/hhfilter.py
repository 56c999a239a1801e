"""Task nodes that thin an alignment with hhfilter (fastfold/workflow/factory/hhfilter.py:10-32)."""
from typing import List, Optional

from ...data import tools
from ..dag import TaskNode
from .task_factory import TaskFactory

class HHfilterFactory(TaskFactory):
    keywords = ["binary_path"]

    def gen_node(self, fasta_path: str, output_path: str, after: Optional[List[TaskNode]] = None) -> TaskNode:
        self.isReady()
        cfg = dict(self.config)

        def hhfilter_node_func():
            runner = tools.HHFilter(binary_path=cfg["binary_path"], id=cfg.get("id", 90), cov=cfg.get("cov", 0))
            return runner.query(fasta_path, output_path)

        return TaskNode(hhfilter_node_func, after, name="hhfilter:%s" % output_path)
