"""Task nodes that run hhblits (fastfold/workflow/factory/hhblits.py:10-29)."""
from typing import List, Optional

from ...data import tools
from ..dag import TaskNode
from .task_factory import TaskFactory

class HHBlitsFactory(TaskFactory):
    keywords = ["binary_path", "databases", "n_cpu"]

    def gen_node(self, fasta_path: str, output_path: str, after: Optional[List[TaskNode]] = None) -> TaskNode:
        self.isReady()
        cfg = dict(self.config)

        def hhblits_node_func():
            runner = tools.HHBlits(binary_path=cfg["binary_path"], databases=cfg["databases"], n_cpu=cfg["n_cpu"])
            with open(output_path, "w") as f:
                f.write(runner.query(fasta_path)["a3m"])
            return output_path

        return TaskNode(hhblits_node_func, after, name="hhblits:%s" % output_path)
