"""Task nodes that run jackhmmer (fastfold/workflow/factory/jackhmmer.py:12-44)."""
from typing import List, Optional

from ...data import parsers, tools
from ..dag import TaskNode
from .task_factory import TaskFactory

class JackHmmerFactory(TaskFactory):
    keywords = ["binary_path", "database_path", "n_cpu", "uniref_max_hits"]

    def gen_node(self, fasta_path: str, output_path: str, after: Optional[List[TaskNode]] = None, output_format: str = "a3m") -> TaskNode:
        self.isReady()
        cfg = dict(self.config)

        def jackhmmer_node_func():
            runner = tools.Jackhmmer(binary_path=cfg["binary_path"], database_path=cfg["database_path"], n_cpu=cfg["n_cpu"])
            sto = runner.query(fasta_path)[0]["sto"]
            text = sto if output_format == "sto" else parsers.convert_stockholm_to_a3m(sto, max_sequences=cfg["uniref_max_hits"])
            with open(output_path, "w") as f:
                f.write(text)
            return output_path

        return TaskNode(jackhmmer_node_func, after, name="jackhmmer:%s" % output_path)
