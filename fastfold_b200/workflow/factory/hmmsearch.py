"""Task nodes that run hmmbuild + hmmsearch, the multimer template search (fastfold/workflow/factory/hmmsearch.py:12-41)."""
from typing import List, Optional

from ...data import parsers, tools
from ..dag import TaskNode
from .task_factory import TaskFactory

class HmmSearchFactory(TaskFactory):
    keywords = ["binary_path", "hmmbuild_binary_path", "database_path", "n_cpu"]

    def gen_node(self, msa_sto_path: str, output_dir: Optional[str] = None, after: Optional[List[TaskNode]] = None) -> TaskNode:
        self.isReady()
        cfg = dict(self.config)

        def hmmsearch_node_func():
            runner = tools.Hmmsearch(binary_path=cfg["binary_path"], hmmbuild_binary_path=cfg["hmmbuild_binary_path"],
                                     database_path=cfg["database_path"])
            sto = open(msa_sto_path).read()
            sto = parsers.remove_empty_columns_from_stockholm_msa(parsers.deduplicate_stockholm_msa(sto))
            return runner.query(sto, output_dir=output_dir)

        return TaskNode(hmmsearch_node_func, after, name="hmmsearch:%s" % msa_sto_path)
