"""``batch_run``: run several workflow graphs as one job (fastfold/workflow/workflow_run.py:7-14)."""
from typing import List, Optional

from .dag import TaskNode, run_dag


def batch_run(workflow_id: str, dags: List[TaskNode], max_workers: Optional[int] = None) -> None:
    print("Workflow %r started." % workflow_id)
    run_dag(list(dags), max_workers=max_workers)
    print("Workflow %r finished." % workflow_id)
