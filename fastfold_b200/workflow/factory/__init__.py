"""Factories that turn a tool configuration into workflow nodes (fastfold/workflow/factory/*.py)."""
from .hhblits import HHBlitsFactory
from .hhfilter import HHfilterFactory
from .hhsearch import HHSearchFactory
from .hmmsearch import HmmSearchFactory
from .jackhmmer import JackHmmerFactory
from .task_factory import TaskFactory

__all__ = ["TaskFactory", "JackHmmerFactory", "HHBlitsFactory", "HHSearchFactory", "HHfilterFactory", "HmmSearchFactory"]
