"""Base class of the task factories: a ``config`` dict (given, or read from ``./config.json``) and the list of entries a factory needs (fastfold/workflow/factory/task_factory.py:12-50)."""
import json
from typing import List, Optional

from ..dag import TaskNode

class TaskFactory:
    """Holds a ``config`` dict; ``keywords`` lists the entries a subclass needs before it can make nodes.

    With neither ``config`` nor ``config_path`` the entry named after the factory (class name minus ``Factory``) is read
    from the ``tools`` section of ``./config.json`` (fastfold/workflow/factory/task_factory.py:12-50).
    """

    keywords: List[str] = []

    def __init__(self, config: Optional[dict] = None, config_path: Optional[str] = None) -> None:
        self.config = {}
        if not self.__class__.keywords:
            return
        if config is not None:
            self.config = dict(config)
        else:
            self.loadConfig(config_path or "./config.json")

    def configure(self, *args, purge: bool = False) -> None:
        """``configure({..})`` merges (or, with ``purge``, replaces) the config; ``configure(key, value)`` sets one entry."""
        if len(args) == 1 and isinstance(args[0], dict):
            self.config = dict(args[0]) if purge else {**self.config, **args[0]}
        elif len(args) == 2:
            self.config[args[0]] = args[1]
        else:
            raise TypeError("configure(dict) or configure(keyword, value)")

    def gen_task(self, after: Optional[List[TaskNode]] = None, *args, **kwargs) -> TaskNode:
        raise NotImplementedError

    def isReady(self) -> None:
        for key in self.__class__.keywords:
            if key not in self.config:
                raise KeyError('%s not ready: "%s" not specified' % (self.__class__.__name__, key))

    def loadConfig(self, config_path: str = "./config.json") -> None:
        with open(config_path) as f:
            cfg = json.load(f)
        if "tools" not in cfg:
            raise KeyError('"tools" not found in global config file')
        name = self.__class__.__name__[: -len("Factory")]
        if name not in cfg["tools"]:
            raise KeyError('"%s" not found in the "tools" section in config' % name)
        self.config = cfg["tools"][name]
