"""Factories that turn a tool configuration into workflow nodes (fastfold/workflow/factory/*.py)."""
import json
from typing import List, Optional

from ...data import parsers, tools
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


class HHfilterFactory(TaskFactory):
    keywords = ["binary_path"]

    def gen_node(self, fasta_path: str, output_path: str, after: Optional[List[TaskNode]] = None) -> TaskNode:
        self.isReady()
        cfg = dict(self.config)

        def hhfilter_node_func():
            runner = tools.HHFilter(binary_path=cfg["binary_path"], id=cfg.get("id", 90), cov=cfg.get("cov", 0))
            return runner.query(fasta_path, output_path)

        return TaskNode(hhfilter_node_func, after, name="hhfilter:%s" % output_path)


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
