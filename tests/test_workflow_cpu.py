"""Alignment tool wrappers, alignment runner and the workflow scheduler, driven by stand-in binaries (shell scripts)."""
import os
import stat
import threading
import time

import pytest

from fastfold_b200.data import parsers, tools
from fastfold_b200.data.data_pipeline import AlignmentRunner, DataPipeline
from fastfold_b200.workflow import TaskNode, WorkflowError, run_dag
from fastfold_b200.workflow.template import FastFoldDataWorkFlow

STO = "# STOCKHOLM 1.0\\n#=GS query DE test\\nquery ACDEFGHIKL\\nhit1  ACDE-GHIKL\\nhit2  ACDEFGHIKV\\n//\\n"
HHR = """Query         query
Match_columns 10

No 1
>1abc_A test template
Probab=99.0  E-value=1e-10  Score=50.0  Aligned_cols=10  Identities=100%  Similarity=1.5  Sum_probs=9.5  Template_Neff=5.0

Q query             1 ACDEFGHIKL   10 (10)
Q Consensus         1 acdefghikl   10 (10)
                      ||||||||||
T Consensus         1 acdefghikl   10 (10)
T 1abc_A            1 ACDEFGHIKL   10 (10)
"""


def _script(path, body):
    with open(path, "w") as f:
        f.write("#!/bin/bash\n" + body)
    os.chmod(path, os.stat(path).st_mode | stat.S_IEXEC)
    return str(path)


@pytest.fixture
def fake_tools(tmp_path):
    # jackhmmer: -A <sto> is the 4th/5th argument; hhblits: -oa3m <path>; hhsearch: -o <path>
    jack = _script(tmp_path / "jackhmmer", 'while [ $# -gt 0 ]; do if [ "$1" = "-A" ]; then out=$2; fi; shift; done\nprintf "%s" > $out\n' % STO)
    hhb = _script(tmp_path / "hhblits", 'while [ $# -gt 0 ]; do if [ "$1" = "-oa3m" ]; then out=$2; fi; shift; done\nprintf ">query\\nACDEFGHIKL\\n>b1\\nACDEFGHIKL\\n" > $out\n')
    hhs = _script(tmp_path / "hhsearch", 'while [ $# -gt 0 ]; do if [ "$1" = "-o" ]; then out=$2; fi; shift; done\ncat > $out <<"XX"\n%sXX\n' % HHR)
    db = tmp_path / "db.fasta"
    db.write_text(">x\nACDEFGHIKL\n")
    (tmp_path / "bfd_hhm.ffdata").write_text("")
    (tmp_path / "pdb70_hhm.ffdata").write_text("")
    fasta = tmp_path / "q.fasta"
    fasta.write_text(">query\nACDEFGHIKL\n")
    return dict(jack=jack, hhb=hhb, hhs=hhs, db=str(db), bfd=str(tmp_path / "bfd"), pdb70=str(tmp_path / "pdb70"), fasta=str(fasta), dir=tmp_path)


def test_missing_binary_is_reported():
    with pytest.raises(tools.ToolNotFound):
        tools.Kalign(binary_path="/nonexistent/kalign")


def test_wrappers_and_runner(fake_tools):
    t = fake_tools
    res = tools.Jackhmmer(binary_path=t["jack"], database_path=t["db"]).query(t["fasta"])
    assert "hit1" in res[0]["sto"]
    out = str(t["dir"] / "aln")
    AlignmentRunner(jackhmmer_binary_path=t["jack"], hhblits_binary_path=t["hhb"], hhsearch_binary_path=t["hhs"], uniref90_database_path=t["db"],
                    mgnify_database_path=t["db"], bfd_database_path=t["bfd"], pdb70_database_path=t["pdb70"], no_cpus=1).run(t["fasta"], out)
    assert sorted(os.listdir(out)) == ["bfd_uniref_hits.a3m", "mgnify_hits.a3m", "pdb70_hits.hhr", "uniref90_hits.a3m"]
    hits = parsers.parse_hhr(open(os.path.join(out, "pdb70_hits.hhr")).read())
    assert hits[0].name.startswith("1abc_A") and hits[0].aligned_cols == 10
    feats = DataPipeline().process_fasta(t["fasta"], out)
    assert feats["msa"].shape[1] == 10 and feats["msa"].shape[0] >= 3


def test_workflow_template(fake_tools):
    t = fake_tools
    out = str(t["dir"] / "wf")
    FastFoldDataWorkFlow(jackhmmer_binary_path=t["jack"], hhblits_binary_path=t["hhb"], hhsearch_binary_path=t["hhs"],
                         uniref90_database_path=t["db"], mgnify_database_path=t["db"], bfd_database_path=t["bfd"],
                         pdb70_database_path=t["pdb70"], no_cpus=1).run(t["fasta"], out)
    assert sorted(os.listdir(out)) == ["bfd_uniref_hits.a3m", "mgnify_hits.a3m", "pdb70_hits.hhr", "uniref90_hits.a3m"]


def test_dag_order_parallelism_and_failure():
    log, lock = [], threading.Lock()

    def mk(name, delay=0.0, fail=False):
        def fn():
            time.sleep(delay)
            if fail:
                raise ValueError("boom")
            with lock:
                log.append(name)
            return name
        return fn

    a = TaskNode(mk("a", 0.05), name="a")
    b = TaskNode(mk("b"), after=[a], name="b")
    c = TaskNode(mk("c"), name="c")
    assert run_dag([b, c]) == ["b", "c"]
    assert log.index("a") < log.index("b") and log.index("c") < log.index("b")     # c did not wait for a
    bad = TaskNode(mk("x", fail=True), name="x")
    never = TaskNode(mk("y"), after=[bad], name="y")
    with pytest.raises(WorkflowError, match="x"):
        run_dag([never])
    assert "y" not in log
    p = TaskNode(mk("p"), name="p")
    q = TaskNode(mk("q"), after=[p], name="q")
    p.after.append(q)
    with pytest.raises(WorkflowError, match="cycle"):
        run_dag([q])
