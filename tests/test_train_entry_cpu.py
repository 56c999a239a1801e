"""``train.py`` end to end on the CPU: the reference's data path (filtered mixture dataset over PDB files with a chain
cache, batch collator, loader with per-batch properties) feeding two optimiser steps of a one-block model."""
import json
import os
import subprocess
import sys

from test_data_modules_cpu import _tree

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_train_py_on_pdb_files(tmp_path):
    names = {"1abc": "ACDEFGHIKLMNPQRSTVWY", "2xyz": "MNPQRSTVWYACDEFGHIKL", "4def": "ACDEFGHIKLACDEFGHIKLMN"}
    data, aln, cache = _tree(tmp_path, names)
    cache_path = tmp_path / "chain_cache.json"
    cache_path.write_text(json.dumps(cache))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--train_data_dir", data, "--train_alignment_dir", aln,
           "--train_chain_data_cache_path", str(cache_path), "--blocks", "1", "--n_res", "16", "--n_seq", "4", "--n_extra", "4",
           "--max_steps", "2", "--train_epoch_len", "2", "--max_epochs", "1", "--val_epoch_len", "0", "--log_interval", "1",
           "--log_path", str(tmp_path / "log"), "--seed", "3"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    log = (tmp_path / "log.log").read_text()
    assert log.count(" loss ") >= 2 and "nan" not in log.lower(), log[-1500:]


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(tmp_path, tag, dap):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
           str(_free_port()), os.path.join(ROOT, "train.py"), "--dap_size", str(dap), "--blocks", "1", "--n_res", "16", "--n_seq", "4", "--n_extra", "4",
           "--max_steps", "2", "--train_epoch_len", "4", "--max_epochs", "1", "--val_epoch_len", "2", "--log_interval", "1",
           "--log_path", str(tmp_path / tag), "--seed", "3"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return (tmp_path / (tag + ".log")).read_text()


def test_train_py_on_two_ranks_dap_and_dp(tmp_path):
    """Two Gloo ranks on synthetic data: as one DAP group (one replica, sharded activations) and as two data-parallel
    replicas (the epoch summary counts the replicas)."""
    dap = _launch(tmp_path, "dap", 2)
    assert dap.count(" loss ") >= 2 and "nan" not in dap.lower() and "over 1 replica(s)" in dap, dap[-1500:]
    assert "validation epoch 0 (2 samples)" in dap and "gdt_ts" in dap, dap[-1500:]
    dp = _launch(tmp_path, "dp", 1)
    assert dp.count(" loss ") >= 2 and "nan" not in dp.lower() and "over 2 replica(s)" in dp, dp[-1500:]
    assert "validation epoch 0 (4 samples)" in dp, dp[-1500:]           # two synthetic samples per replica, summed over the replicas


def test_train_py_on_mmcif_targets_with_templates(tmp_path):
    """mmCIF training targets with alignment directories that hold template hits, a template structure directory and a
    release-date margin: the template path of the training data pipeline feeds the model (one block, two steps)."""
    sys.path.insert(0, os.path.join(ROOT, "tests", "helpers"))
    from synthetic_mmcif import cif_text
    core = "ACMEFGRIKLMNPQ"
    data, mm, aln = tmp_path / "data", tmp_path / "mmcif", tmp_path / "aln"
    for p in (data, mm, aln):
        p.mkdir()
    (mm / "1abc.cif").write_text(cif_text("1abc", "1999-05-01", {"A": ("A", "W" + core[1:])}))
    cache = {}
    for name, seq in {"4tgt_A": "MM" + core + "WW", "5tgt_A": "GG" + core + "KK"}.items():
        (data / (name[:4] + ".cif")).write_text(cif_text(name[:4], "2005-03-01", {"A": ("A", seq)}))
        d = aln / name
        d.mkdir()
        (d / "bfd_uniclust_hits.a3m").write_text(">query\n%s\n>h1\n%s\n>h2\n%s\n" % (seq, seq[:-1] + "A", "A" + seq[1:]))
        (d / "pdb70_hits.hhr").write_text(
            "Query         query\nMatch_columns 18\n\nNo 1\n>1abc_A template\n"
            "Probab=99.00  E-value=1e-10  Score=50.00  Aligned_cols=14  Identities=90%  Similarity=1.500  Sum_probs=13.5  Template_Neff=5.000\n\n"
            "Q query             3 ACMEFGRIKLMNPQ   16 (18)\nQ Consensus         3 acmefgriklmnpq   16 (18)\n                      ||||||||||||||\n"
            "T Consensus         1 wcmefgriklmnpq   14 (14)\nT 1abc_A            1 WCMEFGRIKLMNPQ   14 (14)\n\n")
        cache[name] = {"seq": seq, "resolution": 1.8, "cluster_size": 1, "release_date": "2005-03-01"}
    cache_path = tmp_path / "chain_cache.json"
    cache_path.write_text(json.dumps(cache))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--train_data_dir", str(data), "--train_alignment_dir", str(aln),
           "--train_chain_data_cache_path", str(cache_path), "--template_mmcif_dir", str(mm), "--max_template_date", "2020-01-01",
           "--blocks", "1", "--n_res", "16", "--n_seq", "4", "--n_extra", "4", "--max_steps", "2", "--train_epoch_len", "2", "--max_epochs", "1",
           "--val_epoch_len", "0", "--log_interval", "1", "--log_path", str(tmp_path / "log"), "--seed", "3"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    log = (tmp_path / "log.log").read_text()
    assert log.count(" loss ") >= 2 and "nan" not in log.lower(), log[-1500:]
