"""``inference.py`` end to end on CPU ranks: FASTA -> features -> model (parameter archive, fast trunk) -> PDB.

Follows the reference's tests/test_inference.py:30-76 (world size 1 / 2, chunking, in-place; final atom positions against
the un-injected OpenFold-layout model within 5e-4 A) with a reduced model and a synthetic parameter archive written in the
AlphaFold naming, so the archive import, the weight injection and the entry point are all on the path.
"""
import os
import pickle
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEQ = "MKTAYIAKQRQISFVKSHFSRQ"
OVERRIDES = {"model.evoformer_stack.no_blocks": 2, "model.extra_msa.extra_msa_stack.no_blocks": 1, "model.structure_module.no_blocks": 2}


def _config():
    from fastfold_b200.config import model_config
    config = model_config("model_3")
    for k, v in OVERRIDES.items():
        node = config
        parts = k.split(".")
        for p in parts[:-1]:
            node = node[p]
        node[parts[-1]] = v
    return config


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    """FASTA file + a parameter archive of a reduced model_3 whose zero-initialised layers are randomised (with the stock
    initialisation every residual branch ends in a zero layer and the structure would not depend on the trunk)."""
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.utils.import_weights import export_jax_weights
    d = tmp_path_factory.mktemp("inference_entry")
    (d / "q.fasta").write_text(">q1 test\n%s\n" % SEQ)
    torch.manual_seed(0)
    model = AlphaFold(_config())
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in model.parameters():
            if float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g) * (0.02 if p.dim() < 2 else 0.5 / p.shape[-1] ** 0.5))
    np.savez(str(d / "params_model_3.npz"), **export_jax_weights(model, "model_3"))
    return d


def _run_entry(workdir, out, gpus, extra=()):
    cmd = [sys.executable, os.path.join(ROOT, "inference.py"), "q.fasta", "none", "--output_dir", out, "--gpus", str(gpus), "--model_name", "model_3",
           "--param_path", "params_model_3.npz", "--save_prediction_result", "--data_random_seed", "3"]
    for k, v in OVERRIDES.items():
        cmd += ["--config_override", "%s=%s" % (k, v)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_PORT=str(19000 + os.getpid() % 2000 + 7 * gpus))
    r = subprocess.run(cmd + list(extra), cwd=str(workdir), env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    with open(os.path.join(str(workdir), out, "q1_model_3_output_dict.pkl"), "rb") as fh:
        return pickle.load(fh), r.stdout


def _reference_layout_prediction(workdir):
    """The same prediction from the OpenFold-layout model, in process: no fast trunk, no chunking, one rank."""
    from fastfold_b200.data.data_pipeline import DataPipeline, FeaturePipeline
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.utils.import_weights import import_jax_weights_
    config = _config()
    config.model.template.enabled = False
    raw = DataPipeline(template_featurizer=None).process_sequence(SEQ, "q1", None)
    feats = FeaturePipeline(config.data).process_features(raw, mode="predict", seed=3, is_multimer=False)
    torch.manual_seed(0)
    model = AlphaFold(config)
    import_jax_weights_(model, str(workdir / "params_model_3.npz"), version="model_3")
    with torch.no_grad():
        out = model.eval()(feats)
    return out


def test_entry_point_matches_the_reference_layout_model_on_one_and_two_ranks(workdir):
    want = _reference_layout_prediction(workdir)
    pos = want["final_atom_positions"].numpy()
    mask = want["final_atom_mask"].numpy()[..., None]
    assert float(np.abs(pos * mask).max()) > 3.0              # a structure that depends on the weights, not the identity start
    one, log = _run_entry(workdir, "out1", 1, ["--module_times"])
    assert "evoformer" in log and "structure_module" in log and "Inference time" in log
    assert np.abs((one["final_atom_positions"] - pos) * mask).max() < 5e-4
    assert np.abs(one["plddt"] - want["plddt"].numpy()).max() < 1e-2
    two, _ = _run_entry(workdir, "out2", 2, ["--chunk_size", "4", "--inplace"])
    assert np.abs((two["final_atom_positions"] - pos) * mask).max() < 5e-4
    # the written structure is readable and carries the sequence
    from fastfold_b200.common import protein, residue_constants as rc
    prot = protein.from_pdb_string(open(os.path.join(str(workdir), "out2", "q1_model_3_unrelaxed.pdb")).read())
    assert "".join(rc.restypes[a] for a in prot.aatype) == SEQ
    ca = rc.atom_order["CA"]
    assert np.abs(prot.atom_positions[:, ca] - pos[:, ca]).max() < 2e-3      # PDB columns hold three decimals


def test_config_override_parsing():
    sys.path.insert(0, ROOT)
    import importlib
    inference = importlib.import_module("inference")
    assert inference.parse_overrides(["a.b=3", "c=True", "d=model_1", "e=[1, 2]"]) == {"a.b": 3, "c": True, "d": "model_1", "e": [1, 2]}
    with pytest.raises(ValueError):
        inference.parse_overrides(["novalue"])


def _entry_with_searches(tmp_path, preset, fasta_text, extra):
    """``inference.py`` with database flags: the searches run (against recording stand-in executables), the alignments
    land where the data pipeline reads them, and the reduced model folds the result."""
    sys.path.insert(0, os.path.join(ROOT, "tests", "helpers"))
    from standins import make_tool_standins
    bins = make_tool_standins(tmp_path / "bin")
    (tmp_path / "db.fasta").write_text(">x\nACDEFGHIKL\n")
    for suffix in ("_hhm.ffdata", "_a3m.ffdata", "_cs219.ffdata"):
        (tmp_path / ("hhdb" + suffix)).write_text("")
    (tmp_path / "q.fasta").write_text(fasta_text)
    record = tmp_path / "commands.txt"
    cmd = [sys.executable, os.path.join(ROOT, "inference.py"), "q.fasta", "none", "--output_dir", "out", "--gpus", "1", "--model_preset", preset,
           "--uniref90_database_path", str(tmp_path / "db.fasta"), "--mgnify_database_path", str(tmp_path / "db.fasta"),
           "--bfd_database_path", str(tmp_path / "hhdb"), "--uniclust30_database_path", str(tmp_path / "hhdb"), "--cpus", "2", "--data_random_seed", "1"]
    for tool in ("jackhmmer", "hhblits", "hhsearch", "hmmsearch", "hmmbuild", "kalign"):
        cmd += ["--%s_binary_path" % tool, bins[tool]]
    for k, v in OVERRIDES.items():
        cmd += ["--config_override", "%s=%s" % (k, v)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", RECORD=str(record), MASTER_PORT=str(21000 + os.getpid() % 2000))
    r = subprocess.run(cmd + list(extra), cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return record.read_text().splitlines(), r.stdout


def test_entry_point_runs_the_monomer_searches(tmp_path):
    commands, log = _entry_with_searches(tmp_path, "monomer", ">q1 test\n%s\n" % SEQ,
                                         ["--model_name", "model_3", "--pdb70_database_path", str(tmp_path / "hhdb")])
    tools = sorted(c.split()[0] for c in commands)
    assert tools == ["hhblits", "hhsearch", "jackhmmer", "jackhmmer"], tools
    assert sorted(os.listdir(tmp_path / "out" / "alignments" / "q1")) == ["bfd_uniref_hits.a3m", "mgnify_hits.a3m", "pdb70_hits.hhr", "uniref90_hits.a3m"]
    assert "Alignment data workflow time" in log and os.path.exists(tmp_path / "out" / "q1_model_3_unrelaxed.pdb")


def test_entry_point_runs_the_multimer_searches_per_chain(tmp_path):
    fasta = ">A first\n%s\n>B second\n%s\n>C copy of the first\n%s\n" % (SEQ, SEQ[::-1], SEQ)
    commands, log = _entry_with_searches(tmp_path, "multimer", fasta, ["--uniprot_database_path", str(tmp_path / "db.fasta"),
                                                                       "--pdb_seqres_database_path", str(tmp_path / "db.fasta"), "--enable_workflow"])
    tools = sorted(c.split()[0] for c in commands)
    # two distinct chains: uniref90, mgnify and uniprot searches, one hhblits and one template search (profile + search) each
    assert tools == sorted(["jackhmmer"] * 6 + ["hhblits"] * 2 + ["hmmbuild"] * 2 + ["hmmsearch"] * 2), tools
    for chain in ("A", "B", "C"):
        files = sorted(os.listdir(tmp_path / "out" / "alignments" / chain))
        assert files == ["bfd_uniref_hits.a3m", "hmm_output.sto", "mgnify_hits.sto", "uniprot_hits.sto", "uniref90_hits.sto"], (chain, files)
    from fastfold_b200.common import protein
    prot = protein.from_pdb_string(open(tmp_path / "out" / "A_multimer_unrelaxed.pdb").read())
    assert prot.aatype.shape[0] == 3 * len(SEQ) and len(set(prot.chain_index.tolist())) == 3
