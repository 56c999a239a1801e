#!/usr/bin/env python
"""Structure prediction from a FASTA file.

    python inference.py target.fasta data/pdb_mmcif/mmcif_files --output_dir ./out --gpus 2 \
        --use_precomputed_alignments ./alignments --model_name model_1 --param_path data/params/params_model_1.npz \
        --chunk_size 64 --inplace

Flags follow the reference's inference.py:68-119,491-551.  Alignments are read from
``--use_precomputed_alignments`` (one sub-directory per FASTA tag) or produced by the alignment tools when their
binaries and databases are given (``--enable_workflow`` runs the searches concurrently); without either the query
is folded in single-sequence mode.  Without ``--param_path`` the model keeps its random initialisation (useful for
timing only).  Outputs: ``<tag>_<model>.pdb`` (+ ``.pkl`` with ``--save_prediction_result``), optionally relaxed.
"""
import argparse
import os
import pickle
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def add_data_args(parser):
    for name in ("uniref90_database_path", "mgnify_database_path", "pdb70_database_path", "uniclust30_database_path", "bfd_database_path",
                 "uniprot_database_path", "pdb_seqres_database_path"):
        parser.add_argument("--" + name, type=str, default=None)
    # UniRef30 is the successor of UniClust30 and is searched the same way (hhblits); either flag names the database
    parser.add_argument("--uniref30_database_path", dest="uniclust30_database_path", type=str, default=None)
    parser.add_argument("--jackhmmer_binary_path", type=str, default="/usr/bin/jackhmmer")
    parser.add_argument("--hhblits_binary_path", type=str, default="/usr/bin/hhblits")
    parser.add_argument("--hhsearch_binary_path", type=str, default="/usr/bin/hhsearch")
    parser.add_argument("--hmmsearch_binary_path", type=str, default="/usr/bin/hmmsearch")
    parser.add_argument("--hmmbuild_binary_path", type=str, default="/usr/bin/hmmbuild")
    parser.add_argument("--kalign_binary_path", type=str, default="/usr/bin/kalign")
    parser.add_argument("--max_template_date", type=str, default="2100-01-01")
    parser.add_argument("--obsolete_pdbs_path", type=str, default=None)
    parser.add_argument("--release_dates_path", type=str, default=None)
    parser.add_argument("--chunk_size", type=int, default=None)
    parser.add_argument("--enable_workflow", default=False, action="store_true")
    parser.add_argument("--inplace", default=False, action="store_true")
    parser.add_argument("--module_times", default=False, action="store_true",
                        help="print the device time of every top-level module of the model (max over ranks)")


def parse_overrides(items):
    """``["a.b=3", "c.d=True"]`` -> ``{"a.b": 3, "c.d": True}``; values that are no Python literal stay strings."""
    import ast
    out = {}
    for item in items or ():
        key, sep, value = item.partition("=")
        if not sep or not key:
            raise ValueError("--config_override expects KEY=VALUE, got %r" % item)
        try:
            out[key.strip()] = ast.literal_eval(value)
        except (ValueError, SyntaxError):
            out[key.strip()] = value
    return out


def run_alignments(args, seqs, tags, multimer):
    """Runs the sequence searches and returns the alignment directory the data pipeline reads.  Monomer: one directory
    ``<output_dir>/alignments/<tag>``; multimer: one sub-directory per chain under ``<output_dir>/alignments``, each filled
    from a one-sequence FASTA file of that chain (fastfold inference.py:184-277).  ``--enable_workflow`` runs the searches of
    a chain concurrently through the workflow scheduler instead of the plain runner."""
    import shutil
    from fastfold_b200.data.data_pipeline import AlignmentRunner, AlignmentRunnerMultimer, temp_fasta_file
    from fastfold_b200.workflow.template import FastFoldDataWorkFlow, FastFoldMultimerDataWorkFlow
    common = dict(jackhmmer_binary_path=args.jackhmmer_binary_path, hhblits_binary_path=args.hhblits_binary_path,
                  uniref90_database_path=args.uniref90_database_path, mgnify_database_path=args.mgnify_database_path,
                  bfd_database_path=args.bfd_database_path, uniref30_database_path=args.uniclust30_database_path, no_cpus=args.cpus)
    base = os.path.join(args.output_dir, "alignments")
    t0 = time.perf_counter()
    if not multimer:
        cls = FastFoldDataWorkFlow if args.enable_workflow else AlignmentRunner
        runner = cls(hhsearch_binary_path=args.hhsearch_binary_path, pdb70_database_path=args.pdb70_database_path,
                     use_small_bfd=(args.preset == "reduced_dbs"), **common)
        out = os.path.join(base, tags[0].split()[0] if tags else "query")
        os.makedirs(out, exist_ok=True)
        runner.run(args.fasta_path, out)
    else:
        cls = FastFoldMultimerDataWorkFlow if args.enable_workflow else AlignmentRunnerMultimer
        runner = cls(hmmsearch_binary_path=args.hmmsearch_binary_path, hmmbuild_binary_path=args.hmmbuild_binary_path,
                     uniprot_database_path=args.uniprot_database_path, pdb_seqres_database_path=args.pdb_seqres_database_path,
                     use_small_bfd=(args.preset == "reduced_dbs" or args.bfd_database_path is None), **common)
        done = {}
        for tag, seq in zip(tags, seqs):
            chain_dir = os.path.join(base, tag.split()[0])
            if os.path.exists(chain_dir):
                shutil.rmtree(chain_dir)
            if seq in done:                              # copies of one chain share their searches
                shutil.copytree(done[seq], chain_dir)
                continue
            os.makedirs(chain_dir)
            with temp_fasta_file(">chain_%s\n%s\n" % (tag.split()[0], seq)) as chain_fasta:
                runner.run(chain_fasta, chain_dir)
            done[seq] = chain_dir
            print("Finished running alignment for %s" % tag.split()[0])
        out = base
    print("Alignment data workflow time: %.1f s" % (time.perf_counter() - t0))
    return out


def main(args):
    import numpy as np
    from fastfold_b200.common import protein
    from fastfold_b200.config import model_config
    from fastfold_b200.data.data_pipeline import DataPipeline, FeaturePipeline
    from fastfold_b200.data import parsers
    from fastfold_b200.runtime.inference import run_inference
    os.makedirs(args.output_dir, exist_ok=True)
    seqs, tags = parsers.parse_fasta(open(args.fasta_path).read())
    if args.model_preset == "multimer" and "multimer" not in args.model_name:
        args.model_name = "multimer"
    if args.model_preset == "monomer" and len(seqs) != 1:
        raise ValueError("monomer preset expects one sequence in the FASTA file; use --model_preset multimer")
    config = model_config(args.model_name)
    tag = tags[0].split()[0] if tags else "query"
    multimer = args.model_preset == "multimer"
    alignment_dir = None
    if args.use_precomputed_alignments:
        cand = os.path.join(args.use_precomputed_alignments, tag)
        alignment_dir = args.use_precomputed_alignments if multimer or not os.path.isdir(cand) else cand
    elif args.uniref90_database_path:
        alignment_dir = run_alignments(args, seqs, tags, multimer)
    featurizer = None
    if args.template_mmcif_dir and os.path.isdir(args.template_mmcif_dir) and config.model.template.enabled:
        # monomer: hhsearch hits against PDB70 (pdb70_hits.hhr); multimer: hmmsearch hits against the PDB sequences
        # (hmm_output.sto), which carry no alignment score and are used in search order (fastfold inference.py:175-182, 344-351)
        from fastfold_b200.data.templates import HmmsearchHitFeaturizer, TemplateHitFeaturizer
        featurizer = (HmmsearchHitFeaturizer if multimer else TemplateHitFeaturizer)(
            mmcif_dir=args.template_mmcif_dir, max_template_date=args.max_template_date, max_hits=4, kalign_binary_path=args.kalign_binary_path,
            release_dates_path=args.release_dates_path, obsolete_pdbs_path=args.obsolete_pdbs_path)
    if args.model_preset == "multimer":
        # every chain of the FASTA goes through the monomer pipeline (alignments under <alignment_dir>/<chain id>/), the
        # chains are paired by species and merged (fastfold inference.py:169-338)
        from fastfold_b200.data.data_pipeline import DataPipelineMultimer
        if args.use_precomputed_alignments:
            alignment_dir = args.use_precomputed_alignments
        raw = DataPipelineMultimer(DataPipeline(template_featurizer=featurizer)).process_fasta(args.fasta_path, alignment_dir)
        if int(np.asarray(raw["aatype"]).shape[0]) != sum(len(s_) for s_ in seqs):
            raise RuntimeError("multimer feature assembly lost residues: %d featurised, %d in the FASTA file"
                               % (int(np.asarray(raw["aatype"]).shape[0]), sum(len(s_) for s_ in seqs)))
    else:
        raw = DataPipeline(template_featurizer=featurizer).process_sequence(seqs[0], tag, alignment_dir)
    feats = FeaturePipeline(config.data).process_features(raw, mode="predict", seed=args.data_random_seed or 0,
                                                          is_multimer=args.model_preset == "multimer")
    overrides = {}
    if "template_aatype" not in feats:
        overrides["model.template.enabled"] = False
    overrides.update(parse_overrides(args.config_override))
    out = run_inference(feats, gpus=args.gpus, model_name=args.model_name, param_path=args.param_path, chunk_size=args.chunk_size,
                        inplace=args.inplace, overrides=overrides, module_times=args.module_times)
    print("Inference time: %.3f s (device-timed), peak memory %.2f GiB" % (out["_seconds"], out["_peak_gib"]))
    if "_module_times" in out:
        print(out.pop("_module_times"))
    plddt_b = np.repeat(out["plddt"][..., None], 37, axis=-1)
    f = {"aatype": feats["aatype"][..., 0].numpy(), "residue_index": feats["residue_index"][..., 0].numpy()}
    if "asym_id" in feats:
        f["asym_id"] = feats["asym_id"][..., 0].numpy()
    prot = protein.from_prediction(f, out, b_factors=plddt_b)
    path = os.path.join(args.output_dir, "%s_%s_unrelaxed.pdb" % (tag, args.model_name))
    with open(path, "w") as fh:
        fh.write(protein.to_pdb(prot))
    print("wrote", path)
    if args.relaxation:
        from fastfold_b200.relax import AmberRelaxation
        t0 = time.perf_counter()
        relaxed, _, _ = AmberRelaxation(use_gpu=True, **config.relax).process(prot=prot)
        print("Relaxation time: %.1f s" % (time.perf_counter() - t0))
        with open(os.path.join(args.output_dir, "%s_%s_relaxed.pdb" % (tag, args.model_name)), "w") as fh:
            fh.write(relaxed)
    if args.save_prediction_result:
        with open(os.path.join(args.output_dir, "%s_%s_output_dict.pkl" % (tag, args.model_name)), "wb") as fh:
            pickle.dump(out, fh, protocol=pickle.HIGHEST_PROTOCOL)


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("fasta_path", type=str)
    p.add_argument("template_mmcif_dir", type=str, nargs="?", default=None)
    p.add_argument("--use_precomputed_alignments", type=str, default=None)
    p.add_argument("--output_dir", type=str, default=os.getcwd())
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--model_name", type=str, default="model_1")
    p.add_argument("--param_path", type=str, default=None)
    p.add_argument("--model_preset", type=str, default="monomer", choices=["monomer", "multimer"])
    p.add_argument("--preset", type=str, default="full_dbs", choices=("reduced_dbs", "full_dbs"))
    p.add_argument("--cpus", type=int, default=12)
    p.add_argument("--relaxation", action="store_true", default=False)
    p.add_argument("--save_prediction_result", action="store_true", default=False)
    p.add_argument("--data_random_seed", type=int, default=None)
    p.add_argument("--config_override", action="append", default=[], metavar="KEY=VALUE",
                   help="set one entry of the model config, e.g. model.evoformer_stack.no_blocks=8 (repeatable; the value is "
                        "read as a Python literal).  For reduced models; published parameter archives need the stock config")
    add_data_args(p)
    a = p.parse_args()
    if a.param_path is None:
        a.param_path = os.path.join("data", "params", "params_" + a.model_name + ".npz")
    main(a)
