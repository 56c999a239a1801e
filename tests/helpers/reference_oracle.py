"""Runs the installed reference package (``baseline/_ref``, with the import stand-ins of ``baseline/stubs``) on CPU as an
oracle.  Started as a script in its own process - the reference is a package called ``fastfold`` and must not share an
interpreter with this repository's ``fastfold`` compatibility namespace:

    python reference_oracle.py <mode> <input.pt> <output.pt>

``mode``: ``tools`` (runs every alignment-tool wrapper against recording stand-in executables), ``geometry`` (the struct-of-arrays vectors, rotations and rigids of the multimer model), ``all_atom_multimer`` (torsions to frames to atoms, ground-truth frames, chi angles on the struct-of-arrays types), ``rigid`` (rigid-transform algebra and two feature helpers), ``violations`` (the structural-violation terms and their gradients, bounds supplied by the caller), ``fast_model`` (full forward through the reference's own ``inject_fastnn`` and fast modules - the path its
inference runs - with its two GPU-only kernel entry points, fused LayerNorm and fused softmax, replaced by their PyTorch
definitions so that the path runs on CPU; DAP size 1), ``data_modules`` (training-set filters, ``OpenFoldSingleDataset`` items, the batch collator), ``multimer_pipeline`` (``DataPipelineMultimer.process_fasta`` on per-chain alignment directories), ``pipeline`` (``DataPipeline.process_fasta`` / ``process_mmcif`` on an alignment directory), ``mmcif`` (its mmCIF reader - on the BioPython stand-in of ``baseline/stubs`` - and its template featuriser on
the files of a directory), ``utils`` (PDB writer, dRMSD / GDT, learning-rate schedule), ``parsers`` (FASTA / A3M / Stockholm / HHR / hmmsearch / tblout parsers on the given texts), ``config`` (every preset of ``model_config`` flattened to ``{dotted key: repr(value)}``), ``multimer_merge`` (``feature_processing_multimer.pair_and_merge`` on per-chain feature dicts),
``multimer_tensors`` (the multimer tensor pipeline stage by stage: un-ensembled transforms, seeded row sampling, BERT-style
corruption, clustering and ``msa_feat``), ``import_weights`` (its ``import_jax_weights_`` applied to a parameter archive; returns the state dict),
``features`` (the tensor pipeline on a raw feature dict: the un-ensembled transforms, then one ensemble member
with the given seed and MSA resampling switched off), ``model`` (full ``AlphaFold`` forward in the OpenFold layout), ``loss`` (``AlphaFoldLoss`` with the per-term
breakdown), ``multimer_parts`` (input embedder, structure module and template embedder of the multimer model, called
one by one: the reference's OpenFold-layout trunk does not implement the multimer block ordering, so whole multimer
models cannot be compared).  The input file holds the state dict (OpenFold names), the features and the config edits.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _setup():
    for name, typ in (("int", int), ("float", float), ("bool", bool), ("object", object), ("string_", np.bytes_)):
        if not hasattr(np, name):                 # aliases numpy 2 dropped and the reference's tables still use
            setattr(np, name, typ)
    sys.path.insert(0, os.path.join(ROOT, "baseline", "stubs"))
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import fastfold
    assert os.path.abspath(fastfold.__file__).startswith(os.path.join(ROOT, "baseline", "_ref")), fastfold.__file__


def _config(d):
    from fastfold.config import model_config
    c = model_config(d["name"], train=d.get("train", False))
    for key, value in d["edits"].items():
        node = c
        parts = key.split(".")
        for p in parts[:-1]:
            node = node[p]
        node[parts[-1]] = value
    c.globals.is_multimer = "multimer" in d["name"]
    c.globals.inplace = bool(d.get("inplace", False))
    c.globals.chunk_size = d.get("chunk_size")
    return c


def _detach(tree):
    if torch.is_tensor(tree):
        return tree.detach()
    if isinstance(tree, dict):
        return {k: _detach(v) for k, v in tree.items()}
    return tree


def _tensors(tree):
    if torch.is_tensor(tree):
        return tree
    if hasattr(tree, "to_tensor_4x4"):
        return tree.to_tensor_4x4()
    if isinstance(tree, dict):
        return {k: _tensors(v) for k, v in tree.items() if torch.is_tensor(v) or isinstance(v, dict) or hasattr(v, "to_tensor_4x4")}
    return tree


def all_atom_multimer_case(aam, g, d):
    """The struct-of-arrays all-atom helpers of the multimer model on one chain; ``aam`` / ``g`` are the
    ``all_atom_multimer`` and ``geometry`` modules of the implementation under test, so both sides run this very code."""
    aatype, torsions = d["aatype"], d["torsions"]
    pos37, mask37 = g.Vec3Array.from_array(d["pos37"]), d["mask37"]
    out, failed = {}, []

    def attempt(name, fn):
        try:
            out.update(fn())
        except Exception as e:                      # a helper the implementation cannot run is reported, not fatal
            failed.append("%s: %s" % (name, type(e).__name__))

    def frames():
        f = aam.torsion_angles_to_frames(aatype, g.Rigid3Array.from_tensor_4x4(d["backbone"]), torsions)
        return {"frames8": f.to_tensor_4x4()}

    def atoms():
        p = aam.frames_and_literature_positions_to_atom14_pos(aatype, g.Rigid3Array.from_tensor_4x4(d["frames8"]))
        return {"pos14": p.to_tensor(), "atom37_from_14": aam.atom14_to_atom37(p.to_tensor(), aatype)}

    def gt_frames():
        gt = aam.atom37_to_frames(aatype, pos37, mask37)
        return {"gt_frames": gt["rigidgroups_gt_frames"].to_tensor_4x4(), "alt_gt_frames": gt["rigidgroups_alt_gt_frames"].to_tensor_4x4(),
                "gt_exists": gt["rigidgroups_gt_exists"].float(), "group_exists": gt["rigidgroups_group_exists"].float(),
                "is_ambiguous": gt["rigidgroups_group_is_ambiguous"].float()}

    def chi():
        angles, mask = aam.compute_chi_angles(pos37, mask37, aatype)
        return {"chi": angles, "chi_mask": mask.float()}

    def backbone():
        rigid, mask = aam.make_backbone_affine(pos37, mask37, aatype)
        return {"backbone": rigid.to_tensor_4x4(), "backbone_mask": mask.float()}

    def to14():
        p, m = aam.atom37_to_atom14(aatype, pos37, mask37)
        return {"atom14_from_37": p.to_tensor() if hasattr(p, "to_tensor") else p, "atom14_mask": m.float()}

    def chi_indices():
        return {"chi_atom_indices": torch.as_tensor(aam.get_chi_atom_indices(torch.device("cpu"))).long()}

    for name, fn in (("torsion_angles_to_frames", frames), ("frames_and_literature_positions_to_atom14_pos", atoms), ("atom37_to_frames", gt_frames),
                     ("compute_chi_angles", chi), ("make_backbone_affine", backbone), ("atom37_to_atom14", to14), ("get_chi_atom_indices", chi_indices)):
        attempt(name, fn)
    out["failed"] = failed
    return out


def main(mode, src, dst):
    _setup()
    d = torch.load(src, weights_only=False)
    if mode == "tools":
        from fastfold.data.tools import hhblits, hhsearch, hmmbuild, hmmsearch, jackhmmer, kalign
        b = d["bin"]
        jackhmmer.Jackhmmer(binary_path=b["jackhmmer"], database_path=d["db"]).query(d["fasta"])
        jackhmmer.Jackhmmer(binary_path=b["jackhmmer"], database_path=d["db"], n_cpu=3, n_iter=2, e_value=0.01, z_value=1000, get_tblout=True,
                            dom_e=0.1, incdom_e=0.2).query(d["fasta"])
        hhblits.HHBlits(binary_path=b["hhblits"], databases=[d["hhdb"]]).query(d["fasta"])
        hhblits.HHBlits(binary_path=b["hhblits"], databases=[d["hhdb"], d["hhdb"]], n_cpu=2, n_iter=1, all_seqs=True, alt=3, p=30, z=100).query(d["fasta"])
        hhsearch.HHSearch(binary_path=b["hhsearch"], databases=[d["hhdb"]]).query(d["a3m"])
        hmmbuild.Hmmbuild(binary_path=b["hmmbuild"]).build_profile_from_sto(d["sto"], model_construction="hand")
        hmmbuild.Hmmbuild(binary_path=b["hmmbuild"], singlemx=True).build_profile_from_a3m(d["a3m"])
        hmmsearch.Hmmsearch(binary_path=b["hmmsearch"], hmmbuild_binary_path=b["hmmbuild"], database_path=d["db"]).query(d["sto"])
        kalign.Kalign(binary_path=b["kalign"]).align(d["seqs"])
        from fastfold.data import data_pipeline
        os.environ["RECORD"] = d["record_runner"]
        for tag, small in (("full", False), ("small", True)):
            out_dir = os.path.join(d["out"], "mono_" + tag)
            os.makedirs(out_dir)
            data_pipeline.AlignmentRunner(jackhmmer_binary_path=b["jackhmmer"], hhblits_binary_path=b["hhblits"], hhsearch_binary_path=b["hhsearch"],
                                          uniref90_database_path=d["db"], mgnify_database_path=d["db"], bfd_database_path=d["db"] if small else d["hhdb"],
                                          uniref30_database_path=None if small else d["hhdb"], pdb70_database_path=d["hhdb"], use_small_bfd=small,
                                          no_cpus=4).run(d["fasta"], out_dir)
        out_dir = os.path.join(d["out"], "multi")
        os.makedirs(out_dir)
        data_pipeline.AlignmentRunnerMultimer(jackhmmer_binary_path=b["jackhmmer"], hhblits_binary_path=b["hhblits"], hmmsearch_binary_path=b["hmmsearch"],
                                              hmmbuild_binary_path=b["hmmbuild"], uniref90_database_path=d["db"], mgnify_database_path=d["db"],
                                              bfd_database_path=d["hhdb"], uniref30_database_path=d["hhdb"], uniprot_database_path=d["db"],
                                              pdb_seqres_database_path=d["db"], use_small_bfd=False, no_cpus=8).run(d["fasta"], out_dir)
        torch.save({}, dst)
        return
    if mode == "geometry":
        from fastfold.utils import geometry as g
        from fastfold.utils.geometry import vector as gv
        from fastfold.utils.geometry.quat_rigid import QuatRigid
        a, b, c, e = (g.Vec3Array.from_array(x) for x in (d["a"], d["b"], d["c"], d["e"]))
        rot = g.Rot3Array.from_two_vectors(a, b)
        rotq = g.Rot3Array.from_quaternion(*torch.unbind(d["q"], dim=-1))
        rig, rig2 = g.Rigid3Array(rot, c), g.Rigid3Array(rotq, e)
        lin = QuatRigid(d["act"].shape[-1], full_quat=False)
        lin.load_state_dict(d["quat_state"])
        with torch.no_grad():
            from_act = lin(d["act"])
        out = {"add": (a + b).to_tensor(), "sub": (a - b).to_tensor(), "scale": (a * 2.5).to_tensor(), "div": (a / 2.0).to_tensor(), "neg": (-a).to_tensor(),
               "dot": a.dot(b), "cross": a.cross(b).to_tensor(), "norm": a.norm(), "norm2": a.norm2(), "normalized": a.normalized().to_tensor(),
               "dihedral": gv.dihedral_angle(a, b, c, e),       # its two distance helpers fail on a float epsilon and are left out
               "rot": rot.to_tensor(), "rotq": rotq.to_tensor(), "rot_apply": rot.apply_to_point(c).to_tensor(),
               "rot_inv_apply": rot.apply_inverse_to_point(c).to_tensor(), "rot_inverse": rot.inverse().to_tensor(), "rot_matmul": (rot @ rotq).to_tensor(),
               "rigid_4x4": rig.to_tensor_4x4(), "rigid_compose": (rig @ rig2).to_tensor_4x4(), "rigid_inverse": rig.inverse().to_tensor_4x4(),
               "rigid_apply": rig.apply_to_point(e).to_tensor(), "rigid_inv_apply": rig.apply_inverse_to_point(e).to_tensor(),
               "rigid_from_4x4": g.Rigid3Array.from_tensor_4x4(rig.to_tensor_4x4()).to_tensor_4x4(),
               "rigid_scale": rig.scale_translation(0.1).to_tensor_4x4(), "identity": g.Rigid3Array.identity((3,), "cpu").to_tensor_4x4(),
               "quat_rigid": from_act.to_tensor_4x4()}
        torch.save(out, dst)
        return
    if mode == "all_atom_multimer":
        from fastfold.utils import all_atom_multimer, geometry
        torch.save(all_atom_multimer_case(all_atom_multimer, geometry, d), dst)
        return
    if mode == "rigid":
        from fastfold.utils import rigid_utils as ru
        from fastfold.utils import feats
        q, t, pts, upd = d["quats"], d["trans"], d["points"], d["update"]
        r = ru.Rigid(ru.Rotation(quats=q, normalize_quats=True), t)
        r2 = ru.Rigid.from_3_points(pts[..., 0, :], pts[..., 1, :], pts[..., 2, :], eps=1e-8)
        out = {"t7": r.to_tensor_7(), "t4x4": r.to_tensor_4x4(), "rot_mats": r.get_rots().get_rot_mats(), "apply": r[..., None].apply(pts),
               "invert_apply": r[..., None].invert_apply(pts), "compose": r.compose(r2).to_tensor_4x4(), "invert": r.invert().to_tensor_4x4(),
               "update": r.compose_q_update_vec(upd).to_tensor_7(), "from_3_points": r2.to_tensor_4x4(),
               "from_4x4": ru.Rigid.from_tensor_4x4(r2.to_tensor_4x4()).to_tensor_4x4(), "from_7": ru.Rigid.from_tensor_7(r.to_tensor_7()).to_tensor_4x4(),
               "quat_multiply": ru.quat_multiply(q, d["quats2"]), "quat_to_rot": ru.quat_to_rot(torch.nn.functional.normalize(q, dim=-1)),
               "rot_to_quat": ru.rot_to_quat(r.get_rots().get_rot_mats()), "scale_translation": r.scale_translation(3.0).to_tensor_7(),
               "stop_rot_gradient": r.stop_rot_gradient().to_tensor_7(), "cat": ru.Rigid.cat([r, r2], dim=0).to_tensor_4x4(),
               "atom14_to_atom37": feats.atom14_to_atom37(d["atom14"], d["maps"]), "pseudo_beta": feats.pseudo_beta_fn(d["aatype"], d["atom37"], None)}
        torch.save(out, dst)
        return
    if mode == "violations":
        from fastfold.model.hub import loss as L
        pos = d["pos"].clone().requires_grad_(True)
        out = {"bond": L.between_residue_bond_loss(pos, d["exists"], d["residue_index"], d["aatype"], tolerance_factor_soft=12.0, tolerance_factor_hard=12.0),
               "clash": L.between_residue_clash_loss(pos, d["exists"], d["radius"], d["residue_index"], overlap_tolerance_soft=1.5, overlap_tolerance_hard=1.5),
               "within": L.within_residue_violations(pos, d["exists"], d["lower"], d["upper"], tighten_bounds_for_loss=0.0),
               "ca_ca": L.extreme_ca_ca_distance_violations(pos, d["exists"], d["residue_index"])}
        total = out["bond"]["c_n_loss_mean"] + out["bond"]["ca_c_n_loss_mean"] + out["bond"]["c_n_ca_loss_mean"] + \
            out["clash"]["mean_loss"] + out["within"]["per_atom_loss_sum"].sum()
        total.backward()
        out["grad"] = pos.grad
        out["violation_loss"] = L.violation_loss(d["violations"], d["exists"])
        out["metrics"] = L.compute_violation_metrics({"atom14_atom_exists": d["exists"], "residue_index": d["residue_index"], "seq_mask": d["seq_mask"]},
                                                     d["pos"], d["violations"])
        torch.save(_detach(out), dst)
        return
    if mode == "data_modules":
        from fastfold.data import data_modules as dm
        config = _config(d)
        out = {"filters": [(dm.deterministic_train_filter(e), dm.get_stochastic_train_filter_prob(e)) for e in d["cache_entries"]]}
        ds = dm.OpenFoldSingleDataset(data_dir=d["data_dir"], alignment_dir=d["alignment_dir"], template_mmcif_dir=d["mmcif_dir"],
                                      max_template_date="2100-01-01", config=config.data, kalign_binary_path=None, mode="train", _output_raw=True)
        out["chain_ids"] = [ds.idx_to_chain_id(i) for i in range(len(ds))]
        out["raw"] = {ds.idx_to_chain_id(i): dict(ds[i]) for i in range(len(ds))}
        feats = dm.OpenFoldSingleDataset(data_dir=d["data_dir"], alignment_dir=d["alignment_dir"], template_mmcif_dir=d["mmcif_dir"],
                                         max_template_date="2100-01-01", config=config.data, kalign_binary_path=None, mode="eval")
        out["eval_shapes"] = {k: tuple(v.shape) for k, v in feats[0].items()}
        collated = dm.OpenFoldBatchCollator(config.data, "eval")([ds[0]])           # raw examples in, features out, no batch dim for one
        out["collated_shapes"] = {k: tuple(v.shape) for k, v in collated.items()}
        torch.save(out, dst)
        return
    if mode == "multimer_pipeline":
        from fastfold.data import data_pipeline
        from fastfold.data import templates
        featurizer = templates.TemplateHitFeaturizer(mmcif_dir=d["mmcif_dir"], max_template_date="2100-01-01", max_hits=4, kalign_binary_path=None)
        pipe = data_pipeline.DataPipelineMultimer(data_pipeline.DataPipeline(template_featurizer=featurizer))
        torch.save({"example": dict(pipe.process_fasta(d["fasta"], d["alignment_dir"]))}, dst)
        return
    if mode == "pipeline":
        from fastfold.data import data_pipeline, mmcif_parsing, templates
        featurizer = templates.TemplateHitFeaturizer(mmcif_dir=d["mmcif_dir"], max_template_date=d["max_template_date"], max_hits=4, kalign_binary_path=None)
        pipe = data_pipeline.DataPipeline(template_featurizer=featurizer)
        out = {"fasta": dict(pipe.process_fasta(d["fasta"], d["alignment_dir"]))}
        text = open(os.path.join(d["mmcif_dir"], d["target"][0] + ".cif")).read()
        obj = mmcif_parsing.parse(file_id=d["target"][0], mmcif_string=text).mmcif_object
        out["mmcif"] = dict(pipe.process_mmcif(obj, d["target_alignment_dir"], d["target"][1]))
        torch.save(out, dst)
        return
    if mode == "mmcif":
        import dataclasses
        import datetime
        from fastfold.data import mmcif_parsing, parsers, templates

        def plain(x):
            if dataclasses.is_dataclass(x):
                return {f.name: plain(getattr(x, f.name)) for f in dataclasses.fields(x)}
            if isinstance(x, dict):
                return {k: plain(v) for k, v in x.items()}
            if isinstance(x, (list, tuple)):
                return [plain(v) for v in x]
            return x
        out = {"files": {}}
        for file_id, chain in d["parse"]:
            text = open(os.path.join(d["mmcif_dir"], file_id + ".cif")).read()
            res = mmcif_parsing.parse(file_id=file_id, mmcif_string=text)
            obj = res.mmcif_object
            entry = {"errors": {str(k): repr(v) for k, v in res.errors.items()}}
            if obj is not None:
                pos, mask = mmcif_parsing.get_atom_coords(obj, chain)
                raw, rawmask = mmcif_parsing.get_atom_coords(obj, chain, _zero_center_positions=False)
                entry.update(chain_to_seqres=dict(obj.chain_to_seqres), header=dict(obj.header), seqres_to_structure=plain(obj.seqres_to_structure),
                             pos=pos, mask=mask, raw_pos=raw)
            out["files"][file_id + "/" + chain] = entry
        hits = [parsers.TemplateHit(**h) for h in d["hits"]]
        featurizer = templates.TemplateHitFeaturizer(mmcif_dir=d["mmcif_dir"], max_template_date=d["max_template_date"], max_hits=d["max_hits"],
                                                     kalign_binary_path=d.get("kalign"), obsolete_pdbs_path=d.get("obsolete"))
        runs = {}
        for name, kw in d["queries"].items():
            date = kw.get("query_release_date")
            date = datetime.datetime.strptime(date, "%Y-%m-%d") if date else None
            r = featurizer.get_templates(query_sequence=d["query"], query_release_date=date, hits=hits, query_pdb_code=kw.get("query_pdb_code"))
            runs[name] = {"features": dict(r.features), "errors": list(r.errors), "warnings": list(r.warnings)}
        out["templates"] = runs
        torch.save(out, dst)
        return
    if mode == "utils":
        from fastfold.common import protein
        from fastfold.model.hub.lr_scheduler import AlphaFoldLRScheduler
        from fastfold.utils import validation_utils as vu
        prot = protein.from_prediction(d["features"], d["result"], b_factors=d["b_factors"])
        out = {"pdb": protein.to_pdb(prot), "ideal_atom_mask": protein.ideal_atom_mask(prot)}
        a, b, mask = d["structures"]
        out["drmsd"] = vu.drmsd(a[0], b[0], mask[0])              # the reference's version takes one structure at a time
        out["drmsd_nomask"] = vu.drmsd(a[0], b[0])
        out["gdt_ts"], out["gdt_ha"] = vu.gdt_ts(a, b, mask), vu.gdt_ha(a, b, mask)
        from fastfold.utils.superimposition import superimpose
        out["superimposed"], out["rmsd"] = superimpose(a, b, mask)
        out["validation_metrics"] = vu.compute_validation_metrics(d["val_batch"], d["val_outputs"], superimposition_metrics=True)
        opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1)
        # its constructor passes ``verbose`` to a base class that no longer takes it: evaluate the schedule itself
        sched = AlphaFoldLRScheduler.__new__(AlphaFoldLRScheduler)
        sched.__dict__.update(d["schedule"], optimizer=opt, _get_lr_called_within_step=True)
        lrs = []
        for step in range(1, d["steps"] + 1):
            sched.last_epoch = step
            lrs.append(sched.get_lr()[0])
        out["lrs"] = lrs
        torch.save(out, dst)
        return
    if mode == "parsers":
        import dataclasses
        from fastfold.data import parsers

        def plain(x):
            if dataclasses.is_dataclass(x):
                return {f.name: plain(getattr(x, f.name)) for f in dataclasses.fields(x)}
            if isinstance(x, (list, tuple)):
                return [plain(v) for v in x]
            if isinstance(x, dict):
                return {k: plain(v) for k, v in x.items()}
            if hasattr(x, "sequences") and hasattr(x, "deletion_matrix"):
                return {"sequences": list(x.sequences), "deletion_matrix": plain(x.deletion_matrix), "descriptions": list(x.descriptions)}
            return x
        t = d["texts"]
        out = {"fasta": plain(parsers.parse_fasta(t["fasta"])), "a3m": plain(parsers.parse_a3m(t["a3m"])),
               "sto": plain(parsers.parse_stockholm(t["sto"])), "sto_to_a3m": parsers.convert_stockholm_to_a3m(t["sto"]),
               "sto_to_a3m_keep": parsers.convert_stockholm_to_a3m(t["sto"], remove_first_row_gaps=False),
               "sto_to_a3m_max2": parsers.convert_stockholm_to_a3m(t["sto"], max_sequences=2),
               "sto_dedup": parsers.deduplicate_stockholm_msa(t["sto"]),
               "sto_no_empty": parsers.remove_empty_columns_from_stockholm_msa(t["sto_gappy"]),
               "hhr": plain(parsers.parse_hhr(t["hhr"])), "tblout": plain(parsers.parse_e_values_from_tblout(t["tblout"])),
               "hmmsearch": plain(parsers.parse_hmmsearch_sto(t["hmmsearch_sto"], t["query"]))}
        from fastfold.data import msa_identifiers
        out["species"] = [msa_identifiers.get_identifiers(x).species_id for x in d.get("descriptions", [])]
        torch.save(out, dst)
        return
    if mode == "config":
        from fastfold.config import model_config

        def flat(c, pre=""):
            out = {}
            for k, v in c.items():
                if hasattr(v, "items"):
                    out.update(flat(v, pre + k + "."))
                else:
                    out[pre + k] = repr(v)
            return out
        torch.save({"%s|%s" % (n, t): flat(model_config(n, train=t)) for n in d["names"] for t in (False, True)}, dst)
        return
    if mode == "multimer_merge":
        from fastfold.data import feature_processing_multimer
        torch.save({"example": dict(feature_processing_multimer.pair_and_merge(d["chains"]))}, dst)
        return
    if mode == "multimer_tensors":
        from fastfold.data import data_transforms_multimer as dtm, input_pipeline_multimer as ipm
        config = _config(d)
        common, mode_cfg = config.data.common, config.data[d["mode"]]
        t = {k: torch.as_tensor(np.asarray(v)) for k, v in d["example"].items() if np.asarray(v).dtype != object}
        with torch.no_grad():
            t = ipm.compose(ipm.nonensembled_transform_fns(common, mode_cfg))(t)
            non = {k: v.clone() for k, v in t.items()}
            t = dtm.sample_msa(d["max_seq"], d["max_extra"], seed=d["seed"])(dict(t))
            sampled = {k: v.clone() for k, v in t.items()}
            torch.manual_seed(d["torch_seed"])
            t = dtm.make_masked_msa(common.masked_msa, mode_cfg.masked_msa_replace_fraction, seed=d["seed"] + 1)(t)
            masked = {k: v.clone() for k, v in t.items()}
            t = dtm.create_msa_feat(dtm.nearest_neighbor_clusters()(t))
        torch.save({"non": non, "sampled": sampled, "masked": masked, "final": dict(t)}, dst)
        return
    if mode == "features":
        from fastfold.data import feature_pipeline, input_pipeline
        config = _config(d)
        raw = dict(d["raw"])
        cfg, names = feature_pipeline.make_data_config(config.data, mode=d["mode"], num_res=int(raw["seq_length"][0]))
        if "deletion_matrix_int" in raw:
            raw["deletion_matrix"] = raw.pop("deletion_matrix_int").astype(np.float32)
        t = feature_pipeline.np_to_tensor_dict(np_example=raw, features=names)
        torch.manual_seed(d["torch_seed"])
        with torch.no_grad():
            t = input_pipeline.compose(input_pipeline.nonensembled_transform_fns(cfg.common, cfg[d["mode"]]))(t)
            non = {k: v.clone() for k, v in t.items()}
            ens = input_pipeline.compose(input_pipeline.ensembled_transform_fns(cfg.common, cfg[d["mode"]], d["seed"]))(dict(t))
        torch.save({"non": non, "ens": ens}, dst)
        return
    if mode == "loss":
        from fastfold.model.hub.loss import AlphaFoldLoss
        loss, parts = AlphaFoldLoss(_config(d).loss)(d["out"], d["batch"], _return_breakdown=True)
        torch.save({"loss": float(loss), "parts": {k: float(v) for k, v in parts.items()}}, dst)
        return
    from fastfold.model.hub import AlphaFold
    if mode == "fast_model":
        import importlib
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(d.get("port", 29533)))

        def softmax(x, mask=None, bias=None):          # fastfold/model/fastnn/kernel/softmax.py: softmax(x + 1e9 (mask - 1) + bias)
            if mask is not None:
                while mask.dim() < x.dim():
                    mask = mask.unsqueeze(-2)
                x = x + 1e9 * (mask - 1)
            return torch.softmax(x if bias is None else x + bias, dim=-1)

        class LayerNorm(torch.nn.LayerNorm):
            def __init__(self, normalized_shape, eps=1e-5):
                super().__init__(normalized_shape, eps=eps)
        for name in ("ops", "msa", "triangle", "evoformer", "template", "embedders", "embedders_multimer", "kernel"):
            module = importlib.import_module("fastfold.model.fastnn." + name)
            if hasattr(module, "LayerNorm"):
                module.LayerNorm = LayerNorm
            if hasattr(module, "fused_softmax"):
                module.fused_softmax = softmax
        from fastfold.distributed import init_dap
        from fastfold.utils.inject_fastnn import inject_fastnn
        init_dap(1)
        if "stack" in d:                  # forward and backward of a bare fast Evoformer stack (as benchmark/perf.py builds it)
            from fastfold.model.fastnn import EvoformerStack
            k = d["stack"]
            stack = EvoformerStack(c_m=k["c_m"], c_z=k["c_z"], c_s=k["c_s"], no_blocks=k["no_blocks"], blocks_per_ckpt=None,
                                   is_multimer=k["is_multimer"]).eval()
            stack.load_state_dict(d["state"], strict=True)
            m, z = d["m"].clone().requires_grad_(True), d["z"].clone().requires_grad_(True)
            om, oz, s = stack(m, z, d["msa_mask"], d["pair_mask"], chunk_size=None)
            (om.pow(2).mean() + oz.pow(2).mean() + s.pow(2).mean()).backward()
            torch.save({"m": om.detach(), "z": oz.detach(), "s": s.detach(), "dm": m.grad, "dz": z.grad,
                        "grads": {n: p.grad for n, p in stack.named_parameters()}}, dst)
            return
        model = AlphaFold(_config(d)).eval()
        model.load_state_dict(d["state"], strict=True)
        model = inject_fastnn(model)
        from fastfold.model.fastnn import set_chunk_size
        set_chunk_size(d.get("chunk_size"))
        if d.get("loss"):                 # gradients of the training loss (eval mode: no dropout) with respect to every parameter
            from fastfold.model.hub.loss import AlphaFoldLoss
            out = model(d["batch"])
            out["violation"] = d["violation"]          # computed by the caller: the reference would download its bond-length table
            last = {k: v[..., -1] for k, v in d["batch"].items()}
            loss, parts = AlphaFoldLoss(_config(d).loss)(out, last, _return_breakdown=True)
            loss.backward()
            torch.save({"loss": float(loss), "parts": {k: float(v) for k, v in parts.items()},
                        "grads": {n: p.grad for n, p in model.named_parameters()}}, dst)
            return
        with torch.no_grad():
            torch.save({"out": _tensors(model(d["batch"])), "fast_state": model.state_dict()}, dst)
        return
    model = AlphaFold(_config(d)).eval()
    if mode == "import_weights":
        from fastfold.utils.import_weights import import_jax_weights_
        import_jax_weights_(model, d["npz"], version=d["name"])
        torch.save({"state": model.state_dict()}, dst)
        return
    own = model.state_dict()
    res = {"missing": [k for k in own if k not in d["state"]], "unexpected": [k for k in d["state"] if k not in own]}
    model.load_state_dict(d["state"], strict=False)
    with torch.no_grad():
        if mode == "model":
            res["out"] = _tensors(model(d["batch"]))
        elif mode == "multimer_parts":
            f = d["f"]
            res["sm"] = _tensors(model.structure_module(d["s"], d["z"], f["aatype"], mask=f["seq_mask"]))
            m, z = model.input_embedder(f)
            res["m"], res["z"] = m, z
            pair_mask = f["seq_mask"][..., None] * f["seq_mask"][..., None, :]
            asym = f["asym_id"]
            templ = {k: v for k, v in f.items() if k.startswith("template_")}
            res["te"] = _tensors(model.template_embedder(templ, z, pair_mask.to(z.dtype), 0, chunk_size=None,
                                                         multichain_mask_2d=asym[..., None] == asym[..., None, :]))
        else:
            raise SystemExit("unknown mode %r" % mode)
    torch.save(res, dst)


if __name__ == "__main__":
    main(*sys.argv[1:4])
