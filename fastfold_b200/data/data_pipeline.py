"""From a FASTA file (+ a directory of alignments) to the raw numpy feature dict, and on to model tensors.

``DataPipeline.process_fasta(fasta_path, alignment_dir)`` reads whatever alignments exist in ``alignment_dir``
(``*.a3m`` / ``*.sto`` as written by jackhmmer / hhblits; none -> single-sequence mode) and produces sequence + MSA
features; ``FeaturePipeline.process_features(raw, mode)`` applies the tensor transforms (MSA sampling, clustering,
masking, ``msa_feat``) once per recycling iteration and stacks the iterations on the LAST axis.  Alignment tools
are run by ``AlignmentRunner`` (subprocess wrappers in ``data/tools.py``) when their binaries exist.  Templates from
HHR hits need mmCIF files and are produced by ``data/templates.py`` when available; otherwise template features
are empty.  Same roles as fastfold/data/data_pipeline.py, feature_pipeline.py and input_pipeline.py.
"""
import copy
import os
from typing import Mapping, Optional, Sequence

import numpy as np
import torch

from ..common import residue_constants as rc
from . import data_transforms as dt
from . import parsers

FeatureDict = Mapping[str, np.ndarray]


def make_sequence_features(sequence: str, description: str, num_res: int) -> FeatureDict:
    return {
        "aatype": rc.sequence_to_onehot(sequence, rc.restype_order_with_x, map_unknown_to_x=True),
        "between_segment_residues": np.zeros((num_res,), dtype=np.int32),
        "domain_name": np.array([description.encode("utf-8")], dtype=object),
        "residue_index": np.array(range(num_res), dtype=np.int32),
        "seq_length": np.array([num_res] * num_res, dtype=np.int32),
        "sequence": np.array([sequence.encode("utf-8")], dtype=object),
    }


def make_msa_features(msas, deletion_matrices: Optional[Sequence[parsers.DeletionMatrix]] = None, descriptions=None) -> FeatureDict:
    """Rows of several alignments stacked in order, each distinct row once (first occurrence), as HH-suite residue ids, with
    their deletion counts and the species tag of their description (empty when the description has none; used to pair rows
    across chains).  ``msas``: ``parsers.Msa`` objects (fastfold/data/data_pipeline.py:205-240), or lists of rows together with
    ``deletion_matrices`` (and optionally ``descriptions``)."""
    if not msas:
        raise ValueError("At least one MSA must be provided.")
    if deletion_matrices is not None:
        descriptions = descriptions if descriptions is not None else [[""] * len(m) for m in msas]
        msas = [parsers.Msa(list(m), list(d), list(t)) for m, d, t in zip(msas, deletion_matrices, descriptions)]
    from .msa_pairing import get_identifiers
    int_msa, deletion_matrix, species, seen = [], [], [], set()
    for index, msa in enumerate(msas):
        if not len(msa):
            raise ValueError("MSA %d must contain at least one sequence." % index)
        for seq, dels, desc in zip(msa.sequences, msa.deletion_matrix, msa.descriptions):
            if seq in seen:
                continue
            seen.add(seq)
            int_msa.append([rc.HHBLITS_AA_TO_ID[r] for r in seq])
            deletion_matrix.append(dels)
            species.append(get_identifiers(desc).species_id.encode("utf-8"))
    num_res = len(msas[0].sequences[0])
    return {"deletion_matrix_int": np.array(deletion_matrix, dtype=np.int32), "msa": np.array(int_msa, dtype=np.int32),
            "num_alignments": np.array([len(int_msa)] * num_res, dtype=np.int32), "msa_species_identifiers": np.array(species, dtype=np.object_)}


def empty_template_features(num_res: int) -> FeatureDict:
    return {"template_aatype": np.zeros((0, num_res, 22), np.float32), "template_all_atom_mask": np.zeros((0, num_res, 37), np.float32),
            "template_all_atom_positions": np.zeros((0, num_res, 37, 3), np.float32), "template_domain_names": np.zeros((0,), object),
            "template_sequence": np.zeros((0,), object), "template_sum_probs": np.zeros((0, 1), np.float32)}


empty_template_feats = empty_template_features          # the reference's name for the same function


def make_template_features(input_sequence: str, hits, template_featurizer, query_pdb_code=None, query_release_date=None) -> FeatureDict:
    """Template features of one query from parsed search hits (``{file name: [hits]}`` or a flat list); the empty
    feature set when there is no featuriser, no hit, or no hit survives the featuriser's filters."""
    flat = sum(hits.values(), []) if isinstance(hits, Mapping) else list(hits or [])
    if not flat or template_featurizer is None:
        return empty_template_features(len(input_sequence))
    try:
        result = template_featurizer.get_templates(input_sequence, hits=flat, query_pdb_code=query_pdb_code, query_release_date=query_release_date)
    except TypeError:          # featurisers without the query-identity filters (hmmsearch hits of the multimer pipeline)
        result = template_featurizer.get_templates(input_sequence, hits=flat)
    feats = result.features
    if feats["template_aatype"].shape[0] == 0:
        return empty_template_features(len(input_sequence))
    return feats


def make_protein_features(protein_object, description: str, _is_distillation: bool = False) -> FeatureDict:
    """Sequence features + all-atom ground truth of a ``common.protein.Protein``."""
    aatype = np.asarray(protein_object.aatype)
    sequence = "".join(rc.restypes_with_x[int(a)] for a in aatype)
    feats = dict(make_sequence_features(sequence, description, len(aatype)))
    feats.update(_ground_truth_features(protein_object.atom_positions, protein_object.atom_mask, 0.0, _is_distillation))
    return feats


def make_pdb_features(protein_object, description: str, confidence_threshold: float = 50.0, is_distillation: bool = True) -> FeatureDict:
    """As ``make_protein_features``; for self-distillation targets (predicted structures with the confidence in the
    B-factor column) a residue none of whose atoms exceeds ``confidence_threshold`` is masked out of the ground truth
    (fastfold/data/data_pipeline.py:185-202, whose default of 0.5 on a 0-100 confidence scale keeps everything)."""
    feats = make_protein_features(protein_object, description, _is_distillation=True)
    if is_distillation:
        confident = (np.asarray(protein_object.b_factors) > confidence_threshold).any(axis=-1).astype(np.float32)
        feats["all_atom_mask"] = feats["all_atom_mask"] * confident[:, None]
    else:
        feats["is_distillation"] = np.array(0.0, np.float32)
    return feats


def make_mmcif_features(mmcif_object, chain_id: str) -> FeatureDict:
    """Sequence features + ground truth + resolution / release date of one chain of a parsed mmCIF file."""
    from . import mmcif_parsing
    sequence = mmcif_object.chain_to_seqres[chain_id]
    feats = dict(make_sequence_features(sequence, "%s_%s" % (mmcif_object.file_id, chain_id), len(sequence)))
    pos, mask = mmcif_parsing.get_atom_coords(mmcif_object, chain_id)
    header = mmcif_object.header
    get = header.get if isinstance(header, dict) else (lambda k, d=None: getattr(header, k, d))
    feats.update(_ground_truth_features(pos, mask, float(get("resolution", 0.0) or 0.0), False))
    feats["release_date"] = np.array([str(get("release_date", "")).encode()], dtype=object)
    return feats


def run_msa_tool(msa_runner, fasta_path: str, msa_out_path: str, msa_format: str, max_sto_sequences: Optional[int] = None):
    """Runs one alignment tool on a FASTA file and writes its result (``sto`` or ``a3m`` text) to ``msa_out_path``."""
    if msa_format == "sto" and max_sto_sequences is not None:
        result = msa_runner.query(fasta_path, max_sto_sequences)
    else:
        result = msa_runner.query(fasta_path)
    result = result[0] if isinstance(result, (list, tuple)) else result
    text = result[msa_format] if isinstance(result, Mapping) else result
    with open(msa_out_path, "w") as fh:
        fh.write(text)
    return result


import contextlib
import tempfile


@contextlib.contextmanager
def temp_fasta_file(fasta_str: str):
    """Path of a temporary FASTA file holding ``fasta_str`` (deleted on exit)."""
    with tempfile.NamedTemporaryFile("w", suffix=".fasta") as fh:
        fh.write(fasta_str)
        fh.flush()
        yield fh.name


def convert_monomer_features(monomer_features: FeatureDict, chain_id: str) -> FeatureDict:
    """Monomer-pipeline features in the form the multimer assembly expects: scalars without their leading axis, residue
    types as indices in this package's order, the template mask under its model-side name."""
    out = {"auth_chain_id": np.asarray(chain_id, dtype=object)}
    for name, value in monomer_features.items():
        if name in ("sequence", "domain_name", "num_alignments", "seq_length"):
            value = np.asarray(value[0], dtype=np.asarray(value).dtype)
        elif name == "aatype":
            value = np.argmax(value, axis=-1).astype(np.int32)
        elif name == "template_aatype":
            idx = np.argmax(value, axis=-1).astype(np.int32)
            value = np.take(np.asarray(rc.MAP_HHBLITS_AATYPE_TO_OUR_AATYPE), idx, axis=0)
        elif name == "template_all_atom_masks":
            name = "template_all_atom_mask"
        out[name] = value
    return out


def int_id_to_str_id(num: int) -> str:
    """1 -> A, 2 -> B, ..., 26 -> Z, 27 -> AA, 28 -> BA, 29 -> CA, ...: chain names as mmCIF files count them (least
    significant letter first)."""
    if num <= 0:
        raise ValueError("Only positive integers allowed, got %d." % num)
    num -= 1
    letters = []
    while num >= 0:
        letters.append(chr(ord("A") + num % 26))
        num = num // 26 - 1
    return "".join(letters)


class DataPipeline:
    def __init__(self, template_featurizer=None):
        self.template_featurizer = template_featurizer

    @staticmethod
    def _alignment_files(alignment_dir, _alignment_index=None):
        """``(file name, text)`` of every search output of one target, in name order.  They are the files of
        ``alignment_dir``, or - with ``_alignment_index = {"db": file, "files": [(name, offset, size), ...]}`` - byte ranges
        of one concatenated file ``alignment_dir/db`` (millions of small files become one; fastfold/data/data_pipeline.py:792-843)."""
        if _alignment_index is not None:
            with open(os.path.join(alignment_dir, _alignment_index["db"]), "rb") as fp:
                for name, start, size in sorted(_alignment_index["files"], key=lambda e: e[0]):
                    fp.seek(int(start))
                    yield name, fp.read(int(size)).decode("utf-8")
        elif alignment_dir and os.path.isdir(alignment_dir):
            for f in sorted(os.listdir(alignment_dir)):
                path = os.path.join(alignment_dir, f)
                if os.path.isfile(path) and os.path.splitext(f)[1] in (".a3m", ".sto", ".hhr"):
                    with open(path) as fp:
                        yield f, fp.read()

    @classmethod
    def _read_alignments(cls, alignment_dir, query, _alignment_index=None):
        msas = []
        for name, text in cls._alignment_files(alignment_dir, _alignment_index):
            stem, ext = os.path.splitext(name)
            if ext == ".a3m":
                msa = parsers.Msa(*parsers.parse_a3m(text)[:3])
            elif ext == ".sto" and stem not in ("hmm_output", "hmmsearch_output"):       # those hold template hits, not an MSA
                msa = parsers.Msa(*parsers.parse_stockholm(text)[:3])
            else:
                continue
            if len(msa) and len(msa.sequences[0]) == len(query):
                msas.append(msa)
        if not msas:      # single-sequence mode
            msas = [parsers.Msa([query], [[0] * len(query)], ["dummy"])]
        return msas

    @classmethod
    def _read_template_hits(cls, alignment_dir, input_sequence=None, _alignment_index=None):
        """``{file name: [TemplateHit]}``: hhsearch results (``*.hhr``) and, for the multimer pipeline, the hmmsearch
        alignment against the PDB sequences (``hmm_output.sto``; fastfold/data/data_pipeline.py:845-890)."""
        hits = {}
        for name, text in cls._alignment_files(alignment_dir, _alignment_index):
            if name.endswith(".hhr"):
                hits[name] = parsers.parse_hhr(text)
            elif name in ("hmm_output.sto", "hmmsearch_output.sto") and input_sequence is not None:
                hits[name] = parsers.parse_hmmsearch_sto(text, input_sequence)
        return hits

    def process_fasta(self, fasta_path: str, alignment_dir: Optional[str] = None, _alignment_index=None) -> FeatureDict:
        seqs, descs = parsers.parse_fasta(open(fasta_path).read())
        if len(seqs) != 1:
            raise ValueError("More than one input sequence found in %s." % fasta_path)
        return self.process_sequence(seqs[0], descs[0], alignment_dir, _alignment_index=_alignment_index)

    def process_sequence(self, sequence, description="query", alignment_dir=None, query_pdb_code=None, query_release_date=None,
                         _alignment_index=None) -> FeatureDict:
        """``query_pdb_code`` / ``query_release_date``: identity of the target when it is itself a PDB entry (training),
        so that the entry and anything released within 60 days before it are not used as templates."""
        n = len(sequence)
        feats = dict(make_sequence_features(sequence, description, n))
        feats.update(make_msa_features(self._read_alignments(alignment_dir, sequence, _alignment_index)))
        hits = {}
        if self.template_featurizer is not None and alignment_dir:
            hits = self._read_template_hits(alignment_dir, sequence, _alignment_index)
        feats.update(make_template_features(sequence, hits, self.template_featurizer, query_pdb_code, query_release_date))
        return feats


def _ground_truth_features(positions, mask, resolution=1.0, is_distillation=False):
    return {"all_atom_positions": np.asarray(positions, np.float32), "all_atom_mask": np.asarray(mask, np.float32),
            "resolution": np.array([resolution], np.float32), "is_distillation": np.array(1.0 if is_distillation else 0.0, np.float32)}


def _process_structure(self, sequence, description, alignment_dir, positions, mask, resolution, is_distillation, query_pdb_code=None,
                       query_release_date=None, _alignment_index=None):
    feats = dict(self.process_sequence(sequence, description, alignment_dir, query_pdb_code, query_release_date, _alignment_index=_alignment_index))
    feats.update(_ground_truth_features(positions, mask, resolution, is_distillation))
    return feats


def _process_pdb(self, pdb_path, alignment_dir=None, is_distillation=True, chain_id=None, _structure_index=None, _alignment_index=None):
    """Features + ground truth of one chain of a PDB file; with ``_structure_index`` (same form as an alignment index) the
    text is a byte range of one concatenated file beside ``pdb_path`` (fastfold/data/data_pipeline.py:1000-1047)."""
    from ..common import protein
    if _structure_index is not None:
        _, offset, length = _structure_index["files"][0]
        with open(os.path.join(os.path.dirname(pdb_path), _structure_index["db"]), "rb") as fp:
            fp.seek(int(offset))
            pdb_str = fp.read(int(length)).decode("utf-8")
    else:
        pdb_str = open(pdb_path).read()
    prot = protein.from_pdb_string(pdb_str, chain_id)
    seq = "".join(rc.restypes_with_x[int(a)] for a in prot.aatype)
    tag = os.path.splitext(os.path.basename(pdb_path))[0] + ("_" + chain_id if chain_id else "")
    return _process_structure(self, seq, tag, alignment_dir, prot.atom_positions, prot.atom_mask, 0.0 if is_distillation else 1.0, is_distillation,
                              _alignment_index=_alignment_index)


def _process_mmcif(self, mmcif, alignment_dir=None, chain_id=None, _alignment_index=None):
    """Features + ground truth of one chain of a parsed mmCIF file (fastfold/data/data_pipeline.py:738-778)."""
    from . import mmcif_parsing
    if chain_id is None:
        chains = list(mmcif.chain_to_seqres)
        if len(chains) != 1:
            raise ValueError("chain_id must be given for a file with %d chains" % len(chains))
        chain_id = chains[0]
    seq = mmcif.chain_to_seqres[chain_id]
    pos, mask = mmcif_parsing.get_atom_coords(mmcif, chain_id)
    res = mmcif.header.get("resolution", 0.0) if isinstance(mmcif.header, dict) else getattr(mmcif.header, "resolution", 0.0)
    date = mmcif.header.get("release_date", "") if isinstance(mmcif.header, dict) else getattr(mmcif.header, "release_date", "")
    feats = _process_structure(self, seq, "%s_%s" % (mmcif.file_id, chain_id), alignment_dir, pos, mask, float(res or 0.0), False,
                               query_pdb_code=mmcif.file_id, query_release_date=str(date) if date else None, _alignment_index=_alignment_index)
    feats["release_date"] = np.array([str(date).encode()], dtype=object)
    return feats


def _process_core(self, core_path, alignment_dir=None, _alignment_index=None):
    """Features + backbone ground truth of a ProteinNet ``.core`` record (fastfold/data/data_pipeline.py:1049-1079)."""
    from ..common import protein
    prot = protein.from_proteinnet_string(open(core_path).read())
    seq = "".join(rc.restypes_with_x[int(a)] for a in prot.aatype)
    tag = os.path.splitext(os.path.basename(core_path))[0].upper()
    return _process_structure(self, seq, tag, alignment_dir, prot.atom_positions, prot.atom_mask, 0.0, False, _alignment_index=_alignment_index)


DataPipeline.process_pdb = _process_pdb
DataPipeline.process_mmcif = _process_mmcif
DataPipeline.process_core = _process_core


def np_to_tensor_dict(np_example, features):
    return {k: torch.tensor(np.asarray(v)) for k, v in np_example.items() if k in features and np.asarray(v).dtype != object}


class FeaturePipeline:
    def __init__(self, config):
        self.config = config      # the ``data`` sub-tree of ``model_config``

    def process_features(self, raw_features: FeatureDict, mode: str = "predict", seed: int = 0, is_multimer=None):
        if is_multimer is None:
            is_multimer = "asym_id" in raw_features
        if is_multimer:
            return self._process_multimer(raw_features, mode, seed)
        from . import feature_pipeline as fp
        cfg = copy.deepcopy(self.config)
        raw = dict(raw_features)
        # prediction: templates take part only when the configuration uses them AND the example has at least one hit (the
        # caller switches the model's template stack off when no template features come back).  Training / evaluation
        # keep the static shapes: an example without hits gets zero-padded template features with ``template_mask`` 0.
        t = raw.get("template_aatype")
        has_templates = bool(cfg.common.use_templates) and t is not None and (np.asarray(t).shape[0] > 0 or mode != "predict")
        cfg.common.use_templates = has_templates
        feats = fp.np_example_to_features(raw, cfg, mode, seed=seed)
        if not has_templates:
            feats = {k: v for k, v in feats.items() if not k.startswith("template_")}
        return feats

    def _process_multimer(self, raw_features, mode, seed):
        """Merged multimer example (``DataPipelineMultimer.process_fasta``) -> model features: one pass of the multimer
        tensor transforms per recycling iteration (fresh MSA sample each), stacked on a trailing axis
        (fastfold/data/feature_pipeline.py:100-129, input_pipeline_multimer.py:113-136)."""
        from . import data_transforms_multimer as dtm
        cfg = copy.deepcopy(self.config)
        mode_cfg = cfg[mode]
        tensors = {k: torch.as_tensor(np.asarray(v)) for k, v in raw_features.items() if np.asarray(v).dtype != object}
        n_iter = cfg.common.max_recycling_iters + 1
        per_iter = []
        for it in range(n_iter):
            d = dtm.process_tensors({k: v.clone() for k, v in tensors.items()}, cfg.common, mode_cfg, seed=seed + it)
            # empty placeholders (e.g. ``template_sum_probs`` when no hit carries a score) are not model inputs
            d = {k: v for k, v in d.items() if isinstance(v, torch.Tensor) and v.numel() > 0}
            per_iter.append(d)
        keys = [k for k in per_iter[0] if all(k in d and d[k].shape == per_iter[0][k].shape for d in per_iter)]
        return {k: torch.stack([d[k] for d in per_iter], dim=-1) for k in keys}


# ---------------------------------------------------------------------------
# Running the alignment tools (fastfold/data/data_pipeline.py:262-560)
# ---------------------------------------------------------------------------
class AlignmentRunner:
    """Runs whichever searches have both a binary and a database, and writes their results into ``output_dir``:

    ``uniref90_hits.a3m`` (jackhmmer), ``pdb70_hits.hhr`` (hhsearch on the uniref90 profile), ``mgnify_hits.a3m``
    (jackhmmer) and ``bfd_uniref_hits.a3m`` (hhblits on BFD + UniRef30) or ``small_bfd_hits.sto`` (jackhmmer on small
    BFD).  The three independent searches run concurrently (they are subprocess-bound).
    """

    def __init__(self, jackhmmer_binary_path=None, hhblits_binary_path=None, hhsearch_binary_path=None, uniref90_database_path=None,
                 mgnify_database_path=None, bfd_database_path=None, uniref30_database_path=None, pdb70_database_path=None,
                 use_small_bfd=None, no_cpus=None, uniref_max_hits: int = 10000, mgnify_max_hits: int = 5000, uniprot_max_hits: int = 50000):
        from . import tools
        self.uniprot_max_hits = uniprot_max_hits       # used by the multimer runner's UniProt search
        groups = {"jackhmmer": (jackhmmer_binary_path, [uniref90_database_path, mgnify_database_path, bfd_database_path if use_small_bfd else None]),
                  "hhblits": (hhblits_binary_path, [bfd_database_path if not use_small_bfd else None]),
                  "hhsearch": (hhsearch_binary_path, [pdb70_database_path])}
        for name, (binary, dbs) in groups.items():
            if binary is None and any(d is not None for d in dbs):
                raise ValueError("%s DBs provided but %s binary is None" % (name, name))
        if pdb70_database_path is not None and uniref90_database_path is None:
            raise ValueError("uniref90_database_path must be specified in order to perform template search")
        self.uniref_max_hits, self.mgnify_max_hits, self.use_small_bfd = uniref_max_hits, mgnify_max_hits, use_small_bfd
        n_cpu = no_cpus or os.cpu_count() or 1
        mk_jack = lambda db: tools.Jackhmmer(binary_path=jackhmmer_binary_path, database_path=db, n_cpu=n_cpu) if db else None
        self.jackhmmer_uniref90_runner = mk_jack(uniref90_database_path) if jackhmmer_binary_path else None
        self.jackhmmer_mgnify_runner = mk_jack(mgnify_database_path) if jackhmmer_binary_path else None
        self.jackhmmer_small_bfd_runner = mk_jack(bfd_database_path) if (jackhmmer_binary_path and use_small_bfd) else None
        self.hhblits_bfd_uniref_runner = None
        if bfd_database_path is not None and not use_small_bfd:
            dbs = [bfd_database_path] + ([uniref30_database_path] if uniref30_database_path else [])
            self.hhblits_bfd_uniref_runner = tools.HHBlits(binary_path=hhblits_binary_path, databases=dbs, n_cpu=n_cpu)
        self.hhsearch_pdb70_runner = None
        if pdb70_database_path is not None:
            self.hhsearch_pdb70_runner = tools.HHSearch(binary_path=hhsearch_binary_path, databases=[pdb70_database_path], n_cpu=n_cpu)

    def _uniref_and_templates(self, fasta_path, output_dir):
        if self.jackhmmer_uniref90_runner is None:
            return
        sto = self.jackhmmer_uniref90_runner.query(fasta_path)[0]["sto"]
        a3m = parsers.convert_stockholm_to_a3m(sto, max_sequences=self.uniref_max_hits)
        with open(os.path.join(output_dir, "uniref90_hits.a3m"), "w") as f:
            f.write(a3m)
        if self.hhsearch_pdb70_runner is not None:
            with open(os.path.join(output_dir, "pdb70_hits.hhr"), "w") as f:
                f.write(self.hhsearch_pdb70_runner.query(a3m))

    def _mgnify(self, fasta_path, output_dir):
        if self.jackhmmer_mgnify_runner is None:
            return
        sto = self.jackhmmer_mgnify_runner.query(fasta_path)[0]["sto"]
        with open(os.path.join(output_dir, "mgnify_hits.a3m"), "w") as f:
            f.write(parsers.convert_stockholm_to_a3m(sto, max_sequences=self.mgnify_max_hits))

    def _bfd(self, fasta_path, output_dir):
        if self.use_small_bfd and self.jackhmmer_small_bfd_runner is not None:
            with open(os.path.join(output_dir, "small_bfd_hits.sto"), "w") as f:
                f.write(self.jackhmmer_small_bfd_runner.query(fasta_path)[0]["sto"])
        elif self.hhblits_bfd_uniref_runner is not None:
            with open(os.path.join(output_dir, "bfd_uniref_hits.a3m"), "w") as f:
                f.write(self.hhblits_bfd_uniref_runner.query(fasta_path)["a3m"])

    def run(self, fasta_path: str, output_dir: str):
        from concurrent.futures import ThreadPoolExecutor
        os.makedirs(output_dir, exist_ok=True)
        with ThreadPoolExecutor(max_workers=3) as pool:
            jobs = [pool.submit(fn, fasta_path, output_dir) for fn in (self._uniref_and_templates, self._mgnify, self._bfd)]
            for j in jobs:
                j.result()


class AlignmentRunnerMultimer(AlignmentRunner):
    """Per-chain searches of the multimer pipeline: Stockholm outputs (kept for species pairing), a UniProt search and
    an hmmsearch template search on PDB seqres (fastfold/data/data_pipeline.py:458-560)."""

    def __init__(self, jackhmmer_binary_path=None, hhblits_binary_path=None, hmmsearch_binary_path=None, hmmbuild_binary_path=None,
                 uniref90_database_path=None, mgnify_database_path=None, bfd_database_path=None, uniref30_database_path=None,
                 uniprot_database_path=None, pdb_seqres_database_path=None, use_small_bfd=None, no_cpus=None, uniref_max_hits: int = 10000,
                 mgnify_max_hits: int = 5000, uniprot_max_hits: int = 50000):
        from . import tools
        super().__init__(jackhmmer_binary_path=jackhmmer_binary_path, hhblits_binary_path=hhblits_binary_path,
                         uniref90_database_path=uniref90_database_path, mgnify_database_path=mgnify_database_path,
                         bfd_database_path=bfd_database_path, uniref30_database_path=uniref30_database_path, use_small_bfd=use_small_bfd,
                         no_cpus=no_cpus, uniref_max_hits=uniref_max_hits, mgnify_max_hits=mgnify_max_hits)
        self.uniprot_max_hits = uniprot_max_hits
        n_cpu = no_cpus or os.cpu_count() or 1
        self.jackhmmer_uniprot_runner = None
        if uniprot_database_path is not None:
            self.jackhmmer_uniprot_runner = tools.Jackhmmer(binary_path=jackhmmer_binary_path, database_path=uniprot_database_path, n_cpu=n_cpu)
        self.hmmsearch_pdb_runner = None
        if pdb_seqres_database_path is not None:
            self.hmmsearch_pdb_runner = tools.Hmmsearch(binary_path=hmmsearch_binary_path, hmmbuild_binary_path=hmmbuild_binary_path,
                                                        database_path=pdb_seqres_database_path)

    def _uniref_and_templates(self, fasta_path, output_dir):
        if self.jackhmmer_uniref90_runner is None:
            return
        sto = self.jackhmmer_uniref90_runner.query(fasta_path, max_sequences=self.uniref_max_hits)[0]["sto"]
        with open(os.path.join(output_dir, "uniref90_hits.sto"), "w") as f:
            f.write(sto)
        if self.hmmsearch_pdb_runner is not None:
            clean = parsers.remove_empty_columns_from_stockholm_msa(parsers.deduplicate_stockholm_msa(sto))
            # the search writes <output_dir>/hmm_output.sto, the name under which the data pipeline looks for template hits
            self.hmmsearch_pdb_runner.query(clean, output_dir=output_dir)

    def _mgnify(self, fasta_path, output_dir):
        if self.jackhmmer_mgnify_runner is None:
            return
        with open(os.path.join(output_dir, "mgnify_hits.sto"), "w") as f:
            f.write(self.jackhmmer_mgnify_runner.query(fasta_path, max_sequences=self.mgnify_max_hits)[0]["sto"])

    def _uniprot(self, fasta_path, output_dir):
        if self.jackhmmer_uniprot_runner is None:
            return
        with open(os.path.join(output_dir, "uniprot_hits.sto"), "w") as f:
            f.write(self.jackhmmer_uniprot_runner.query(fasta_path, max_sequences=self.uniprot_max_hits)[0]["sto"])

    def run(self, fasta_path: str, output_dir: str):
        from concurrent.futures import ThreadPoolExecutor
        os.makedirs(output_dir, exist_ok=True)
        with ThreadPoolExecutor(max_workers=4) as pool:
            jobs = [pool.submit(fn, fasta_path, output_dir) for fn in (self._uniref_and_templates, self._mgnify, self._bfd, self._uniprot)]
            for j in jobs:
                j.result()


# ---------------------------------------------------------------------------
# Multimer (fastfold/data/data_pipeline.py:1010-1189)
# ---------------------------------------------------------------------------
class DataPipelineMultimer:
    """Features of a complex from a multi-sequence FASTA: every distinct chain goes through the monomer pipeline
    (alignments under ``<alignment_dir>/<chain id>/``), its UniProt hits (``uniprot_hits.sto``) supply the species-tagged
    rows for cross-chain pairing, then ``msa_pairing.pair_and_merge`` assembles the complex."""

    def __init__(self, monomer_data_pipeline: DataPipeline, max_uniprot_hits: int = 50000):
        self._monomer = monomer_data_pipeline
        self._max_uniprot_hits = max_uniprot_hits

    def _all_seq_features(self, chain_alignment_dir, sequence):
        from . import msa_pairing
        path = os.path.join(chain_alignment_dir, "uniprot_hits.sto") if chain_alignment_dir else None
        if not path or not os.path.exists(path):
            msa, dels, descs = [sequence], [[0] * len(sequence)], ["query"]
        else:
            msa, dels, descs = parsers.parse_stockholm(open(path).read())
            msa, dels, descs = msa[:self._max_uniprot_hits], dels[:self._max_uniprot_hits], descs[:self._max_uniprot_hits]
        feats = make_msa_features([parsers.Msa(list(msa), list(dels), list(descs))])
        return {k + "_all_seq": feats[k] for k in ("msa", "deletion_matrix_int", "msa_species_identifiers")}

    def _process_chain(self, chain_id, sequence, description, alignment_dir, is_homomer_or_monomer):
        chain_dir = os.path.join(alignment_dir, chain_id) if alignment_dir else None
        feats = dict(self._monomer.process_sequence(sequence, description, chain_dir if chain_dir and os.path.isdir(chain_dir) else None))
        if not is_homomer_or_monomer:
            feats.update(self._all_seq_features(chain_dir, sequence))
        return feats

    def process_fasta(self, fasta_path: str, alignment_dir: Optional[str] = None) -> FeatureDict:
        from . import msa_pairing
        seqs, descs = parsers.parse_fasta(open(fasta_path).read())
        is_homomer_or_monomer = len(set(seqs)) == 1
        cache, all_chains = {}, {}
        for i, (seq, desc) in enumerate(zip(seqs, descs)):
            chain_id = desc.split()[0] if desc.split() else "chain_%d" % i
            if seq not in cache:
                cache[seq] = self._process_chain(chain_id, seq, desc, alignment_dir, is_homomer_or_monomer)
            all_chains["%d_%s" % (i, chain_id)] = copy.deepcopy(cache[seq])
        all_chains = msa_pairing.add_assembly_features(all_chains)
        example = msa_pairing.pair_and_merge(all_chains)
        return msa_pairing.pad_msa(example, 512)


# fastfold/data/data_pipeline.py:727-781 defines these two beside the pipelines; they live with the other assembly code.
from .msa_pairing import add_assembly_features, pad_msa  # noqa: E402,F401
