"""Multimer feature assembly: species identifiers, cross-chain MSA row pairing, and merging per-chain features into
one complex (roles of fastfold/data/msa_identifiers.py, msa_pairing.py and feature_processing_multimer.py).

Pipeline (``pair_and_merge``):

1. every chain arrives with monomer-style features plus ``*_all_seq`` features from its UniProt search (these carry a
   species identifier per row);
2. rows of different chains that come from the same species are paired (within a species, rows are matched by their
   rank of similarity to the chain's query), the paired block is ordered by how many chains each row covers;
3. rows already used in the paired block are removed from the chains' own (unpaired) MSAs;
4. per-residue features are concatenated along the residue axis, paired MSAs side by side, unpaired MSAs
   block-diagonally (gaps elsewhere), templates side by side;
5. masks and bookkeeping features (``asym_id`` / ``entity_id`` / ``sym_id``, ``num_alignments``) are finalised.
"""
import collections
import dataclasses
import re
import string
from typing import Dict, Iterable, List, Mapping, MutableMapping, Optional, Sequence

import numpy as np

from ..common import residue_constants as rc

MSA_GAP_IDX = rc.restypes_with_x_and_gap.index("-") if hasattr(rc, "restypes_with_x_and_gap") else 21
SEQUENCE_GAP_CUTOFF = 0.5
SEQUENCE_SIMILARITY_CUTOFF = 0.9
MSA_PAD_VALUES = {"msa_all_seq": MSA_GAP_IDX, "msa_mask_all_seq": 1, "deletion_matrix_all_seq": 0, "deletion_matrix_int_all_seq": 0, "msa": MSA_GAP_IDX,
                  "msa_mask": 1, "deletion_matrix": 0, "deletion_matrix_int": 0}
MSA_FEATURES = ("msa", "msa_mask", "deletion_matrix", "deletion_matrix_int")
SEQ_FEATURES = ("residue_index", "aatype", "all_atom_positions", "all_atom_mask", "seq_mask", "between_segment_residues", "has_alt_locations",
                "has_hetatoms", "asym_id", "entity_id", "sym_id", "entity_mask", "deletion_mean", "prediction_atom_mask", "literature_positions",
                "atom_indices_to_group_indices", "rigid_group_default_frame")
TEMPLATE_FEATURES = ("template_aatype", "template_all_atom_positions", "template_all_atom_mask")
CHAIN_FEATURES = ("num_alignments", "seq_length")
REQUIRED_FEATURES = frozenset({
    "aatype", "all_atom_mask", "all_atom_positions", "all_chains_entity_ids", "all_crops_all_chains_mask", "all_crops_all_chains_positions",
    "all_crops_all_chains_residue_ids", "assembly_num_chains", "asym_id", "bert_mask", "cluster_bias_mask", "deletion_matrix", "deletion_mean",
    "entity_id", "entity_mask", "mem_peak", "msa", "msa_mask", "num_alignments", "num_templates", "queue_size", "residue_index", "resolution",
    "seq_length", "seq_mask", "sym_id", "template_aatype", "template_all_atom_mask", "template_all_atom_positions"})


# ---------------------------------------------------------------------------
# identifiers (fastfold/data/msa_identifiers.py)
# ---------------------------------------------------------------------------
_UNIPROT_PATTERN = re.compile(
    r"""^(?:tr|sp)\|(?:[A-Za-z0-9]{6,10})(?:_\d)?\|(?:[A-Za-z0-9]+)_(?P<SpeciesIdentifier>[A-Za-z0-9]{1,5})(?:_\d+)?$""")


@dataclasses.dataclass(frozen=True)
class Identifiers:
    species_id: str = ""


def get_identifiers(description: str) -> Identifiers:
    """Species identifier from a UniProt-style MSA row description (``tr|A0A146SKV9|A0A146SKV9_FUNHE/2-98``)."""
    first = description.split()[0].partition("/")[0] if description.split() else ""     # drop the residue range
    m = _UNIPROT_PATTERN.match(first.strip())
    return Identifiers(species_id=m.group("SpeciesIdentifier")) if m else Identifiers()


# ---------------------------------------------------------------------------
# pairing
# ---------------------------------------------------------------------------
def _is_homomer_or_monomer(chains: Iterable[Mapping[str, np.ndarray]]) -> bool:
    ids = np.concatenate([np.unique(c["entity_id"][c["entity_id"] > 0]) for c in chains])
    return len(set(ids.tolist())) == 1


def _similarity_to_query(msa: np.ndarray) -> np.ndarray:
    return (msa == msa[0][None]).mean(axis=-1)


def _species_rows(chain: Mapping[str, np.ndarray]) -> Dict[bytes, np.ndarray]:
    """species id -> row indices of the chain's ``*_all_seq`` MSA, most query-like first."""
    species = np.asarray(chain["msa_species_identifiers_all_seq"])
    msa = chain["msa_all_seq"]
    sim = _similarity_to_query(msa)
    gap_frac = (msa == MSA_GAP_IDX).mean(axis=-1)
    out: Dict[bytes, List[int]] = collections.defaultdict(list)
    order = np.argsort(-sim, kind="stable")
    for r in order:
        if gap_frac[r] >= SEQUENCE_GAP_CUTOFF and r != 0:
            continue
        out[bytes(species[r]) if not isinstance(species[r], bytes) else species[r]].append(int(r))
    return {k: np.array(v) for k, v in out.items()}


def pair_sequences(chains: Sequence[Mapping[str, np.ndarray]]) -> np.ndarray:
    """Row index table ``[num_paired_rows, num_chains]`` (-1: chain absent from that row); row 0 pairs the queries."""
    n = len(chains)
    per_chain = [_species_rows(c) for c in chains]
    all_species = set()
    for d in per_chain:
        all_species |= set(d)
    all_species.discard(b"")
    rows = [np.zeros((1, n), dtype=np.int64)]
    by_count: Dict[int, List[np.ndarray]] = collections.defaultdict(list)
    for sp in sorted(all_species):
        present = [i for i in range(n) if sp in per_chain[i]]
        if len(present) < 2:
            continue
        if any(len(per_chain[i][sp]) > 600 for i in present):      # species with huge families: pairing is unreliable
            continue
        depth = min(len(per_chain[i][sp]) for i in present)
        block = -np.ones((depth, n), dtype=np.int64)
        for i in present:
            block[:, i] = per_chain[i][sp][:depth]
        by_count[len(present)].append(block)
    for k in sorted(by_count, reverse=True):                       # rows covering more chains first
        rows.extend(by_count[k])
    return np.concatenate(rows, axis=0)


def create_paired_features(chains: Sequence[MutableMapping[str, np.ndarray]]) -> List[MutableMapping[str, np.ndarray]]:
    """Re-orders every chain's ``*_all_seq`` features into the common paired row order (gap rows where a chain has no partner)."""
    chains = list(chains)
    if len(chains) < 2:
        return chains
    table = pair_sequences(chains)
    out = []
    for i, chain in enumerate(chains):
        new = {k: v for k, v in chain.items() if "_all_seq" not in k}
        idx = table[:, i]
        for key in ("msa_all_seq", "msa_mask_all_seq", "deletion_matrix_all_seq", "deletion_matrix_int_all_seq"):
            if key not in chain:
                continue
            feat = chain[key]
            pad = np.full((1,) + feat.shape[1:], MSA_PAD_VALUES[key], dtype=feat.dtype)
            padded = np.concatenate([feat, pad], axis=0)
            new[key] = padded[np.where(idx >= 0, idx, feat.shape[0])]
        if "msa_species_identifiers_all_seq" in chain:
            sp = np.asarray(chain["msa_species_identifiers_all_seq"], dtype=object)
            new["msa_species_identifiers_all_seq"] = np.array([sp[j] if j >= 0 else b"" for j in idx], dtype=object)
        new["num_alignments_all_seq"] = np.asarray(len(idx))
        out.append(new)
    return out


def deduplicate_unpaired_sequences(chains: Sequence[MutableMapping[str, np.ndarray]]) -> List[MutableMapping[str, np.ndarray]]:
    """Drops rows of the unpaired MSAs that already appear in the chain's paired block."""
    out = []
    for chain in chains:
        chain = dict(chain)
        if "msa_all_seq" in chain:
            paired = {row.tobytes() for row in chain["msa_all_seq"].astype(np.int8)}
            keep = [i for i, row in enumerate(chain["msa"].astype(np.int8)) if row.tobytes() not in paired]
            for k in MSA_FEATURES:
                if k in chain:
                    chain[k] = chain[k][keep]
            chain["num_alignments"] = np.array(len(keep), dtype=np.int32)
        out.append(chain)
    return out


# ---------------------------------------------------------------------------
# merging
# ---------------------------------------------------------------------------
def block_diag(*arrs: np.ndarray, pad_value: float = 0.0) -> np.ndarray:
    """Block-diagonal arrangement of 2-D (or higher: leading two axes) arrays with ``pad_value`` off the diagonal."""
    return _block_diag(list(arrs), pad_value)


def pad_features(feature: np.ndarray, feature_name: str) -> np.ndarray:
    """Appends the "absent partner" row to a paired (``*_all_seq``) MSA feature: the row a chain contributes to a
    paired alignment row in which it has no sequence.  Other features are returned unchanged."""
    if feature_name in ("msa_all_seq", "msa_mask_all_seq", "deletion_matrix_all_seq", "deletion_matrix_int_all_seq"):
        pad = np.full((1,) + feature.shape[1:], MSA_PAD_VALUES[feature_name], dtype=feature.dtype)
        return np.concatenate([feature, pad], axis=0)
    if feature_name == "msa_species_identifiers_all_seq":
        return np.concatenate([np.asarray(feature, dtype=object), np.array([b""], dtype=object)], axis=0)
    return feature


def reorder_paired_rows(all_paired_msa_rows_dict: Mapping[int, np.ndarray]) -> np.ndarray:
    """``{number of chains a row covers: [rows, chains] index table}`` -> one table: rows covering more chains first,
    within a group the rows whose indices are smallest (most query-like in every chain) first."""
    out = []
    for n_chains in sorted(all_paired_msa_rows_dict, reverse=True):
        rows = np.asarray(all_paired_msa_rows_dict[n_chains])
        if rows.size == 0:
            continue
        rank = np.abs(np.prod(rows.astype(np.float64), axis=1))
        out.extend(rows[np.argsort(rank, kind="stable")])
    return np.array(out)


def crop_chains(chains_list: Sequence[MutableMapping[str, np.ndarray]], msa_crop_size: int, pair_msa_sequences: bool,
                max_templates: int) -> List[MutableMapping[str, np.ndarray]]:
    """Caps the MSA depth and the template count of every chain before merging.  With pairing, at most half of the
    budget goes to the paired block, and the unpaired rows get what is left after the chain's NON-GAP paired rows were
    counted, so that every chain ends up with about ``msa_crop_size`` sequences of its own
    (fastfold/data/feature_processing_multimer.py:87-166)."""
    out = []
    for chain in chains_list:
        chain = dict(chain)
        depth = int(chain["msa"].shape[0])
        keep_paired = 0
        if pair_msa_sequences and "msa_all_seq" in chain:
            depth_paired = int(chain["msa_all_seq"].shape[0])
            keep_paired = min(depth_paired, msa_crop_size // 2)
            block = chain["msa_all_seq"][:keep_paired]
            own_rows = int(np.sum(np.any(block != MSA_GAP_IDX, axis=1)))
            keep = min(depth, max(msa_crop_size - min(own_rows, keep_paired), 0))
        else:
            keep = min(depth, msa_crop_size)
        n_templates = None
        if "template_aatype" in chain and max_templates:
            n_templates = min(chain["template_aatype"].shape[0], max_templates)
        for k in list(chain):
            base = k.split("_all_seq")[0]
            if base in TEMPLATE_FEATURES and n_templates is not None:
                chain[k] = chain[k][:n_templates]
            elif base in MSA_FEATURES or base == "msa_species_identifiers":
                if "_all_seq" in k:
                    if pair_msa_sequences:
                        chain[k] = chain[k][:keep_paired]
                else:
                    chain[k] = chain[k][:keep]
        chain["num_alignments"] = np.asarray(keep, dtype=np.int32)
        if n_templates is not None:
            chain["num_templates"] = np.asarray(n_templates, dtype=np.int32)
        if pair_msa_sequences and "msa_all_seq" in chain:
            chain["num_alignments_all_seq"] = np.asarray(keep_paired, dtype=np.int32)
        out.append(chain)
    return out


def _block_diag(arrs: Sequence[np.ndarray], pad_value) -> np.ndarray:
    rows = sum(a.shape[0] for a in arrs)
    cols = sum(a.shape[1] for a in arrs)
    out = np.full((rows, cols) + arrs[0].shape[2:], pad_value, dtype=arrs[0].dtype)
    r = c = 0
    for a in arrs:
        out[r:r + a.shape[0], c:c + a.shape[1]] = a
        r += a.shape[0]
        c += a.shape[1]
    return out


def _pad_templates(chains, max_templates=4):
    """Every chain gets exactly ``max_templates`` template slots (zero-filled), so the template axis lines up when the
    chains are concatenated along the residues."""
    for c in chains:
        for k in TEMPLATE_FEATURES:
            if k in c:
                pad = max_templates - c[k].shape[0]
                if pad > 0:
                    c[k] = np.pad(c[k], [(0, pad)] + [(0, 0)] * (c[k].ndim - 1))
    return chains


def _merge_group(chains, dense: bool) -> Dict[str, np.ndarray]:
    """One feature dict from several: per-residue features are concatenated, template features concatenated along the
    residues, per-chain counts added up, anything else taken from the first chain.  Alignment features are concatenated
    along the residues when ``dense`` (the chains share their rows) - as the ``*_all_seq`` (paired) blocks always are - and
    laid out block-diagonally, gap-filled, otherwise."""
    merged: Dict[str, np.ndarray] = {}
    for k in chains[0]:
        vals = [c[k] for c in chains]
        base = k.split("_all_seq")[0]
        if base in MSA_FEATURES:
            merged[k] = np.concatenate(vals, axis=1) if (dense or "_all_seq" in k) else _block_diag(vals, MSA_PAD_VALUES[k])
        elif base in SEQ_FEATURES:
            merged[k] = np.concatenate(vals, axis=0)
        elif base in TEMPLATE_FEATURES:
            merged[k] = np.concatenate(vals, axis=1)
        elif base in CHAIN_FEATURES:
            merged[k] = np.sum([np.asarray(v) for v in vals], axis=0).astype(np.int32)
        else:
            merged[k] = vals[0]
    return merged


def _merge_homomers_dense_msa(chains) -> List[Dict[str, np.ndarray]]:
    """Copies of one sequence (same ``entity_id``) share their alignment: they are merged first, their rows side by side,
    which keeps the MSA of a homo-oligomer dense instead of block-diagonal (fastfold/data/msa_pairing.py:391-415)."""
    by_entity: Dict[int, list] = collections.defaultdict(list)
    for c in chains:
        by_entity[int(np.asarray(c["entity_id"]).reshape(-1)[0])].append(c)
    return [_merge_group(by_entity[e], dense=True) for e in sorted(by_entity)]


def merge_chain_features(np_chains_list: Sequence[MutableMapping[str, np.ndarray]], pair_msa_sequences: bool, max_templates: int = 4) -> Dict[str, np.ndarray]:
    """All chains into one example (fastfold/data/msa_pairing.py:270-333, 433-460): templates padded to a common count,
    copies of one sequence merged densely, the entities' own rows laid out block-diagonally, the species-paired rows (if
    any) stacked on top, then the features that only exist for the whole complex:

    * ``seq_length`` (total, repeated per residue) and ``num_alignments``;
    * ``cluster_bias_mask``: 1 on the rows that must always be among the cluster centres - the first row of the merged MSA
      when rows are paired, else the first row (the entity's own sequence) of every diagonal block;
    * ``bert_mask``: 1 where a row really covers a residue; the gap-filled off-diagonal area is never scored.
    """
    chains = _pad_templates([dict(c) for c in np_chains_list], max_templates)
    groups = _merge_homomers_dense_msa(chains)
    merged = _merge_group(groups, dense=False)
    own_rows = _block_diag([np.ones(g["msa"].shape, dtype=np.float32) for g in groups], 0)
    if pair_msa_sequences:
        for k in MSA_FEATURES:
            if k in merged and k + "_all_seq" in merged:
                merged[k] = np.concatenate([merged[k + "_all_seq"], merged[k]], axis=0)
        bias = np.zeros(merged["msa"].shape[0])
        bias[0] = 1
        paired_rows = np.concatenate([np.ones(g["msa_all_seq"].shape, dtype=np.float32) for g in groups], axis=1)
        merged["bert_mask"] = np.concatenate([paired_rows, own_rows], axis=0)
    else:
        bias = np.concatenate([np.eye(1, g["msa"].shape[0])[0] for g in groups])
        merged["bert_mask"] = own_rows
    merged["cluster_bias_mask"] = bias
    num_res = merged["aatype"].shape[0]
    merged["seq_length"] = np.asarray([num_res] * num_res, dtype=np.int32)
    merged["num_alignments"] = np.asarray(merged["msa"].shape[0], dtype=np.int32)
    return merged


def _correct_msa_restypes(msa: np.ndarray) -> np.ndarray:
    return np.take(np.array(rc.MAP_HHBLITS_AATYPE_TO_OUR_AATYPE, dtype=msa.dtype), msa, axis=0)


def process_unmerged_features(chains: Sequence[MutableMapping[str, np.ndarray]]) -> List[MutableMapping[str, np.ndarray]]:
    n_chains = len(chains)
    out = []
    for c in chains:
        c = dict(c)
        if "deletion_matrix_int" in c:
            c["deletion_matrix"] = np.asarray(c.pop("deletion_matrix_int"), dtype=np.float32)
        if "deletion_matrix_int_all_seq" in c:
            c["deletion_matrix_all_seq"] = np.asarray(c.pop("deletion_matrix_int_all_seq"), dtype=np.float32)
        c["deletion_mean"] = np.mean(c["deletion_matrix"], axis=0)
        if c["aatype"].ndim == 2:
            c["aatype"] = np.argmax(c["aatype"], axis=-1).astype(np.int32)
        if "template_aatype" in c and c["template_aatype"].ndim == 3:
            t = np.argmax(c["template_aatype"], axis=-1).astype(np.int32)
            c["template_aatype"] = _correct_msa_restypes(t)
        if "template_all_atom_masks" in c:
            c["template_all_atom_mask"] = c.pop("template_all_atom_masks")
        n = c["aatype"].shape[0]
        c["seq_length"] = np.asarray(n, dtype=np.int32)
        c["seq_mask"] = np.ones(n, dtype=np.float32)
        c["msa_mask"] = np.ones(c["msa"].shape, dtype=np.float32)
        if "msa_all_seq" in c:
            c["msa_mask_all_seq"] = np.ones(c["msa_all_seq"].shape, dtype=np.float32)
        if "all_atom_mask" not in c:
            # inference has no structure: the atoms each residue type has, at the origin (fastfold/data/feature_processing_multimer.py:235-241)
            c["all_atom_mask"] = np.asarray(rc.restype_atom37_mask, dtype=np.int32)[np.clip(c["aatype"], 0, 20)]
            c["all_atom_positions"] = np.zeros(c["all_atom_mask"].shape + (3,))
        c["assembly_num_chains"] = np.asarray(n_chains)
        c["entity_mask"] = (c["entity_id"] != 0).astype(np.int32)
        out.append(c)
    return out


def process_final(example: MutableMapping[str, np.ndarray]) -> Dict[str, np.ndarray]:
    example = dict(example)
    example["msa"] = _correct_msa_restypes(example["msa"].astype(np.int64)).astype(np.int32)
    example["seq_mask"] = (example["entity_id"] > 0).astype(np.float32)
    example["msa_mask"] = (example["msa"] != MSA_GAP_IDX).astype(np.float32) if "msa_mask" not in example else example["msa_mask"].astype(np.float32)
    first_row_ok = example["seq_mask"]
    example["msa_mask"] = example["msa_mask"] * first_row_ok[None]
    if "template_aatype" in example and "num_templates" not in example:     # else: the first chain's count after cropping
        example["num_templates"] = np.asarray(example["template_aatype"].shape[0], dtype=np.int32)
    return {k: v for k, v in example.items() if k in REQUIRED_FEATURES or k.startswith("template_") or k in ("cluster_bias_mask",)}


def pair_and_merge(all_chain_features: Mapping[str, MutableMapping[str, np.ndarray]], max_msa_crop: int = 2048, max_templates: int = 4) -> Dict[str, np.ndarray]:
    """From ``{chain id: features}`` to the merged feature dict of the complex
    (fastfold/data/feature_processing_multimer.py:44-90)."""
    chains = process_unmerged_features(list(all_chain_features.values()))
    pair = not _is_homomer_or_monomer(chains) and all("msa_all_seq" in c for c in chains)
    if pair:
        chains = create_paired_features(chains)
        chains = deduplicate_unpaired_sequences(chains)
    chains = crop_chains(chains, msa_crop_size=max_msa_crop, pair_msa_sequences=pair, max_templates=max_templates)
    merged = merge_chain_features(chains, pair_msa_sequences=pair, max_templates=max_templates)
    return process_final(merged)


# ---------------------------------------------------------------------------
# assembly bookkeeping (fastfold/data/data_pipeline.py: add_assembly_features, convert_monomer_features)
# ---------------------------------------------------------------------------
def add_assembly_features(all_chain_features: Mapping[str, MutableMapping[str, np.ndarray]]) -> Dict[str, MutableMapping[str, np.ndarray]]:
    """Adds ``asym_id`` (chain number), ``entity_id`` (number of the distinct sequence) and ``sym_id`` (copy number of
    that sequence); chain ids become ``<letter>_<copy>``."""
    seq_to_entity: Dict[str, int] = {}
    grouped: Dict[int, List[MutableMapping[str, np.ndarray]]] = collections.defaultdict(list)
    for feats in all_chain_features.values():
        first = np.asarray(feats["sequence"]).reshape(-1)[0]          # [1] from the monomer pipeline, 0-d after convert_monomer_features
        seq = first.decode() if isinstance(first, bytes) else str(first)
        ent = seq_to_entity.setdefault(seq, len(seq_to_entity) + 1)
        grouped[ent].append(feats)
    out, chain_no = {}, 1
    for ent, group in grouped.items():
        for sym, feats in enumerate(group, 1):
            n = int(np.asarray(feats["seq_length"]).reshape(-1)[0])
            feats = dict(feats)
            feats["asym_id"] = chain_no * np.ones(n, dtype=np.int64)
            feats["sym_id"] = sym * np.ones(n, dtype=np.int64)
            feats["entity_id"] = ent * np.ones(n, dtype=np.int64)
            out["%s_%d" % (string.ascii_uppercase[(ent - 1) % 26], sym)] = feats
            chain_no += 1
    return out


def pad_msa(example: MutableMapping[str, np.ndarray], min_num_seq: int) -> MutableMapping[str, np.ndarray]:
    example = dict(example)
    n = example["msa"].shape[0]
    if n < min_num_seq:
        pad = min_num_seq - n
        for k in ("msa", "deletion_matrix", "bert_mask", "msa_mask"):
            if k in example:
                example[k] = np.pad(example[k], ((0, pad), (0, 0)))      # zeros everywhere: the rows are switched off by msa_mask
        if "cluster_bias_mask" in example:
            example["cluster_bias_mask"] = np.pad(example["cluster_bias_mask"], ((0, pad),))
    return example
