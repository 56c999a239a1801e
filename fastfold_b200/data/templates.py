"""Template features from template-search hits and mmCIF files.

For every hit (best ``sum_probs`` first) until ``max_hits`` templates are accepted: cheap rejections first (released
after the cut-off date, a near-duplicate of the query, too short, too little of the query aligned), then the mmCIF
file of the hit is parsed, the hit sequence is located in one of its chains (exact chain, any chain containing the
sequence, or - as a last resort - a kalign realignment of the hit against the chain's real sequence), and the chain's
atom coordinates are scattered to query positions through the hit's alignment.  The result is the feature set the
model's template embedder consumes: ``template_aatype`` (one-hot over the 22 HH-suite letters), ``template_all_atom_
positions`` / ``_masks`` (atom37), ``template_sequence``, ``template_domain_names``, ``template_sum_probs``.

Same role and acceptance rules as fastfold/data/templates.py (prefilter :173-246, chain search :249-307, realignment
:310-417, feature extraction :458-612, featurizer classes :828-1221); mmCIF files are read by the dependency-free
parser in ``mmcif_parsing``.
"""
import dataclasses
import datetime
import glob
import logging
import os
import re
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

import numpy as np

from ..common import residue_constants as rc
from . import mmcif_parsing, parsers
from .tools import Kalign

log = logging.getLogger(__name__)


class Error(Exception):
    pass


class NoChainsError(Error):
    pass


class SequenceNotInTemplateError(Error):
    pass


class NoAtomDataInTemplateError(Error):
    pass


class TemplateAtomMaskAllZerosError(Error):
    pass


class QueryToTemplateAlignError(Error):
    pass


class CaDistanceError(Error):
    pass


class MultipleChainsError(Error):
    pass


class PrefilterError(Exception):
    pass


class PdbIdError(PrefilterError):
    """The hit is the query's own PDB entry."""


class DateError(PrefilterError):
    pass


class AlignRatioError(PrefilterError):
    pass


class DuplicateError(PrefilterError):
    pass


class LengthError(PrefilterError):
    pass


TEMPLATE_FEATURES = {"template_aatype": np.int64, "template_all_atom_mask": np.float32, "template_all_atom_positions": np.float32,
                     "template_domain_names": object, "template_sequence": object, "template_sum_probs": np.float32}


# ---------------------------------------------------------------------------
# small helpers
# ---------------------------------------------------------------------------
def _hit_pdb_id_and_chain(hit: parsers.TemplateHit) -> Tuple[str, str]:
    m = re.match(r"[a-zA-Z\d]{4}_[a-zA-Z0-9.]+", hit.name)
    if not m:
        raise ValueError("hit.name did not start with PDBID_chain: %s" % hit.name)
    pdb_id, chain = m.group(0).split("_")
    return pdb_id.lower(), chain


def _parse_release_dates(path: str) -> Mapping[str, datetime.datetime]:
    """``{pdb id: release date}`` from a JSON cache (``{"1abc": {"release_date": "1999-01-01"}, ...}``) or a two-column text file."""
    if path.endswith("json"):
        import json
        data = json.load(open(path))
        return {k.lower(): datetime.datetime.strptime(v["release_date"] if isinstance(v, dict) else v, "%Y-%m-%d") for k, v in data.items()}
    out = {}
    for line in open(path):
        parts = line.replace(":", " ").split()
        if len(parts) >= 2:
            out[parts[0].strip().lower()] = datetime.datetime.strptime(parts[1][:10], "%Y-%m-%d")
    return out


def generate_release_dates_cache(mmcif_dir: str, out_path: str) -> Mapping[str, str]:
    """Parses every ``*.cif`` of ``mmcif_dir`` once and writes ``{pdb id: {"release_date": "YYYY-MM-DD"}}`` as JSON: the
    cache ``TemplateHitFeaturizer(release_dates_path=...)`` reads, so that hits can be date-filtered without opening
    their files."""
    import json
    dates = {}
    for name in sorted(os.listdir(mmcif_dir)):
        if not name.endswith(".cif"):
            continue
        file_id = os.path.splitext(name)[0]
        with open(os.path.join(mmcif_dir, name)) as fh:
            parsed = mmcif_parsing.parse(file_id=file_id, mmcif_string=fh.read())
        if parsed.mmcif_object is None:
            log.info("Failed to parse %s. Skipping...", name)
            continue
        header = parsed.mmcif_object.header
        date = header.get("release_date") if isinstance(header, dict) else getattr(header, "release_date", None)
        if date:
            dates[file_id] = {"release_date": str(date)}
    with open(out_path, "w") as fh:
        json.dump(dates, fh)
    return dates


def _parse_obsolete(path: str) -> Mapping[str, Optional[str]]:
    """The PDB's ``obsolete.dat``: ``OBSLTE  date  old  [new]`` lines -> ``{old: new or None}``."""
    out = {}
    for line in open(path):
        if line.startswith("OBSLTE"):
            f = line.split()
            if len(f) >= 3:
                out[f[2].lower()] = f[3].lower() if len(f) > 3 else None
    return out


def _is_after_cutoff(pdb_id, release_dates, cutoff: Optional[datetime.datetime]) -> bool:
    if cutoff is None:
        raise ValueError("The release_date_cutoff must not be None.")
    if pdb_id in release_dates:
        return release_dates[pdb_id] > cutoff
    return False


def build_query_to_hit_index_mapping(hit_query_sequence, hit_sequence, indices_hit, indices_query, original_query_sequence) -> Dict[int, int]:
    """Index in the original query -> index in the hit's (gap-free) aligned sequence, for the columns where both have a
    residue.  The alignment's own indices (``-1`` = gap) are first made relative to their smallest entry on both sides; the
    query side is then moved to where the aligned query segment occurs in the original query - the search may have been
    run with a part of it.  Pairs that would fall outside either sequence are dropped (fastfold/data/templates.py:681-738)."""
    if not hit_query_sequence:
        return {}
    offset = original_query_sequence.find(hit_query_sequence.replace("-", ""))
    n_hit = len(hit_sequence.replace("-", ""))

    def relative(indices):
        present = [x for x in indices if x > -1]
        low = min(present) if present else 0
        return [x - low if x > -1 else -1 for x in indices]

    mapping = {}
    for q, t in zip(relative(indices_query), relative(indices_hit)):
        if q != -1 and t != -1 and t < n_hit and q + offset < len(original_query_sequence):
            mapping[q + offset] = t
    return mapping


# ---------------------------------------------------------------------------
# prefilter
# ---------------------------------------------------------------------------
def assess_hit(hit: parsers.TemplateHit, hit_pdb_code: str, query_sequence: str, release_dates: Mapping[str, datetime.datetime],
               release_date_cutoff: Optional[datetime.datetime], max_subsequence_ratio: float = 0.95, min_align_ratio: float = 0.1) -> bool:
    """Raises a ``PrefilterError`` subclass when the hit must not be used; returns True otherwise."""
    aligned_cols = hit.aligned_cols
    align_ratio = aligned_cols / len(query_sequence)
    template_sequence = hit.hit_sequence.replace("-", "")
    length_ratio = float(len(template_sequence)) / len(query_sequence)
    duplicate = template_sequence in query_sequence and length_ratio > max_subsequence_ratio
    if release_date_cutoff is not None and _is_after_cutoff(hit_pdb_code, release_dates, release_date_cutoff):
        raise DateError("Date (%s) > max template date (%s)." % (release_dates[hit_pdb_code], release_date_cutoff))
    if align_ratio <= min_align_ratio:
        raise AlignRatioError("Proportion of residues aligned to query too small. Align ratio: %s." % align_ratio)
    if duplicate:
        raise DuplicateError("Template is an exact subsequence of query with large coverage. Length ratio: %s." % length_ratio)
    if len(template_sequence) < 10:
        raise LengthError("Template too short. Length: %d." % len(template_sequence))
    return True


# ---------------------------------------------------------------------------
# locating the hit in the structure
# ---------------------------------------------------------------------------
def _find_template_in_pdb(template_chain_id: str, template_sequence: str, mmcif_object) -> Tuple[str, str, int]:
    """(sequence of the chain used, its id, offset of the template sequence inside it)."""
    chain_seq = mmcif_object.chain_to_seqres.get(template_chain_id)
    if chain_seq and template_sequence in chain_seq:
        return chain_seq, template_chain_id, chain_seq.find(template_sequence)
    for cid, seq in mmcif_object.chain_to_seqres.items():
        if seq and template_sequence in seq:
            return seq, cid, seq.find(template_sequence)
    # 'X' in the hit matches anything
    pattern = re.compile("".join("." if ch == "X" else "(?:%s|X)" % ch for ch in template_sequence))
    for cid, seq in mmcif_object.chain_to_seqres.items():
        m = pattern.search(seq)
        if m:
            return seq, cid, m.start()
    raise SequenceNotInTemplateError("Could not find the template sequence in %s_%s. Template sequence: %s, chain_to_seqres: %s" % (
        mmcif_object.file_id, template_chain_id, template_sequence, mmcif_object.chain_to_seqres))


def _realign_pdb_template_to_query(old_template_sequence: str, template_chain_id: str, mmcif_object, old_mapping: Mapping[int, int],
                                   kalign_binary_path: str) -> Tuple[str, Mapping[int, int]]:
    """The search database may hold an outdated sequence: align it against the chain's actual sequence (kalign) and
    translate the query -> template mapping through that alignment."""
    aligner = Kalign(binary_path=kalign_binary_path)
    new_seq = mmcif_object.chain_to_seqres.get(template_chain_id, "")
    if not new_seq:
        if len(mmcif_object.chain_to_seqres) == 1:
            template_chain_id, new_seq = next(iter(mmcif_object.chain_to_seqres.items()))
        else:
            raise QueryToTemplateAlignError("Could not find chain %s in %s." % (template_chain_id, mmcif_object.file_id))
    try:
        aligned, _, _ = parsers.parse_a3m(aligner.align([old_template_sequence, new_seq]))
        old_al, new_al = aligned
    except Exception as e:  # noqa: BLE001
        raise QueryToTemplateAlignError("Could not align old template %s to template %s (%s_%s). Error: %s" % (
            old_template_sequence, new_seq, mmcif_object.file_id, template_chain_id, e))
    old_to_new, io_, in_, same = {}, -1, -1, 0
    for a, b in zip(old_al, new_al):
        io_ += a != "-"
        in_ += b != "-"
        if a != "-" and b != "-":
            old_to_new[io_] = in_
            same += a == b
    if float(same) / min(len(old_template_sequence), len(new_seq)) < 0.9:
        raise QueryToTemplateAlignError("Insufficient similarity of the sequence in the database: %s to the actual sequence in the mmCIF "
                                        "file %s_%s: %s. We require at least 90 %% similarity wrt to the shorter of the sequences." % (
                                            old_template_sequence, mmcif_object.file_id, template_chain_id, new_seq))
    new_mapping = {q: old_to_new.get(t, -1) for q, t in old_mapping.items()}
    return new_seq.replace("-", ""), new_mapping


def _check_residue_distances(all_positions: np.ndarray, all_positions_mask: np.ndarray, max_ca_ca_distance: float):
    ca = rc.atom_order["CA"]
    prev, prev_known = None, False
    for i, (coords, mask) in enumerate(zip(all_positions, all_positions_mask)):
        known = bool(mask[ca])
        if known:
            if prev_known:
                d = np.linalg.norm(coords[ca] - prev)
                if d > max_ca_ca_distance:
                    raise CaDistanceError("The distance between residues %d and %d is %f > limit %f." % (i, i + 1, d, max_ca_ca_distance))
            prev = coords[ca]
        prev_known = known


def _get_atom_positions(mmcif_object, auth_chain_id: str, max_ca_ca_distance: float, _zero_center_positions: bool = True) -> Tuple[np.ndarray, np.ndarray]:
    if auth_chain_id not in mmcif_object.chain_to_seqres:
        raise NoChainsError("chain %s not in %s" % (auth_chain_id, mmcif_object.file_id))
    pos, mask = mmcif_parsing.get_atom_coords(mmcif_object, auth_chain_id, _zero_center_positions=_zero_center_positions)
    _check_residue_distances(pos, mask, max_ca_ca_distance)
    return pos, mask


def extract_template_features(mmcif_object, pdb_id: str, mapping: Mapping[int, int], template_sequence: str, query_sequence: str,
                              template_chain_id: str, kalign_binary_path: Optional[str], _zero_center_positions: bool = True) -> Tuple[Dict[str, Any], Optional[str]]:
    if mmcif_object is None or not mmcif_object.chain_to_seqres:
        raise NoChainsError("No chains in PDB: %s_%s" % (pdb_id, template_chain_id))
    warning = None
    try:
        seqres, chain_id, offset = _find_template_in_pdb(template_chain_id, template_sequence, mmcif_object)
    except SequenceNotInTemplateError:
        chain_id = template_chain_id
        warning = "The exact sequence %s was not found in %s_%s. Realigning the template to the actual sequence." % (
            template_sequence, pdb_id, chain_id)
        if not kalign_binary_path:
            raise
        seqres, mapping = _realign_pdb_template_to_query(template_sequence, template_chain_id, mmcif_object, mapping, kalign_binary_path)
        offset = 0
    try:
        all_pos, all_mask = _get_atom_positions(mmcif_object, chain_id, max_ca_ca_distance=150.0, _zero_center_positions=_zero_center_positions)
    except (CaDistanceError, KeyError) as e:
        raise NoAtomDataInTemplateError("Could not get atom data (%s_%s): %s" % (pdb_id, chain_id, e))
    n = len(query_sequence)
    out_pos = np.zeros((n, rc.atom_type_num, 3), np.float32)
    out_mask = np.zeros((n, rc.atom_type_num), np.float32)
    out_seq = ["-"] * n
    for q, t in mapping.items():
        if t == -1 or not (0 <= q < n):
            continue
        k = t + offset
        if 0 <= k < len(seqres):
            out_pos[q] = all_pos[k]
            out_mask[q] = all_mask[k]
            out_seq[q] = seqres[k]
    if out_mask.sum() < 5:
        raise TemplateAtomMaskAllZerosError("Template all atom mask was all zeros: %s_%s. Residue range: %d-%d" % (
            pdb_id, chain_id, min(mapping.values(), default=0) + offset, max(mapping.values(), default=0) + offset))
    out_seq = "".join(out_seq)
    aatype = rc.sequence_to_onehot(out_seq, rc.HHBLITS_AA_TO_ID)
    return ({"template_all_atom_positions": out_pos, "template_all_atom_mask": out_mask, "template_sequence": out_seq.encode(),
             "template_aatype": np.array(aatype), "template_domain_names": ("%s_%s" % (pdb_id.lower(), chain_id)).encode()}, warning)


# ---------------------------------------------------------------------------
# featurizers
# ---------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class SingleHitResult:
    features: Optional[Mapping[str, Any]]
    error: Optional[str]
    warning: Optional[str]


@dataclasses.dataclass(frozen=True)
class TemplateSearchResult:
    features: Mapping[str, Any]
    errors: Sequence[str]
    warnings: Sequence[str]


@dataclasses.dataclass(frozen=True)
class PrefilterResult:
    valid: bool
    error: Optional[str]
    warning: Optional[str]


class TemplateHitFeaturizer:
    """Turns HHSearch hits into template features (fastfold/data/templates.py:828-1063)."""

    def __init__(self, mmcif_dir: str, max_template_date: str, max_hits: int, kalign_binary_path: Optional[str] = None,
                 release_dates_path: Optional[str] = None, obsolete_pdbs_path: Optional[str] = None, strict_error_check: bool = False,
                 _shuffle_top_k_prefiltered: Optional[int] = None, _zero_center_positions: bool = True):
        self._mmcif_dir = mmcif_dir
        if not glob.glob(os.path.join(mmcif_dir, "*.cif")):
            raise ValueError("Could not find CIFs in %s" % mmcif_dir)
        try:
            self._max_template_date = datetime.datetime.strptime(max_template_date, "%Y-%m-%d")
        except ValueError:
            raise ValueError("max_template_date must be set and have format YYYY-MM-DD.")
        self.max_hits = max_hits
        self._kalign_binary_path = kalign_binary_path
        self._strict_error_check = strict_error_check
        self._release_dates = _parse_release_dates(release_dates_path) if release_dates_path else {}
        self._obsolete_pdbs = _parse_obsolete(obsolete_pdbs_path) if obsolete_pdbs_path else {}
        self._shuffle_top_k_prefiltered = _shuffle_top_k_prefiltered
        self._zero_center_positions = _zero_center_positions

    # -- one hit -------------------------------------------------------------
    def _prefilter(self, query_sequence, hit):
        pdb_id, _ = _hit_pdb_id_and_chain(hit)
        if pdb_id not in self._release_dates and pdb_id in self._obsolete_pdbs and self._obsolete_pdbs[pdb_id]:
            pdb_id = self._obsolete_pdbs[pdb_id]
        try:
            assess_hit(hit, pdb_id, query_sequence, self._release_dates, self._max_template_date)
        except PrefilterError as e:
            msg = "hit %s did not pass prefilter: %s" % (hit.name, e)
            if self._strict_error_check and isinstance(e, (DateError, DuplicateError)):
                return SingleHitResult(None, msg, None)
            return SingleHitResult(None, None, None)
        return None

    def _process_hit(self, query_sequence: str, hit: parsers.TemplateHit) -> SingleHitResult:
        pdb_id, chain_id = _hit_pdb_id_and_chain(hit)
        if pdb_id not in self._release_dates and pdb_id in self._obsolete_pdbs and self._obsolete_pdbs[pdb_id]:
            pdb_id = self._obsolete_pdbs[pdb_id]
        mapping = build_query_to_hit_index_mapping(hit.query, hit.hit_sequence, hit.indices_hit, hit.indices_query, query_sequence)
        template_sequence = hit.hit_sequence.replace("-", "")
        cif_path = os.path.join(self._mmcif_dir, pdb_id + ".cif")
        try:
            cif_string = open(cif_path).read()
        except OSError as e:
            return SingleHitResult(None, None, "could not read %s: %s" % (cif_path, e))
        parsed = mmcif_parsing.parse(file_id=pdb_id, mmcif_string=cif_string)
        if parsed.mmcif_object is not None and "release_date" in parsed.mmcif_object.header:
            date = datetime.datetime.strptime(parsed.mmcif_object.header["release_date"], "%Y-%m-%d")
            if date > self._max_template_date:
                msg = "Template %s date (%s) > max template date (%s)." % (pdb_id, date, self._max_template_date)
                return SingleHitResult(None, msg if self._strict_error_check else None, None)
        try:
            feats, warning = extract_template_features(parsed.mmcif_object, pdb_id, mapping, template_sequence, query_sequence, chain_id,
                                                       self._kalign_binary_path, _zero_center_positions=self._zero_center_positions)
            feats["template_sum_probs"] = [hit.sum_probs if hit.sum_probs is not None else 0.0]
            return SingleHitResult(feats, None, warning)
        except (NoChainsError, NoAtomDataInTemplateError, TemplateAtomMaskAllZerosError) as e:
            msg = "%s_%s (sum_probs: %s, rank: %s): feature extracting errors: %s, mmCIF parsing errors: %s" % (
                pdb_id, chain_id, hit.sum_probs, hit.index, e, parsed.errors)
            return SingleHitResult(None, msg if self._strict_error_check else None, None if self._strict_error_check else msg)
        except Error as e:
            return SingleHitResult(None, "%s_%s (sum_probs: %s, rank: %s): feature extracting errors: %s" % (
                pdb_id, chain_id, hit.sum_probs, hit.index, e), None)

    # -- all hits ------------------------------------------------------------
    def get_templates(self, query_sequence: str, query_release_date: Optional[datetime.datetime] = None,
                      hits: Optional[Sequence[parsers.TemplateHit]] = None, query_pdb_code: Optional[str] = None) -> TemplateSearchResult:
        """Argument order of fastfold/data/templates.py:995-1001; ``get_templates(query_sequence, hits)`` (the order of the
        hmmsearch featurizer, :1110-1114) is understood too.  ``query_pdb_code`` / ``query_release_date`` (training on PDB
        entries): the query's own entry is never its template, and the date cutoff moves to 60 days before the query's
        release when that is earlier than ``max_template_date`` (:1003-1063)."""
        if hits is None and isinstance(query_release_date, (list, tuple)):
            hits, query_release_date = query_release_date, None
        if hits is None:
            raise TypeError("get_templates() needs the template hits")
        log.info("Searching for template for: %s", query_sequence)
        collected = {k: [] for k in TEMPLATE_FEATURES}
        errors, warnings = [], []
        candidates = []
        saved_cutoff = self._max_template_date
        if query_release_date is not None:
            if isinstance(query_release_date, str):
                query_release_date = datetime.datetime.strptime(query_release_date, "%Y-%m-%d")
            self._max_template_date = min(saved_cutoff, query_release_date - datetime.timedelta(days=60))
        try:
            return self._get_templates(query_sequence, hits, query_pdb_code, collected, errors, warnings, candidates)
        finally:
            self._max_template_date = saved_cutoff

    def _get_templates(self, query_sequence, hits, query_pdb_code, collected, errors, warnings, candidates):
        for hit in sorted(hits, key=lambda h: h.sum_probs if h.sum_probs is not None else 0.0, reverse=True):
            if query_pdb_code is not None and _hit_pdb_id_and_chain(hit)[0].lower() == query_pdb_code.lower():
                continue
            rejected = self._prefilter(query_sequence, hit)
            if rejected is None:
                candidates.append(hit)
            elif rejected.error:
                errors.append(rejected.error)
        if self._shuffle_top_k_prefiltered:
            k = self._shuffle_top_k_prefiltered
            head = candidates[:k]
            np.random.shuffle(head)
            candidates[:k] = head
        accepted = 0
        for hit in candidates:
            if accepted >= self.max_hits:
                break
            res = self._process_hit(query_sequence, hit)
            if res.error:
                errors.append(res.error)
            if res.warning:
                warnings.append(res.warning)
            if res.features is None:
                continue
            accepted += 1
            for k in collected:
                collected[k].append(res.features[k])
        n = len(query_sequence)
        if accepted:
            feats = {k: np.stack(collected[k], axis=0).astype(TEMPLATE_FEATURES[k]) for k in collected}
        else:
            feats = {"template_aatype": np.zeros((0, n, 22), np.int64), "template_all_atom_mask": np.zeros((0, n, rc.atom_type_num), np.float32),
                     "template_all_atom_positions": np.zeros((0, n, rc.atom_type_num, 3), np.float32),
                     "template_domain_names": np.zeros((0,), object), "template_sequence": np.zeros((0,), object),
                     "template_sum_probs": np.zeros((0, 1), np.float32)}
        return TemplateSearchResult(features=feats, errors=errors, warnings=warnings)


HhsearchHitFeaturizer = TemplateHitFeaturizer


class HmmsearchHitFeaturizer(TemplateHitFeaturizer):
    """Hits of the multimer pipeline's hmmsearch against PDB seqres (fastfold/data/templates.py:1066-1221): same
    processing; hits carry no ``sum_probs`` and keep their search order, and near-duplicates of the query are allowed
    (a chain of a complex is often its own best template)."""

    def _prefilter(self, query_sequence, hit):
        pdb_id, _ = _hit_pdb_id_and_chain(hit)
        try:
            assess_hit(hit, pdb_id, query_sequence, self._release_dates, self._max_template_date, max_subsequence_ratio=2.0)
        except PrefilterError as e:
            if self._strict_error_check and isinstance(e, DateError):
                return SingleHitResult(None, "hit %s did not pass prefilter: %s" % (hit.name, e), None)
            return SingleHitResult(None, None, None)
        return None

    def get_templates(self, query_sequence, hits, query_pdb_code=None, query_release_date=None):
        ordered = [dataclasses.replace(h, sum_probs=float(len(hits) - i)) if h.sum_probs is None else h for i, h in enumerate(hits)]
        res = super().get_templates(query_sequence, query_release_date=query_release_date, hits=ordered, query_pdb_code=query_pdb_code)
        feats = dict(res.features)
        feats["template_sum_probs"] = np.zeros_like(feats["template_sum_probs"])
        return TemplateSearchResult(features=feats, errors=res.errors, warnings=res.warnings)
