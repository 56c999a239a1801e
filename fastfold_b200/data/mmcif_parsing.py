"""A dependency-free mmCIF reader for template featurisation.

The reference parses mmCIF files with BioPython (fastfold/data/mmcif_parsing.py:1-485); BioPython is not required
here.  The reader tokenises the file itself (data names, ``loop_`` tables, quoted and ``;``-delimited values) and
builds the same information the template pipeline consumes:

* ``header``: structure method, release date (earliest revision), resolution
* ``chain_to_seqres``: author chain id -> one-letter SEQRES sequence (from ``_entity_poly_seq`` / ``_struct_asym``)
* ``seqres_to_structure``: per chain, SEQRES index -> ``ResidueAtPosition`` (author numbering, hetero flag, missing?)
* ``atoms``: per chain, (residue number, insertion code) -> {atom name: (x, y, z)} of the first model
"""
import collections
import dataclasses
import io
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

from ..common import residue_constants as rc

# Parent amino acid of the modified residues that occur most often in the sequence records of PDB entries (selenomethionine
# above all: crystallographers' stand-in for methionine).  The reference looks names up in BioPython's much longer SCOP table
# (fastfold/data/mmcif_parsing.py:284); a name in neither table is read as X.
MODIFIED_RESIDUE_LETTERS = {
    "MSE": "M", "SEC": "U", "PYL": "O", "SEP": "S", "TPO": "T", "PTR": "Y", "HYP": "P", "MLY": "K", "CSO": "C", "CME": "C", "OCS": "C",
    "CSD": "C", "KCX": "K", "LLP": "K", "M3L": "K", "MLZ": "K", "ALY": "K", "PCA": "E", "CGU": "E", "FME": "M", "MHO": "M", "NLE": "L",
    "ABA": "A", "AIB": "A", "DAL": "A", "HIC": "H", "NEP": "H", "TYS": "Y", "TRO": "W", "DPR": "P", "SAC": "S", "BMT": "T", "UNK": "X",
}


ChainId = str
PdbHeader = Mapping[str, Any]


@dataclasses.dataclass(frozen=True)
class ResiduePosition:
    chain_id: str
    residue_number: int
    insertion_code: str


@dataclasses.dataclass(frozen=True)
class ResidueAtPosition:
    position: Optional[ResiduePosition]
    name: str
    is_missing: bool
    hetflag: str


@dataclasses.dataclass(frozen=True)
class Monomer:
    """One residue of an entity's polymer sequence (``_entity_poly_seq``): its three-letter id and its position."""
    id: str
    num: int


@dataclasses.dataclass(frozen=True)
class AtomSite:
    """The columns of one ``_atom_site`` row that link an atom to its residue and chain."""
    residue_name: str
    author_chain_id: str
    mmcif_chain_id: str
    author_seq_num: str
    mmcif_seq_num: int
    insertion_code: str
    hetatm_atom: str
    model_num: int


@dataclasses.dataclass(frozen=True)
class MmcifObject:
    file_id: str
    header: PdbHeader
    atoms: Mapping[ChainId, Mapping[Tuple[int, str], Mapping[str, Tuple[float, float, float]]]]
    chain_to_seqres: Mapping[ChainId, str]
    seqres_to_structure: Mapping[ChainId, Mapping[int, ResidueAtPosition]]
    raw_string: Any

    # the reference exposes a BioPython ``structure``; callers here use ``atoms`` instead
    @property
    def structure(self):
        return self.atoms


@dataclasses.dataclass(frozen=True)
class ParsingResult:
    mmcif_object: Optional[MmcifObject]
    errors: Mapping[Tuple[str, str], Any]


class ParseError(Exception):
    pass


# ---------------------------------------------------------------------------
# tokeniser
# ---------------------------------------------------------------------------
def _tokens(text: str):
    """Yields the whitespace-separated values of a CIF file, honouring quotes, ``;`` text fields and comments."""
    lines = text.splitlines()
    i = 0
    while i < len(lines):
        line = lines[i]
        if line.startswith(";"):
            buf = [line[1:]]
            i += 1
            while i < len(lines) and not lines[i].startswith(";"):
                buf.append(lines[i])
                i += 1
            yield "\n".join(buf).strip(), True
            i += 1
            continue
        pos, n = 0, len(line)
        while pos < n:
            ch = line[pos]
            if ch in " \t":
                pos += 1
            elif ch == "#":
                break
            elif ch in "'\"":
                end = pos + 1
                while True:
                    end = line.find(ch, end)
                    if end == -1:
                        end = n
                        break
                    if end + 1 >= n or line[end + 1] in " \t":
                        break
                    end += 1
                yield line[pos + 1:end], True
                pos = end + 1
            else:
                end = pos
                while end < n and line[end] not in " \t":
                    end += 1
                yield line[pos:end], False
                pos = end
        i += 1


def parse_cif_dict(text: str) -> Dict[str, List[str]]:
    """``{data name: [values]}``: single items become one-element lists, loop columns keep one value per row."""
    out: Dict[str, List[str]] = collections.OrderedDict()
    toks = list(_tokens(text))
    i, n = 0, len(toks)
    while i < n:
        tok, quoted = toks[i]
        low = tok.lower()
        if not quoted and low.startswith("data_"):
            out.setdefault("data_", []).append(tok[5:])
            i += 1
        elif not quoted and low == "loop_":
            i += 1
            names = []
            while i < n and not toks[i][1] and toks[i][0].startswith("_"):
                names.append(toks[i][0])
                i += 1
            cols = [[] for _ in names]
            k = 0
            while i < n:
                t, q = toks[i]
                if not q and (t.startswith("_") or t.lower() == "loop_" or t.lower().startswith("data_")):
                    break
                cols[k % len(names)].append(t)
                k += 1
                i += 1
            if names and k % len(names):
                raise ParseError("loop with %d columns holds %d values" % (len(names), k))
            for name, col in zip(names, cols):
                out[name] = col
        elif not quoted and tok.startswith("_"):
            if i + 1 >= n:
                raise ParseError("data name %s without a value" % tok)
            out[tok] = [toks[i + 1][0]]
            i += 2
        else:
            i += 1
    return out


def mmcif_loop_to_list(prefix: str, parsed: Mapping[str, Sequence[str]]) -> List[Dict[str, str]]:
    cols = [(k, v) for k, v in parsed.items() if k.startswith(prefix)]
    if not cols:
        return []
    n = len(cols[0][1])
    if any(len(v) != n for _, v in cols):
        raise ParseError("mmCIF error: not all loops of %s are the same length" % prefix)
    return [{k: v[i] for k, v in cols} for i in range(n)]


def mmcif_loop_to_dict(prefix: str, index: str, parsed: Mapping[str, Sequence[str]]) -> Dict[str, Dict[str, str]]:
    return {row[index]: row for row in mmcif_loop_to_list(prefix, parsed)}


# ---------------------------------------------------------------------------
# header
# ---------------------------------------------------------------------------
def get_release_date(parsed: Mapping[str, Sequence[str]]) -> str:
    dates = parsed.get("_pdbx_audit_revision_history.revision_date")
    if not dates:
        raise ParseError("no release date")
    return min(dates)


def _get_header(parsed) -> PdbHeader:
    header = {}
    methods = mmcif_loop_to_list("_exptl.", parsed)
    header["structure_method"] = ",".join(m.get("_exptl.method", "").lower() for m in methods)
    if "_pdbx_audit_revision_history.revision_date" in parsed:
        header["release_date"] = get_release_date(parsed)
    header["resolution"] = 0.00
    for key in ("_refine.ls_d_res_high", "_em_3d_reconstruction.resolution", "_reflns.d_resolution_high"):
        if key in parsed:
            try:
                header["resolution"] = float(parsed[key][0])
                break
            except ValueError:
                pass
    return header


# ---------------------------------------------------------------------------
# main entry
# ---------------------------------------------------------------------------
def _is_set(v: str) -> bool:
    return v not in (".", "?")


def parse(*, file_id: str, mmcif_string: str, catch_all_errors: bool = True) -> ParsingResult:
    """Parses one mmCIF file.  Errors are returned, not raised, unless ``catch_all_errors`` is False."""
    errors = {}
    try:
        parsed = parse_cif_dict(mmcif_string)
        header = _get_header(parsed)

        # polymer entities and the chains that instantiate them
        entity_seq: Dict[str, List[Tuple[int, str, str]]] = collections.defaultdict(list)
        for row in mmcif_loop_to_list("_entity_poly_seq.", parsed):
            entity_seq[row["_entity_poly_seq.entity_id"]].append((int(row["_entity_poly_seq.num"]), row["_entity_poly_seq.mon_id"],
                                                                  row.get("_entity_poly_seq.hetero", "n")))
        chem = mmcif_loop_to_dict("_chem_comp.", "_chem_comp.id", parsed)
        chain_entity = {row["_struct_asym.id"]: row["_struct_asym.entity_id"] for row in mmcif_loop_to_list("_struct_asym.", parsed)}
        protein_chains = {}
        for chain, ent in chain_entity.items():
            seq = entity_seq.get(ent)
            if seq and any("peptide" in chem.get(mon, {}).get("_chem_comp.type", "peptide").lower() for _, mon, _ in seq):
                protein_chains[chain] = seq
        if not protein_chains:
            return ParsingResult(None, {(file_id, ""): "No protein chains found in this file."})

        # atoms of the first model
        atom_rows = mmcif_loop_to_list("_atom_site.", parsed)
        first_model = atom_rows[0].get("_atom_site.pdbx_PDB_model_num", "1") if atom_rows else "1"
        mmcif_to_author: Dict[str, str] = {}
        seq_to_pos: Dict[str, Dict[int, ResidueAtPosition]] = collections.defaultdict(dict)
        atoms: Dict[str, Dict[Tuple[int, str], Dict[str, Tuple[float, float, float]]]] = collections.defaultdict(dict)
        seq_start: Dict[str, int] = {}
        for row in atom_rows:
            if row.get("_atom_site.pdbx_PDB_model_num", first_model) != first_model:
                continue
            mm_chain = row["_atom_site.label_asym_id"]
            auth_chain = row.get("_atom_site.auth_asym_id", mm_chain)
            mmcif_to_author[mm_chain] = auth_chain
            if mm_chain not in protein_chains:
                continue
            alt = row.get("_atom_site.label_alt_id", ".")
            ins = row.get("_atom_site.pdbx_PDB_ins_code", "?")
            ins = ins if _is_set(ins) else " "
            resnum = int(row["_atom_site.auth_seq_id"])
            name = row["_atom_site.label_atom_id"]
            key = (resnum, ins)
            res_atoms = atoms[auth_chain].setdefault(key, {})
            if name not in res_atoms or not _is_set(alt) or alt == "A":
                res_atoms[name] = (float(row["_atom_site.Cartn_x"]), float(row["_atom_site.Cartn_y"]), float(row["_atom_site.Cartn_z"]))
            group = row.get("_atom_site.group_PDB", "ATOM")
            het = " "
            if group == "HETATM":
                het = "W" if row["_atom_site.label_comp_id"] in ("HOH", "WAT") else "H_" + row["_atom_site.label_comp_id"]
            seq_id = int(row["_atom_site.label_seq_id"]) if _is_set(row.get("_atom_site.label_seq_id", ".")) else None
            if seq_id is None:
                continue
            start = seq_start.setdefault(mm_chain, min(n for n, _, _ in protein_chains[mm_chain]))
            seq_to_pos[mm_chain][seq_id - start] = ResidueAtPosition(ResiduePosition(auth_chain, resnum, ins), row["_atom_site.label_comp_id"],
                                                                     False, het)
        # residues of SEQRES without coordinates are marked missing
        for chain, seq in protein_chains.items():
            cur = seq_to_pos[chain]
            seen = set()
            idx = -1
            for num, mon, _ in seq:
                if num in seen:          # micro-heterogeneity: keep the first monomer of a position
                    continue
                seen.add(num)
                idx += 1
                if idx not in cur:
                    cur[idx] = ResidueAtPosition(None, mon, True, " ")

        chain_to_seqres, author_seq_to_structure = {}, {}
        for chain, seq in protein_chains.items():
            author = mmcif_to_author.get(chain)
            if author is None:
                continue
            letters, seen = [], set()
            for num, mon, _ in seq:
                if num in seen:
                    continue
                seen.add(num)
                code = rc.restype_3to1.get(mon) or MODIFIED_RESIDUE_LETTERS.get(mon, "X")
                letters.append(code if len(code) == 1 else "X")
            chain_to_seqres[author] = "".join(letters)
            author_seq_to_structure[author] = seq_to_pos[chain]
        obj = MmcifObject(file_id=file_id, header=header, atoms={c: dict(v) for c, v in atoms.items()}, chain_to_seqres=chain_to_seqres,
                          seqres_to_structure=author_seq_to_structure, raw_string=parsed)
        return ParsingResult(obj, errors)
    except Exception as e:      # noqa: BLE001 - a malformed file must not stop a template search
        errors[(file_id, "")] = e
        if not catch_all_errors:
            raise
        return ParsingResult(None, errors)


def get_atom_coords(mmcif_object: MmcifObject, chain_id: str, _zero_center_positions: bool = True):
    """All-atom positions (atom37 order) and mask of one chain, indexed by SEQRES position; by default translated so that
    the resolved atoms have zero mean (fastfold/data/mmcif_parsing.py:432-485)."""
    import numpy as np
    seq_map = mmcif_object.seqres_to_structure[chain_id]
    chain_atoms = mmcif_object.atoms.get(chain_id, {})
    n = len(mmcif_object.chain_to_seqres[chain_id])
    pos = np.zeros([n, rc.atom_type_num, 3], dtype=np.float32)
    mask = np.zeros([n, rc.atom_type_num], dtype=np.float32)
    for i in range(n):
        r = seq_map.get(i)
        if r is None or r.is_missing:
            continue
        res = chain_atoms.get((r.position.residue_number, r.position.insertion_code), {})
        for name, xyz in res.items():
            if name in rc.atom_order:
                pos[i, rc.atom_order[name]] = xyz
                mask[i, rc.atom_order[name]] = 1.0
            elif name.upper() == "SE" and r.name == "MSE":      # selenomethionine: SE stands in for SD
                pos[i, rc.atom_order["SD"]] = xyz
                mask[i, rc.atom_order["SD"]] = 1.0
        # arginine: NH1 is the nitrogen closer to CD; swap if the file names them the other way round
        if r.name == "ARG" and all(a in res for a in ("CD", "NH1", "NH2")):
            cd, nh1, nh2 = (np.asarray(res[a]) for a in ("CD", "NH1", "NH2"))
            if np.linalg.norm(nh1 - cd) > np.linalg.norm(nh2 - cd):
                i1, i2 = rc.atom_order["NH1"], rc.atom_order["NH2"]
                pos[i, [i1, i2]] = pos[i, [i2, i1]]
                mask[i, [i1, i2]] = mask[i, [i2, i1]]
    if _zero_center_positions and mask.any():
        present = mask.astype(bool)
        pos[present] -= pos[present].mean(axis=0)
    return pos, mask
