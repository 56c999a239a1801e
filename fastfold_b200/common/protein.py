"""Protein structure container and PDB text I/O (no BioPython).

``Protein`` holds atom37 coordinates / masks, residue types and indices, B-factors and chain indices;
``from_prediction`` builds one from model features + outputs, ``to_pdb`` writes PDB text, ``from_pdb_string`` reads the
ATOM records of one model back.  Same role as fastfold/common/protein.py:213-359.
"""
import dataclasses
import string
from typing import Optional

import numpy as np

from . import residue_constants as rc

PDB_CHAIN_IDS = string.ascii_uppercase + string.ascii_lowercase + string.digits
PDB_MAX_CHAINS = len(PDB_CHAIN_IDS)


@dataclasses.dataclass(frozen=True)
class Protein:
    atom_positions: np.ndarray      # [num_res, 37, 3], angstroms
    aatype: np.ndarray              # [num_res]
    atom_mask: np.ndarray           # [num_res, 37]
    residue_index: np.ndarray       # [num_res], as in the PDB
    b_factors: np.ndarray           # [num_res, 37]
    chain_index: Optional[np.ndarray] = None


def from_prediction(features, result, b_factors=None, remove_leading_feature_dimension=False):
    def fix(x):
        x = np.asarray(x)
        return x[0] if remove_leading_feature_dimension else x
    n = np.asarray(result["final_atom_mask"]).shape[0]
    chain = fix(features["asym_id"]) - 1 if "asym_id" in features else np.zeros(n, dtype=np.int64)
    if b_factors is None:
        b_factors = np.zeros_like(np.asarray(result["final_atom_mask"]))
    return Protein(aatype=fix(features["aatype"]), atom_positions=np.asarray(result["final_atom_positions"]),
                   atom_mask=np.asarray(result["final_atom_mask"]), residue_index=fix(features["residue_index"]) + 1,
                   b_factors=np.asarray(b_factors), chain_index=np.asarray(chain))


def _chain_end(atom_index, end_resname, chain_name, residue_index):
    return "%-6s%5d      %3s %1s%4d" % ("TER", atom_index, end_resname, chain_name, residue_index)


def to_pdb(prot: Protein) -> str:
    restypes = rc.restypes + ["X"]
    res_1to3 = lambda r: rc.restype_1to3.get(restypes[r], "UNK")
    atom_types = rc.atom_types
    lines = []
    aatype = prot.aatype.astype(np.int64)
    pos, mask = prot.atom_positions, prot.atom_mask
    ridx = prot.residue_index.astype(np.int64)
    chain_index = prot.chain_index.astype(np.int64) if prot.chain_index is not None else np.zeros_like(aatype)
    if np.any(aatype > rc.restype_num):
        raise ValueError("Invalid aatypes.")
    if np.any(chain_index >= PDB_MAX_CHAINS):
        raise ValueError("The PDB format supports at most %d chains." % PDB_MAX_CHAINS)
    lines.append("MODEL     1")
    atom_index = 1
    last_chain = chain_index[0]
    for i in range(aatype.shape[0]):
        if last_chain != chain_index[i]:
            lines.append(_chain_end(atom_index, res_1to3(aatype[i - 1]), PDB_CHAIN_IDS[chain_index[i - 1]], ridx[i - 1]))
            last_chain = chain_index[i]
            atom_index += 1
        rname = res_1to3(aatype[i])
        for name, p, m, b in zip(atom_types, pos[i], mask[i], prot.b_factors[i]):
            if m < 0.5:
                continue
            nm = name if len(name) == 4 else " " + name
            lines.append("%-6s%5d %-4s%1s%3s %1s%4d%1s   %8.3f%8.3f%8.3f%6.2f%6.2f          %2s%2s" % (
                "ATOM", atom_index, nm, "", rname, PDB_CHAIN_IDS[chain_index[i]], ridx[i], "", p[0], p[1], p[2], 1.00, b, name[0], ""))
            atom_index += 1
    lines.append(_chain_end(atom_index, res_1to3(aatype[-1]), PDB_CHAIN_IDS[chain_index[-1]], ridx[-1]))
    lines.append("ENDMDL")
    lines.append("END")
    return "\n".join(l.ljust(80) for l in lines) + "\n"


def from_pdb_string(pdb_str: str, chain_id: Optional[str] = None) -> Protein:
    rows = {}
    order = []
    chains = []
    for line in pdb_str.splitlines():
        if line.startswith("ENDMDL"):
            break
        if not line.startswith("ATOM"):
            continue
        ch = line[21]
        if chain_id is not None and ch != chain_id:
            continue
        name, resname, rnum = line[12:16].strip(), line[17:20], int(line[22:26])
        key = (ch, rnum, line[26])
        if key not in rows:
            rows[key] = (resname, np.zeros((37, 3)), np.zeros(37), np.zeros(37))
            order.append(key)
            if ch not in chains:
                chains.append(ch)
        if name in rc.atom_order:
            _, p, m, b = rows[key]
            j = rc.atom_order[name]
            p[j] = [float(line[30:38]), float(line[38:46]), float(line[46:54])]
            m[j] = 1.0
            b[j] = float(line[60:66])
    aatype = np.array([rc.restype_order.get(rc.restype_3to1.get(rows[k][0], "X"), rc.restype_num) for k in order])
    return Protein(atom_positions=np.stack([rows[k][1] for k in order]), atom_mask=np.stack([rows[k][2] for k in order]), aatype=aatype,
                   residue_index=np.array([k[1] for k in order]), b_factors=np.stack([rows[k][3] for k in order]),
                   chain_index=np.array([chains.index(k[0]) for k in order]))


def ideal_atom_mask(prot: Protein) -> np.ndarray:
    return rc.STANDARD_ATOM_MASK[prot.aatype]


PICO_TO_ANGSTROM = 0.01


def from_proteinnet_string(proteinnet_str: str) -> Protein:
    """One ProteinNet text record (``[PRIMARY]`` sequence, ``[TERTIARY]`` three rows x / y / z of N, CA, C coordinates in
    picometres, ``[MASK]`` of ``+`` / ``-`` per residue) as a backbone-only ``Protein`` in angstroms."""
    import re
    fields, key = {}, None
    for line in proteinnet_str.splitlines():
        m = re.fullmatch(r"\[([A-Z]+)\]", line.strip())
        if m:
            key = m.group(1)
            fields[key] = []
        elif key is not None and line.strip():
            fields[key].append(line.strip())
    seq = "".join(fields["PRIMARY"])
    aatype = np.array([rc.restype_order.get(ch, rc.restype_num) for ch in seq], dtype=np.int64)
    n = len(seq)
    backbone = [rc.atom_order[a] for a in ("N", "CA", "C")]
    positions = np.zeros((n, rc.atom_type_num, 3), dtype=np.float32)
    if "TERTIARY" in fields:
        xyz = np.array([[float(v) for v in row.split()] for row in fields["TERTIARY"][:3]], dtype=np.float32)     # [3, 3 n]
        for i, slot in enumerate(backbone):
            positions[:, slot, :] = xyz[:, i::3].T * PICO_TO_ANGSTROM
    present = np.ones(n, dtype=np.float32)
    if "MASK" in fields:
        present = np.array([1.0 if ch == "+" else 0.0 for ch in "".join(fields["MASK"])], dtype=np.float32)
    mask = np.zeros((n, rc.atom_type_num), dtype=np.float32)
    mask[:, backbone] = present[:, None]
    return Protein(atom_positions=positions, atom_mask=mask, aatype=aatype, residue_index=np.arange(n), b_factors=np.zeros_like(mask))

