"""A small but fussy synthetic mmCIF entry for the reader, template and training-data tests."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def cif_text(pdb_id, date, chains, resolution="1.80"):
    """A small but fussy mmCIF file.  ``chains``: ``{label chain: (author chain, sequence)}``; residue 4 of every chain has
    no coordinates, residue 2 is selenomethionine written as HETATM when the sequence has M there, author numbering starts
    at 11 with an insertion code on residue 6, waters follow, and a second model repeats the first atom."""
    from fastfold_b200.common import residue_constants as rc
    three = {c: [rc.restype_1to3[a] if a != "M" else "MSE" for a in seq] for c, (_, seq) in chains.items()}
    comps = sorted({t for v in three.values() for t in v} | {"HOH"})
    lines = ["data_%s" % pdb_id.upper(), "#", "_entry.id %s" % pdb_id.upper(), "_exptl.method 'X-RAY DIFFRACTION'", "_refine.ls_d_res_high %s" % resolution,
             "#", "loop_", "_pdbx_audit_revision_history.ordinal", "_pdbx_audit_revision_history.revision_date", "1 %s" % date, "2 2031-07-13", "#",
             "loop_", "_struct_asym.id", "_struct_asym.entity_id"] + ["%s %d" % (c, i + 1) for i, c in enumerate(chains)] + ["W %d" % (len(chains) + 1), "#",
             "loop_", "_chem_comp.id", "_chem_comp.type", "_chem_comp.name"]
    lines += ["%s %s '%s'" % (t, "non-polymer" if t == "HOH" else "'L-peptide linking'", "water" if t == "HOH" else "amino acid; %s" % t.lower()) for t in comps]
    lines += ["#", "loop_", "_entity_poly_seq.entity_id", "_entity_poly_seq.num", "_entity_poly_seq.mon_id", "_entity_poly_seq.hetero"]
    for e, c in enumerate(chains):
        lines += ["%d %d %s n" % (e + 1, i + 1, t) for i, t in enumerate(three[c])]
    lines += ["#", "loop_"] + ["_atom_site." + k for k in ("group_PDB", "id", "type_symbol", "label_atom_id", "label_alt_id", "label_comp_id",
                                                         "label_asym_id", "label_entity_id", "label_seq_id", "pdbx_PDB_ins_code", "Cartn_x",
                                                         "Cartn_y", "Cartn_z", "occupancy", "B_iso_or_equiv", "auth_seq_id", "auth_asym_id",
                                                         "pdbx_PDB_model_num")]
    k = 1
    for e, (c, (author, seq)) in enumerate(chains.items()):
        for i, t in enumerate(three[c]):
            if i == 3:
                continue
            atoms = ["N", "CA", "C", "O"] + (["CB"] if t != "GLY" else []) + (["SE"] if t == "MSE" else []) + (["CD", "NH1", "NH2"] if t == "ARG" else [])
            number, icode = (i + 11, "?") if i < 6 else (i + 10, "A") if i == 6 else (i + 10, "?")
            for a, name in enumerate(atoms):
                x, y, z = 3.8 * i + 0.37 * a + 40.0 * e, 1.0 + 1.1 * a - 0.01 * i * a, -2.0 + 0.5 * a + 7.0 * e
                lines.append("%s %d %s %s . %s %s %d %d %s %.3f %.3f %.3f 1.00 20.00 %d %s 1" % (
                    "HETATM" if t == "MSE" else "ATOM", k, name[0], name, t, c, e + 1, i + 1, icode, x, y, z, number, author))
                k += 1
    lines.append("HETATM %d O O . HOH W %d . ? 1.000 2.000 3.000 1.00 30.00 201 %s 1" % (k, len(chains) + 1, list(chains.values())[0][0]))
    lines.append("ATOM %d N N . %s %s 1 1 ? 9.000 9.000 9.000 1.00 20.00 11 %s 2" % (k + 1, list(three.values())[0][0], list(chains)[0], list(chains.values())[0][0]))
    return "\n".join(lines) + "\n#\n"
