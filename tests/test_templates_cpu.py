"""mmCIF reader and template featuriser on a synthetic structure file."""
import os

import numpy as np
import pytest

from fastfold_b200.common import residue_constants as rc
from fastfold_b200.data import mmcif_parsing, parsers, templates

SEQ = "ACDEFGHIKLMNPQ"


def _cif(seq=SEQ, pdb_id="1abc", date="1999-05-01", chain="A"):
    three = [rc.restype_1to3[c] for c in seq]
    lines = ["data_%s" % pdb_id.upper(), "#", "_exptl.method 'X-RAY DIFFRACTION'", "_refine.ls_d_res_high 1.80", "#",
             "loop_", "_pdbx_audit_revision_history.ordinal", "_pdbx_audit_revision_history.revision_date", "1 %s" % date, "2 2031-07-13", "#",
             "loop_", "_struct_asym.id", "_struct_asym.entity_id", "%s 1" % chain, "#",
             "loop_", "_chem_comp.id", "_chem_comp.type"] + ["%s 'L-peptide linking'" % t for t in sorted(set(three))] + ["#",
             "loop_", "_entity_poly_seq.entity_id", "_entity_poly_seq.num", "_entity_poly_seq.mon_id", "_entity_poly_seq.hetero"]
    lines += ["1 %d %s n" % (i + 1, t) for i, t in enumerate(three)]
    lines += ["#", "loop_"] + ["_atom_site." + k for k in ("group_PDB", "id", "type_symbol", "label_atom_id", "label_alt_id", "label_comp_id",
                                                         "label_asym_id", "label_entity_id", "label_seq_id", "pdbx_PDB_ins_code", "Cartn_x",
                                                         "Cartn_y", "Cartn_z", "occupancy", "B_iso_or_equiv", "auth_seq_id", "auth_asym_id",
                                                         "pdbx_PDB_model_num")]
    k = 1
    for i, t in enumerate(three):
        if i == 3:
            continue                                   # one residue without coordinates
        for a, name in enumerate(("N", "CA", "C", "O")):
            x, y, z = 3.8 * i + 0.1 * a, 1.0 + a, -2.0 + 0.5 * a
            lines.append("ATOM %d %s %s . %s %s 1 %d ? %.3f %.3f %.3f 1.00 20.00 %d %s 1" % (k, name[0], name, t, chain, i + 1, x, y, z, i + 11, chain))
            k += 1
    return "\n".join(lines) + "\n#\n"


def test_mmcif_reader():
    res = mmcif_parsing.parse(file_id="1abc", mmcif_string=_cif())
    assert not res.errors, res.errors
    obj = res.mmcif_object
    assert obj.chain_to_seqres == {"A": SEQ}
    assert obj.header["release_date"] == "1999-05-01" and abs(obj.header["resolution"] - 1.8) < 1e-6
    assert obj.seqres_to_structure["A"][3].is_missing and not obj.seqres_to_structure["A"][4].is_missing
    assert obj.seqres_to_structure["A"][0].position.residue_number == 11
    pos, mask = mmcif_parsing.get_atom_coords(obj, "A", _zero_center_positions=False)
    centred, _ = mmcif_parsing.get_atom_coords(obj, "A")               # default: resolved atoms translated to zero mean
    assert np.abs(centred[mask.astype(bool)].mean(axis=0)).max() < 1e-4
    assert np.allclose((centred - pos)[mask.astype(bool)], (centred - pos)[mask.astype(bool)][0], atol=1e-4)
    assert pos.shape == (len(SEQ), 37, 3) and mask[3].sum() == 0 and mask[0, rc.atom_order["CA"]] == 1
    assert np.allclose(pos[2, rc.atom_order["CA"]], [3.8 * 2 + 0.1, 2.0, -1.5], atol=1e-3)


def test_quoted_and_multiline_values():
    d = mmcif_parsing.parse_cif_dict("data_x\n_a.b 'it''s fine'\n_a.c\n;line one\nline two\n;\nloop_\n_l.x\n_l.y\n1 \"two words\"\n3 4\n")
    assert d["_a.c"] == ["line one\nline two"] and d["_l.y"] == ["two words", "4"] and d["_l.x"] == ["1", "3"]


def test_template_featurizer(tmp_path):
    (tmp_path / "1abc.cif").write_text(_cif())
    (tmp_path / "2xyz.cif").write_text(_cif(pdb_id="2xyz", date="2030-01-01"))
    query = "MM" + SEQ + "WW"
    hit = parsers.TemplateHit(index=1, name="1abc_A some protein", aligned_cols=len(SEQ), sum_probs=12.0, query=SEQ, hit_sequence=SEQ,
                              indices_query=list(range(2, 2 + len(SEQ))), indices_hit=list(range(len(SEQ))))
    late = parsers.TemplateHit(index=2, name="2xyz_A too new", aligned_cols=len(SEQ), sum_probs=20.0, query=SEQ, hit_sequence=SEQ,
                               indices_query=list(range(2, 2 + len(SEQ))), indices_hit=list(range(len(SEQ))))
    # indices_query are positions in the query as an HHR file gives them; a hit whose indices are relative to the aligned
    # fragment (the fragment is located inside the full query) maps to the same residues
    relative = parsers.TemplateHit(**{**hit.__dict__, "indices_query": list(range(len(SEQ)))})
    f = templates.TemplateHitFeaturizer(mmcif_dir=str(tmp_path), max_template_date="2020-01-01", max_hits=4, _zero_center_positions=False)
    assert np.array_equal(f.get_templates(query, [relative]).features["template_all_atom_mask"], f.get_templates(query, [hit]).features["template_all_atom_mask"])
    res = f.get_templates(query, [hit, late])
    feats = res.features
    assert feats["template_aatype"].shape == (1, len(query), 22)
    assert feats["template_all_atom_positions"].shape == (1, len(query), 37, 3)
    assert feats["template_domain_names"][0] == b"1abc_A"
    ca = rc.atom_order["CA"]
    assert feats["template_all_atom_mask"][0, 2, ca] == 1 and feats["template_all_atom_mask"][0, 0, ca] == 0
    assert feats["template_all_atom_mask"][0, 2 + 3].sum() == 0                         # the residue without coordinates
    assert np.allclose(feats["template_all_atom_positions"][0, 2 + 2, ca], [3.8 * 2 + 0.1, 2.0, -1.5], atol=1e-3)
    assert feats["template_sequence"][0].decode() == "--" + SEQ + "--"
    assert abs(feats["template_sum_probs"][0, 0] - 12.0) < 1e-6
    # training on PDB entries: the query's own entry is never its template, and the date cutoff follows the query
    assert f.get_templates(query, hits=[hit, late], query_pdb_code="1ABC").features["template_aatype"].shape[0] == 0
    assert f.get_templates(query, "1999-06-01", [hit, late]).features["template_aatype"].shape[0] == 0    # 60-day margin
    assert f.get_templates(query, hits=[hit, late], query_release_date="1999-09-01").features["template_aatype"].shape[0] == 1
    assert f.get_templates(query, [hit, late]).features["template_aatype"].shape[0] == 1                                        # cutoff restored
    from fastfold_b200.data.data_pipeline import make_template_features
    assert make_template_features(query, {"pdb70_hits.hhr": [hit, late]}, f, query_pdb_code="1abc")["template_aatype"].shape == (0, len(query), 22)


def test_prefilter_rules():
    q = "A" * 40
    mk = lambda seq, cols: parsers.TemplateHit(1, "1abc_A", cols, 1.0, seq, seq, list(range(len(seq))), list(range(len(seq))))
    with pytest.raises(templates.AlignRatioError):
        templates.assess_hit(mk("C" * 20, 3), "1abc", q, {}, None)
    with pytest.raises(templates.DuplicateError):
        templates.assess_hit(mk("A" * 39, 39), "1abc", q, {}, None)
    with pytest.raises(templates.LengthError):
        templates.assess_hit(mk("CDEFGHIK", 8), "1abc", q, {}, None)
    assert templates.assess_hit(mk("CDEFGHIKLMNP", 12), "1abc", q, {}, None)
