"""PDB clean-up before an OpenMM minimisation (fastfold/relax/cleanup.py:1-127): pdbfixer adds the missing heavy
atoms and hydrogens, non-standard residues are replaced, heterogens removed.  Needs ``pdbfixer``; the violation back
end of ``amber_minimize`` does not use this module."""
import io


def fix_pdb_string(pdb_str: str, alterations_info=None) -> str:
    try:
        import pdbfixer
        from openmm import app
    except ImportError as e:
        raise ImportError("PDB clean-up for the OpenMM back end needs pdbfixer and openmm: %s" % e)
    fixer = pdbfixer.PDBFixer(pdbfile=io.StringIO(pdb_str))
    fixer.findNonstandardResidues()
    if alterations_info is not None:
        alterations_info["nonstandard_residues"] = fixer.nonstandardResidues
    fixer.replaceNonstandardResidues()
    fixer.removeHeterogens(keepWater=False)
    fixer.findMissingResidues()
    fixer.findMissingAtoms()
    if alterations_info is not None:
        alterations_info["missing_heavy_atoms"] = fixer.missingAtoms
        alterations_info["missing_terminals"] = fixer.missingTerminals
    fixer.addMissingAtoms(seed=0)
    fixer.addMissingHydrogens()
    out = io.StringIO()
    app.PDBFile.writeFile(fixer.topology, fixer.positions, out, keepIds=True)
    return out.getvalue()


def fix_pdb(pdbfile, alterations_info) -> str:
    """``fix_pdb_string`` for an open file handle (the reference's calling convention)."""
    return fix_pdb_string(pdbfile.read(), alterations_info)


def clean_structure(pdb_structure, alterations_info):
    """Edge cases pdbfixer leaves behind, on an OpenMM ``PdbStructure`` in place: selenomethionine's SE atom becomes
    the SD of a methionine, and chains of a single residue (which the force field cannot terminate) are dropped."""
    changed = []
    for res in pdb_structure.iter_residues():
        if res.get_name_with_spaces().strip() == "MET":
            se = getattr(res, "get_atom", lambda n: None)("SE") if hasattr(res, "get_atom") else None
            if se is not None:
                se.name = "SD"
                se.element_symbol = "S"
                changed.append(res.number)
    alterations_info["Se_in_MET"] = changed
    removed = {}
    for model in pdb_structure.iter_models():
        keep = [c for c in model.iter_chains() if len(c) > 1]
        dropped = [c.chain_id for c in model.iter_chains() if len(c) <= 1]
        model.chains = keep
        model.chains_by_id = {c.chain_id: c for c in keep} if hasattr(model, "chains_by_id") else None
        removed[model.number] = dropped
    alterations_info["removed_chains"] = removed

