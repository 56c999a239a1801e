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
