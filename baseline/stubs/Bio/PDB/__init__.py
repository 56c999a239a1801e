"""Stand-in for ``Bio.PDB`` (BioPython is not installed).  ``PDBParser`` only satisfies an import of the reference package;
``MMCIFParser`` reads an mmCIF file into the tag dictionary and the structure hierarchy that the reference's
``fastfold/data/mmcif_parsing.py`` consumes.  It shares no code with the package under test: its tokenizer and structure
builder are written here, so that the reference stays an independent oracle for the mmCIF and template code."""
import numpy as np

from . import Structure  # noqa: F401  (accessed as Bio.PDB.Structure.Structure)
from .Structure import Atom, Structure as _Structure


class PDBParser:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("BioPython is not installed; this stand-in only satisfies the import")


def _tokens(text):
    """mmCIF tokens: bare words, quoted strings (a quote ends only before white space), and text fields that open and
    close with a semicolon in the first column; ``#`` starts a comment outside of these."""
    lines = text.splitlines()
    i = 0
    while i < len(lines):
        line = lines[i]
        if line.startswith(";"):
            parts = [line[1:]]
            i += 1
            while i < len(lines) and not lines[i].startswith(";"):
                parts.append(lines[i])
                i += 1
            yield ("value", "\n".join(parts).rstrip("\n") if len(parts) > 1 else parts[0])
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
                    if end < 0:
                        raise ValueError("unterminated quote: %r" % line)
                    if end + 1 >= n or line[end + 1] in " \t":
                        break
                    end += 1
                yield ("value", line[pos + 1:end])
                pos = end + 1
            else:
                end = pos
                while end < n and line[end] not in " \t":
                    end += 1
                yield ("word", line[pos:end])
                pos = end
        i += 1


def _mmcif_to_dict(text):
    """``{tag: value or [values]}`` as BioPython's ``MMCIF2Dict``: looped tags map to lists, single items to strings."""
    out, toks = {}, list(_tokens(text))
    i = 0
    while i < len(toks):
        kind, tok = toks[i]
        if kind == "word" and tok.lower().startswith("data_"):
            out["data_"] = tok[5:]
            i += 1
        elif kind == "word" and tok.lower() == "loop_":
            i += 1
            tags = []
            while i < len(toks) and toks[i][0] == "word" and toks[i][1].startswith("_"):
                tags.append(toks[i][1])
                i += 1
            for t in tags:
                out[t] = []
            col = 0
            while i < len(toks) and not (toks[i][0] == "word" and (toks[i][1].startswith("_") or toks[i][1].lower() in ("loop_",) or
                                                                   toks[i][1].lower().startswith("data_"))):
                out[tags[col % len(tags)]].append(toks[i][1])
                col += 1
                i += 1
        elif kind == "word" and tok.startswith("_"):
            out[tok] = toks[i + 1][1]
            i += 2
        else:
            i += 1
    return out


class MMCIFParser:
    def __init__(self, QUIET=False, **kwargs):
        self._mmcif_dict = None

    def get_structure(self, structure_id, handle):
        d = self._mmcif_dict = _mmcif_to_dict(handle.read())

        def column(tag, default=None):
            v = d.get(tag)
            if v is None:
                return default
            return v if isinstance(v, list) else [v]
        names = column("_atom_site.label_atom_id")
        n = len(names)
        group, resname = column("_atom_site.group_PDB"), column("_atom_site.label_comp_id")
        chain_ids = column("_atom_site.auth_asym_id") or column("_atom_site.label_asym_id")
        seq_ids = column("_atom_site.auth_seq_id") or column("_atom_site.label_seq_id")
        icodes = column("_atom_site.pdbx_PDB_ins_code", ["?"] * n)
        models = column("_atom_site.pdbx_PDB_model_num", ["1"] * n)
        occupancy = column("_atom_site.occupancy", ["1.0"] * n)
        elements = column("_atom_site.type_symbol", ["?"] * n)
        xs, ys, zs = column("_atom_site.Cartn_x"), column("_atom_site.Cartn_y"), column("_atom_site.Cartn_z")
        structure = _Structure(structure_id)
        for k in range(n):
            if group[k] == "HETATM":
                hetflag = "W" if resname[k] in ("HOH", "WAT") else "H_" + resname[k]
            else:
                hetflag = " "
            icode = " " if icodes[k] in ("?", ".") else icodes[k]
            chain = structure.model(int(models[k]) - 1).chain(chain_ids[k])
            residue = chain.residue((hetflag, int(seq_ids[k]), icode), resname[k])
            residue.add(Atom(names[k], np.array([float(xs[k]), float(ys[k]), float(zs[k])], dtype=np.float32), float(occupancy[k]), elements[k]))
        return structure
