"""Stand-in for ``Bio.Data.SCOPData``: one-letter codes of the residue names that occur in protein chains (the twenty
standard amino acids, selenomethionine / selenocysteine / pyrrolysine and a few frequent modified residues).  BioPython's
table is longer; names missing here are read as ``X`` by the code that uses the table."""
protein_letters_3to1 = {
    "ALA": "A", "ARG": "R", "ASN": "N", "ASP": "D", "CYS": "C", "GLN": "Q", "GLU": "E", "GLY": "G", "HIS": "H", "ILE": "I",
    "LEU": "L", "LYS": "K", "MET": "M", "PHE": "F", "PRO": "P", "SER": "S", "THR": "T", "TRP": "W", "TYR": "Y", "VAL": "V",
    "MSE": "M", "SEC": "U", "PYL": "O", "SEP": "S", "TPO": "T", "PTR": "Y", "HYP": "P", "MLY": "K", "CSO": "C", "UNK": "X",
}
